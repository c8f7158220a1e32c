"""Host-side logic of running the decode path on N GPUs of one node: which sequences a rank owns and how the ranks'
timings and byte counts become one whole-job number. Sequences are independent, so the data path has no collective;
torch.distributed carries only the barrier and two small reductions (NCCL on GPUs, gloo in the CPU tests)."""
import torch
import torch.distributed as dist

from .synthetic import partition_longest_first, ragged_lengths


def rank_batch(seed, rank, world, scaling, sequences=64):
    """(lengths, seeds) of the sequences `rank` decodes.

    weak: every rank has a batch of `sequences` with the same seeded lengths and its own seeded contents
    (per-GPU work fixed as N grows).
    strong: one batch of `sequences` dealt over the ranks, longest first, by K/V bytes."""
    if scaling == "weak":
        lengths = ragged_lengths(seed, sequences)
        return lengths, [seed * 1000 + rank * 100 + i for i in range(len(lengths))]
    if scaling != "strong":
        raise ValueError(f"unknown scaling {scaling!r}")
    lengths = ragged_lengths(seed, sequences)
    mine = partition_longest_first(lengths, world)[rank]
    return [lengths[i] for i in mine], [seed * 1000 + i for i in mine]


def whole_job(times_ms, sums, device=None):
    """Max over ranks of each entry of times_ms, sum over ranks of each entry of sums (lists of floats)."""
    t = torch.tensor(list(times_ms), dtype=torch.float64, device=device)
    s = torch.tensor(list(sums), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(s, op=dist.ReduceOp.SUM)
    return [float(x) for x in t.cpu()], [float(x) for x in s.cpu()]
