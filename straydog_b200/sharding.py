"""Host-side logic of running the attention path on N GPUs of one node.

GQA decode: which sequences a rank owns and how the ranks' timings and byte counts become one whole-job number. Sequences are
independent, so that data path has no collective; torch.distributed carries only the barrier and two small reductions.
Latent sparse attention: the heads are dealt over the ranks (the latent rows are shared by all heads, so every rank holds the
cache); a rank's outputs [rows][heads / N][dim] are all-gathered into [N][rows][heads / N][dim] (NCCL on GPUs, gloo in the CPU tests)."""
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


def head_range(heads, rank, world):
    """(first head, head count) of `rank` when `heads` are dealt evenly over `world` ranks (heads % world == 0)."""
    if heads % world:
        raise ValueError(f"{heads} heads do not divide over {world} ranks")
    each = heads // world
    return rank * each, each


def gather_heads(shard):
    """All-gather of a rank's outputs [rows][heads / N][dim] -> [N][rows][heads / N][dim] (rank-major, what NCCL delivers without a
    transpose; the consumer's contraction runs over (rank, head, dim) in that order). Runs on the current stream."""
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    full = torch.empty((world,) + tuple(shard.shape), dtype=shard.dtype, device=shard.device)
    if world == 1:
        full[0].copy_(shard)
    else:
        dist.all_gather_into_tensor(full.view(-1), shard.reshape(-1))
    return full


def heads_from_gathered(full):
    """[N][rows][heads / N][dim] -> [rows][heads][dim] (a view-changing copy, for checks)."""
    world, rows, each, dim = full.shape
    return full.permute(1, 0, 2, 3).reshape(rows, world * each, dim)


def gathered_buffer_of(step):
    """Which of a rank's TWO gathered buffers call number `step` of sdx_sparse_attention_gather stores into (steps count from 1).

    A rank leaves call n only when every peer's counter shows n, i.e. when every peer has finished the attention kernel of its own
    call n; a peer's stream runs that kernel behind its readers of call n - 1. So while a rank stores call n + 1 into buffer
    (n + 1) % 2 a slow peer may still read buffer n % 2 (call n), and nothing of call n - 1 is read any more anywhere."""
    return step % 2
