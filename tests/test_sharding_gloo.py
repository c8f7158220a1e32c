"""The N > 1 host logic on CPU: two gloo ranks shard the batch and reduce their timings as bench.py does on GPUs."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from straydog_b200 import sharding
from straydog_b200.synthetic import ragged_lengths

SEED = 1234


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    strong, _ = sharding.rank_batch(SEED, rank, world, "strong")
    weak, _ = sharding.rank_batch(SEED, rank, world, "weak")
    times, sums = sharding.whole_job([10.0 + rank, 3.0 - rank], [float(sum(strong)), float(len(strong)), float(sum(weak))])
    results[rank] = (strong, weak, times, sums)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_and_reduce():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
    everything = ragged_lengths(SEED)
    strong = [results[r][0] for r in range(world)]
    assert sorted(strong[0] + strong[1]) == sorted(everything), "the strong shards cover the batch once"
    loads = [sum(s) for s in strong]
    assert abs(loads[0] - loads[1]) <= max(everything), "longest-first packing balances to within one sequence"
    for r in range(world):
        _, weak, times, sums = results[r]
        assert len(weak) == 64 and weak == ragged_lengths(SEED)
        assert times == [11.0, 3.0], "max over ranks"
        assert sums[0] == float(sum(everything)) and sums[1] == 64.0
        assert sums[2] == 2.0 * float(sum(ragged_lengths(SEED)))


def test_partition_edge_cases():
    from straydog_b200.synthetic import partition_longest_first
    assert partition_longest_first([5], 4) == [[0], [], [], []]
    parts = partition_longest_first([1, 1, 1, 1, 10], 2)
    assert sorted(parts[0] + parts[1]) == [0, 1, 2, 3, 4] and [4] in parts
    single, _ = sharding.rank_batch(SEED, 0, 1, "strong")
    assert single == ragged_lengths(SEED)


def head_worker(rank, world, port, results):
    import numpy as np
    import oracle
    from util import sparse_attention_case
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    c = sparse_attention_case(2, 8)
    c["q"] = c["q"].reshape(c["rows"], c["heads"], c["dim"])
    first, each = sharding.head_range(c["heads"], rank, world)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(c["dim"])))
    mine = oracle.sparse_attention(np.ascontiguousarray(c["q"][:, first:first + each]), c["raw"], c["raw_rows"], c["positions"], c["window"], c["halves"],
                                   c["selected"], c["selections"], c["sinks"][first:first + each], c["rows"], each, c["dim"], scale,
                                   c["rope_dims"], c["freq"])
    full = sharding.gather_heads(torch.from_numpy(mine))
    results[rank] = sharding.heads_from_gathered(full).numpy()
    dist.barrier()
    dist.destroy_process_group()


def test_head_shards_gather_to_the_unsharded_result():
    """Heads are independent in the latent attention: a rank's slice of q and sinks gives that slice of the output bit for bit, and
    the all-gather (rank-major) rearranges to the unsharded [rows][heads][dim]."""
    import numpy as np
    import oracle
    from util import sparse_attention_case
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(head_worker, args=(world, free_port(), results), nprocs=world, join=True)
    c = sparse_attention_case(2, 8)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(c["dim"])))
    whole = oracle.sparse_attention(c["q"], c["raw"], c["raw_rows"], c["positions"], c["window"], c["halves"], c["selected"],
                                    c["selections"], c["sinks"], c["rows"], c["heads"], c["dim"], scale, c["rope_dims"], c["freq"])
    for r in range(world):
        assert np.array_equal(results[r].view(np.uint32), whole.view(np.uint32))
    with __import__("pytest").raises(ValueError):
        sharding.head_range(10, 0, 4)


def test_two_gathered_buffers_are_enough_and_one_is_not():
    """sdx_sparse_attention_gather's buffer rule, as a schedule on CPU: every rank runs, per call n, [kernel: store its slot of call n
    into every rank's gathered buffer, raise its counters to n, wait until its own counters all show n] and then [consumer: read its
    own gathered buffer of call n], each rank's phases in stream order, the ranks interleaved at random. With two buffers taken in
    turn (sharding.gathered_buffer_of) a consumer always finds call n in every slot; with one buffer some interleaving lets a rank
    that is a call ahead overwrite what a slow peer has not read yet."""
    import random

    def run(world, calls, buffers, seed):
        random.seed(seed)
        store = [[[0] * world for _ in range(buffers)] for _ in range(world)]     # store[gpu][buffer][slot] = call whose data sits there
        counters = [[0] * world for _ in range(world)]                            # counters[gpu][peer]
        call, phase = [1] * world, ["store"] * world                              # store -> wait -> read
        while any(c <= calls for c in call):
            rank = random.choice([r for r in range(world) if call[r] <= calls])
            n = call[rank]
            which = sharding.gathered_buffer_of(n) if buffers == 2 else 0
            if phase[rank] == "store":
                for gpu in range(world):
                    store[gpu][which][rank] = n
                    counters[gpu][rank] = n
                phase[rank] = "wait"
            elif phase[rank] == "wait":
                if all(seen >= n for seen in counters[rank]):
                    phase[rank] = "read"
            else:
                if any(slot != n for slot in store[rank][which]):
                    return False
                call[rank], phase[rank] = n + 1, "store"
        return True

    assert all(run(world, 40, 2, seed) for world in (2, 4, 8) for seed in range(30))
    assert not all(run(4, 40, 1, seed) for seed in range(30))
