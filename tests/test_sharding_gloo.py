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
