"""sd_op_top_k against the reference's rule on its own tie-heavy cases (tests/fused_gpu.rs:359-389); sd_op_to_bf16."""
import numpy as np
import pytest

import oracle
from util import XorShift, bf16_round, tie_scores

pytestmark = pytest.mark.gpu


def test_top_k_matches_its_reference_with_many_ties(gpu):
    random = XorShift(0x2F6B91D3C0A54E77)
    k = 512
    for groups in [511, 512, 513, 600, 4096, 30000, 65536, 131072]:
        scores = tie_scores(random, 2, groups)
        dev = gpu.upload(scores)
        out = gpu.buffer(2 * k * 4)
        gpu.top_k(dev.pointer, 2, groups, k, out.pointer)
        got = gpu.read(out, np.int32, (2, k))
        want = oracle.top_k(scores, k)
        assert np.array_equal(got, want), groups
        gpu.release(dev)
        gpu.release(out)


@pytest.mark.parametrize("rows,groups,k", [(1, 1, 1), (3, 10, 16), (32, 65536, 2048), (5, 2049, 2048), (2, 100000, 1)])
def test_top_k_random_scores(gpu, rows, groups, k):
    rng = np.random.default_rng(rows * 7 + groups)
    scores = rng.normal(0, 1, (rows, groups)).astype(np.float32)
    scores[:, ::5] = np.round(scores[:, ::5], 1)     # ties
    dev = gpu.upload(scores)
    out = gpu.buffer(rows * k * 4)
    gpu.top_k(dev.pointer, rows, groups, k, out.pointer)
    assert np.array_equal(gpu.read(out, np.int32, (rows, k)), oracle.top_k(scores, k))
    gpu.release(dev)
    gpu.release(out)


def check(gpu, scores, k):
    rows, groups = scores.shape
    dev = gpu.upload(scores)
    out = gpu.buffer(rows * k * 4)
    gpu.top_k(dev.pointer, rows, groups, k, out.pointer)
    got = gpu.read(out, np.int32, (rows, k))
    gpu.release(dev)
    gpu.release(out)
    assert np.array_equal(got, oracle.top_k(scores, k))


@pytest.mark.parametrize("rows,groups,k", [(1, 65536, 2048), (4, 65536, 512), (20, 32768, 2048), (20, 16384, 2048), (50, 8192, 100), (3, 16387, 4096)])
def test_a_row_shared_by_several_blocks(gpu, rows, groups, k):
    """Few rows: a row's slices go to a cluster of 8, 4 or 2 blocks. The k-th score's equals are spread over the slices."""
    rng = np.random.default_rng(groups + rows)
    scores = rng.normal(0, 1, (rows, groups)).astype(np.float32)
    above = int((scores[0] > 2.0).sum())
    if above < k:
        ties = rng.choice(groups, size=min(groups // 4, 3000), replace=False)
        scores[:, ties] = 2.0
    check(gpu, scores, k)


def test_rows_that_leave_the_shared_lists_in_a_cluster(gpu):
    """Equal scores everywhere (a band of the whole row), k above the shared lists' room, fewer live scores than k."""
    check(gpu, np.zeros((2, 65536), np.float32), 1000)
    rng = np.random.default_rng(5)
    check(gpu, rng.normal(0, 1, (2, 65536)).astype(np.float32), 5000)
    sparse = np.full((2, 40000), -np.inf, np.float32)
    sparse[:, rng.choice(40000, size=100, replace=False)] = rng.normal(0, 1, 100).astype(np.float32)
    check(gpu, sparse, 3000)
    few = rng.integers(0, 3, (3, 50000)).astype(np.float32)     # three values: the band is a third of the row
    check(gpu, few, 2048)


def test_slices_of_more_than_a_million_scores_keep_the_matching_count(gpu):
    """A block's slice over 2^20 - 1024 scores no longer fits the first read's 16-bit private counts: it counts with the warp-wide match
    instead. One row of nine million scores (eight blocks of 1 125 000), with ties at the k-th score; and a row that is one block's
    (many rows) at 1 100 000."""
    rng = np.random.default_rng(11)
    scores = rng.normal(0, 1, (1, 9_000_000)).astype(np.float32)
    scores[0, rng.choice(9_000_000, size=5000, replace=False)] = 4.25
    check(gpu, scores, 3000)
    scores = rng.normal(0, 1, (80, 1_100_000)).astype(np.float32)
    check(gpu, scores, 64)


def test_rounding_into_bf16_is_to_the_nearest_even(gpu):
    # tests/ds_state_bf16_gpu.rs:50-69
    values = XorShift(0x243F6A8885A308D3).floats_scaled(10_000, 1e3)
    extra = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 3.4028235e38, 1.17549435e-38, 1 + 1 / 256, 1 + 3 / 256], np.float32)
    values = np.concatenate([values, extra, np.array([0x3F808000, 0x3F818000], np.uint32).view(np.float32)])
    dev = gpu.upload(values)
    out = gpu.buffer(values.size * 2)
    gpu.to_bf16(dev.pointer, values.size, out.pointer)
    got = gpu.read(out, np.uint16, (values.size,))
    want, _ = bf16_round(values)
    nan = np.isnan(values)
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all(np.isnan((got[nan].astype(np.uint32) << 16).view(np.float32)))
    gpu.release(dev)
    gpu.release(out)
