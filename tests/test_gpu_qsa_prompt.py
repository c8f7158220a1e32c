"""Causal prompt attention over Q8_0 K/V (sdx_qsa_prompt, the tcgen05/TMEM kernel) against the oracle.

K and V enter the tensor cores as FP16 hi + lo planes (their exact values), so only the softmax weights are rounded to FP16 (2^-12
of each weight, which a row of a few keys with values near 10 shows as about 1e-3): every output is held to the benchmark's
tolerance, max-abs 2e-3 or max-rel 1e-2 per element, with no allowance for the size of the values."""
import numpy as np
import pytest

import oracle
from util import close, q8_state, queries_f16

pytestmark = pytest.mark.gpu
GUARD, CANARY = 8, np.float32(12345.125)


def run_prompt(gpu, state_np, context, first, rows, heads, kv_heads, q, scale=1 / 16):
    state = gpu.upload(state_np)
    q_dev = gpu.upload(q)
    out = gpu.upload(np.full(rows * heads * 256 + 2 * GUARD, CANARY, np.float32))
    gpu.qsa_prompt(state, context, first, rows, heads, kv_heads, scale, q_dev.pointer, out.at(GUARD * 4))
    got = gpu.read(out, np.float32, (rows * heads * 256 + 2 * GUARD,))
    assert gpu.decode_status() == 0
    assert np.all(got[:GUARD] == CANARY) and np.all(got[-GUARD:] == CANARY), "output guard"
    for b in (state, q_dev, out):
        gpu.release(b)
    return got[GUARD:-GUARD].reshape(rows, heads, 256)


@pytest.mark.parametrize("first,rows,heads,kv_heads", [(0, 1, 16, 2), (0, 16, 16, 2), (0, 17, 16, 2), (5, 40, 16, 2), (63, 2, 16, 2), (64, 64, 16, 2),
                                                       (100, 33, 8, 2), (30, 50, 4, 2), (7, 130, 2, 2), (200, 70, 8, 1), (1000, 300, 16, 2),
                                                       # groups that do not divide a block's 128 rows (the reference's own 24 / 2 and 12 / 1), and one of 16
                                                       (37, 45, 24, 2), (0, 21, 12, 1), (10, 30, 6, 2), (50, 20, 16, 1), (3, 26, 10, 2), (500, 64, 24, 2)])
def test_small_chunks_every_row(gpu, first, rows, heads, kv_heads):
    rng = np.random.default_rng(first * 131 + rows)
    context = first + rows + 3
    state = q8_state(rng, context, kv_heads)
    q = queries_f16(rng, rows, heads, 256)
    got = run_prompt(gpu, state, context, first, rows, heads, kv_heads, q)
    want = oracle.gqa_prompt_q8(state, context, first, heads, kv_heads, q, 1 / 16, f64=True)
    ok, worst = close(got, want)
    assert ok, worst


def test_the_chunk_may_end_at_a_context_that_is_no_multiple_of_the_tile(gpu):
    # the last tile of every plane is partly past the context: those positions must read as zeros, not as the next plane's rows
    rng = np.random.default_rng(9)
    first, rows, context = 70, 31, 101
    state = q8_state(rng, context, 2)
    q = queries_f16(rng, rows, 16, 256)
    got = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    want = oracle.gqa_prompt_q8(state, context, first, 16, 2, q, 1 / 16, f64=True)
    ok, worst = close(got, want)
    assert ok, worst


def test_peaked_rows_force_rescaling(gpu):
    # keys whose scores rise steeply along the context: the running maximum grows by far more than 2^8 from tile to tile, and scores
    # of several hundred make any rounding of the keys visible (values up to 33 here)
    rng = np.random.default_rng(5)
    context, first, rows = 600, 200, 64
    state = q8_state(rng, context, 2)
    ramp = (np.arange(context, dtype=np.float32) / context * 0.25 + 0.01).astype(np.float16)
    state[:2, :, 256:] = np.repeat(ramp[None, :, None], 8, axis=2).view(np.uint8).reshape(1, context, 16)
    q = np.abs(queries_f16(rng, rows, 16, 256))
    state[:2, :, :256] = np.abs(state[:2, :, :256].view(np.int8)).view(np.uint8)      # positive keys x positive queries: monotone scores
    got = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    want = oracle.gqa_prompt_q8(state, context, first, 16, 2, q, 1 / 16, f64=True)
    ok, worst = close(got, want)
    assert ok, worst


@pytest.mark.parametrize("first,rows", [(2048, 2048), (8192, 8192)])
def test_chunk_after_cache_sampled_rows(gpu, first, rows):
    # the benchmark's prompt configuration (8192 new tokens after 8192 cached) and a quarter of it; the oracle checks sampled rows
    rng = np.random.default_rng(77 + first)
    context = first + rows
    state = q8_state(rng, context, 2)
    q = queries_f16(rng, rows, 16, 256)
    got = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    sample = [0, 1, 15, 16, 63, 64, 1000, rows // 2 + 5, rows - 17, rows - 1]
    want = oracle.gqa_prompt_q8(state, context, first, 16, 2, q, 1 / 16, rows=sample, f64=True)
    for r in sample:
        ok, worst = close(got[r], want[r])
        assert ok and worst < 1e-3, (r, worst)   # (thousands of keys a row: the weights' rounding averages out)
    assert np.all(np.isfinite(got))


def test_prompt_row_equals_decode_of_the_same_position(gpu):
    # a prompt row and a one-token decode of the same query over the same prefix agree within the tolerance
    rng = np.random.default_rng(78)
    first, rows, context = 300, 20, 400
    state = q8_state(rng, context, 2)
    q = queries_f16(rng, rows, 16, 256)
    got = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    dev_state, q_dev, out = gpu.upload(state), gpu.upload(q[7:8]), gpu.buffer(16 * 256 * 4)
    gpu.qsa_decode([dev_state], [context], [first + 8], 16, 2, 1 / 16, q_dev.pointer, out.pointer)
    decode = gpu.read(out, np.float32, (16, 256))
    ok, worst = close(got[7], decode)
    assert ok, worst
    for b in (dev_state, q_dev, out):
        gpu.release(b)


def test_invalid_chunks_are_refused(gpu):
    from straydog_b200.backend import StraydogError
    state = gpu.buffer(4 * 64 * 272)
    q = gpu.buffer(64 * 16 * 256 * 2)
    out = gpu.buffer(64 * 16 * 256 * 4)
    for first, rows, heads, kv_heads, scale in [(60, 5, 16, 2, 1 / 16), (0, 0, 16, 2, 1 / 16), (0, 4, 34, 2, 1 / 16), (0, 4, 16, 3, 1 / 16),
                                                (0, 4, 16, 2, 0.0), (0, 4, 16, 2, -1.0), (0, 4, 16, 2, float("nan"))]:
        with pytest.raises(StraydogError):
            gpu.qsa_prompt(state, 64, first, rows, heads, kv_heads, scale, q.pointer, out.pointer)
    for b in (state, q, out):
        gpu.release(b)
