"""Causal prompt attention over Q8_0 K/V (sdx_qsa_prompt) against the oracle: the mma.sync kernel (SDX_PROMPT_KERNEL=mma);
the default tcgen05 kernel runs the same cases in test_gpu_y_prompt_tcgen05.py."""
import numpy as np
import pytest

import oracle
from util import close, q8_state, q8_value_bound, queries_f16

pytestmark = pytest.mark.gpu
GUARD, CANARY = 8, np.float32(12345.125)


@pytest.fixture(autouse=True)
def use_mma_sync(monkeypatch):
    monkeypatch.setenv("SDX_PROMPT_KERNEL", "mma")


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
                                                       (100, 33, 8, 2), (30, 50, 4, 2), (7, 130, 2, 2), (200, 70, 8, 1)])
def test_small_chunks_every_row(gpu, first, rows, heads, kv_heads):
    rng = np.random.default_rng(first * 131 + rows)
    context = first + rows + 3
    state = q8_state(rng, context, kv_heads)
    q = queries_f16(rng, rows, heads, 256)
    got = run_prompt(gpu, state, context, first, rows, heads, kv_heads, q)
    want = oracle.gqa_prompt_q8(state, context, first, heads, kv_heads, q, 1 / 16, f64=True)
    # K and V enter the tensor cores rounded to FP16 (as in the reference's own kernel): rows of a few keys whose large values
    # cancel are held to 1e-3 of the largest value instead of to the sum's own size
    ok, worst = close(got, want, value_bound=q8_value_bound(state))
    assert ok, worst


def test_chunk_after_cache_sampled_rows(gpu):
    # config 2's layout at a quarter of its size: 2048 new tokens after 2048 cached; the oracle checks sampled rows
    rng = np.random.default_rng(77)
    first, rows, context = 2048, 2048, 4096
    state = q8_state(rng, context, 2)
    q = queries_f16(rng, rows, 16, 256)
    got = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    sample = [0, 1, 15, 16, 63, 64, 1000, 2047]
    want = oracle.gqa_prompt_q8(state, context, first, 16, 2, q, 1 / 16, rows=sample, f64=True)
    for r in sample:
        ok, worst = close(got[r], want[r])
        assert ok, (r, worst)
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
    for first, rows, heads, kv_heads in [(60, 5, 16, 2), (0, 0, 16, 2), (0, 4, 24, 2), (0, 4, 16, 3)]:
        with pytest.raises(StraydogError):
            gpu.qsa_prompt(state, 64, first, rows, heads, kv_heads, 1 / 16, q.pointer, out.pointer)
    for b in (state, q, out):
        gpu.release(b)
