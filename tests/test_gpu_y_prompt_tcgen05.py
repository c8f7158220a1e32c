"""The tcgen05/TMEM prompt-attention kernel (the default of sdx_qsa_prompt) against the oracle and against the mma.sync kernel."""
import numpy as np
import pytest

import oracle
from test_gpu_qsa_prompt import run_prompt
from util import close, q8_state, q8_value_bound, queries_f16

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def use_tcgen05(monkeypatch):
    monkeypatch.delenv("SDX_PROMPT_KERNEL", raising=False)


@pytest.mark.parametrize("first,rows,heads,kv_heads", [(0, 16, 16, 2), (0, 1, 16, 2), (0, 17, 16, 2), (5, 40, 16, 2), (63, 2, 16, 2), (64, 64, 16, 2),
                                                       (100, 33, 8, 2), (30, 50, 4, 2), (7, 130, 2, 2), (200, 70, 8, 1), (1000, 300, 16, 2)])
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


def test_peaked_rows_force_rescaling(gpu, monkeypatch):
    # keys whose scores rise steeply along the context: the running maximum grows by far more than 2^8 from tile to tile
    rng = np.random.default_rng(5)
    context, first, rows = 600, 200, 64
    state = q8_state(rng, context, 2)
    ramp = (np.arange(context, dtype=np.float32) / context * 0.25 + 0.01).astype(np.float16)
    state[:2, :, 256:] = np.repeat(ramp[None, :, None], 8, axis=2).view(np.uint8).reshape(1, context, 16)
    q = np.abs(queries_f16(rng, rows, 16, 256))
    state[:2, :, :256] = np.abs(state[:2, :, :256].view(np.int8)).view(np.uint8)      # positive keys x positive queries: monotone scores
    got = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    want = oracle.gqa_prompt_q8(state, context, first, 16, 2, q, 1 / 16, f64=True)
    ok, worst = close(got, want, value_bound=q8_value_bound(state))   # values up to 33 here: FP16 operands carry 2^-11 of that
    assert ok, worst
    monkeypatch.setenv("SDX_PROMPT_KERNEL", "mma")
    mma = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    ok, worst = close(got, mma, value_bound=q8_value_bound(state))
    assert ok, worst


def test_agrees_with_the_mma_sync_kernel(gpu, monkeypatch):
    rng = np.random.default_rng(6)
    first, rows, context = 1024, 512, 1536
    state = q8_state(rng, context, 2)
    q = queries_f16(rng, rows, 16, 256)
    tc = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    monkeypatch.setenv("SDX_PROMPT_KERNEL", "mma")
    mma = run_prompt(gpu, state, context, first, rows, 16, 2, q)
    ok, worst = close(tc, mma, atol=5e-4, rtol=5e-3)
    assert ok, worst
