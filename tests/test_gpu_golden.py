"""This library's kernels against outputs of the reference's own GPU library (tests/golden/reference_b200.npz)."""
import os

import numpy as np
import pytest

from util import XorShift, attention_sequence_input, close, latent_decode_case, op_attention_case, q8_state, sparse_attention_case, tie_scores
from test_gpu_sparse import run as run_sparse

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz"))


@pytest.mark.parametrize("steps,selected,base,context,kind", [(4, 2052, 3000, 4096, "sparse"), (3, 64, 100, 256, "dense"), (8, 513, 20, 64, "sparse")])
def test_attention_sequence(gpu, steps, selected, base, context, kind):
    rng = np.random.default_rng(steps * 1000 + selected)
    state_np = q8_state(rng, context, 2, filled=base)
    inp = attention_sequence_input(rng, steps, selected, base, context, kind)
    state = gpu.allocate(state_np.nbytes)
    gpu.write(state, state_np)
    got = gpu.attention_sequence(state, context, base, steps, selected, inp)
    after = gpu.download(state, np.empty_like(state_np))
    key = f"sequence_{steps}_{selected}_{base}_{context}_{kind}"
    assert np.array_equal(after[:, base:base + steps], GOLDEN[key + "_rows"])
    ok, worst = close(got, GOLDEN[key], atol=1e-4, rtol=1e-3)
    assert ok, worst
    gpu.release(state)


@pytest.mark.parametrize("rows,heads,kv_heads,dim,context", [(15, 16, 2, 256, 137), (1, 2, 1, 256, 137), (17, 4, 2, 256, 35), (16, 4, 2, 128, 35)])
def test_op_attention(gpu, rows, heads, kv_heads, dim, context):
    c = op_attention_case(rows, heads, kv_heads, dim, context)
    qs, ks, vs, gs, ps = (gpu.upload(c[k]) for k in ("q", "keys", "values", "gate", "positions"))
    scratch = gpu.buffer(rows * heads * 64 * (dim + 2) * 4)
    out = gpu.buffer(c["q"].size * 4)
    for gated in (0, 1):
        gpu.attention(qs.pointer, ks.pointer, vs.pointer, context, ps.pointer, rows, heads, kv_heads, dim, c["scale"],
                      gs.pointer if gated else None, scratch, out.pointer)
        got = gpu.read(out, np.float32, (rows, heads, dim))
        ok, worst = close(got, GOLDEN[f"attention_{rows}_{heads}_{kv_heads}_{dim}_{context}_{gated}"], atol=1e-5, rtol=1e-4)
        assert ok, worst
    for b in (qs, ks, vs, gs, ps, scratch, out):
        gpu.release(b)


@pytest.mark.parametrize("rows,heads", [(1, 32), (4, 32)])
def test_sparse_attention(gpu, rows, heads):
    c = sparse_attention_case(rows, heads)
    got = run_sparse(gpu, c, c["halves"], tagged=True)
    ok, worst = close(got, GOLDEN[f"sparse_{rows}_{heads}"])
    assert ok, worst


def test_latent_decode_shape(gpu):
    seed, rows, heads, dim, context, selections = 11, 2, 16, 576, 1024, 256
    c = latent_decode_case(seed, rows, heads, dim, context, selections)
    got = run_sparse(gpu, c, c["halves"], tagged=True)
    ok, worst = close(got, GOLDEN[f"latent_{seed}_{rows}_{heads}_{dim}_{context}_{selections}"])
    assert ok, worst


def test_top_k_bit_for_bit(gpu):
    random = XorShift(0x2F6B91D3C0A54E77)
    for groups in [511, 512, 513, 600, 4096, 30000]:
        scores = tie_scores(random, 2, groups)
        dev = gpu.upload(scores)
        out = gpu.buffer(2 * 512 * 4)
        gpu.top_k(dev.pointer, 2, groups, 512, out.pointer)
        assert np.array_equal(gpu.read(out, np.int32, (2, 512)), GOLDEN[f"topk_{groups}"]), groups
        gpu.release(dev)
        gpu.release(out)
