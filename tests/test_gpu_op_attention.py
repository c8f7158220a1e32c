"""sd_op_attention against the F64 softmax and per-output error bound of the reference's own test
(crates/straydog-engine/tests/attention_gpu.rs): the same shapes, seeds, positions, gate and canary guards."""
import numpy as np
import pytest

import oracle
from util import XorShift

pytestmark = pytest.mark.gpu
GUARD, CANARY = 7, np.float32(12345.125)

SHAPES = [(15, 4, 2, 256, 33), (16, 4, 2, 256, 33), (17, 4, 2, 256, 35), (31, 6, 2, 256, 65), (32, 4, 4, 256, 129),
          (16, 4, 2, 128, 35), (1, 2, 1, 256, 137), (17, 1, 1, 256, 1), (15, 16, 2, 256, 137)]


def check(gpu, rows, heads, kv_heads, dim, context, zero_queries):
    random = XorShift(0x9E3779B97F4A7C15 ^ rows ^ (dim << 16))
    q = random.floats_unit(rows * heads * dim)
    if zero_queries:
        q[:] = 0
    keys = random.floats_unit(context * kv_heads * dim)
    values = random.floats_unit(context * kv_heads * dim)
    special = [0, 1, 15, 16, context - 1, context + 7]
    positions = np.array([special[r] if r < len(special) else (r * 17 + 3) % context for r in range(rows)], np.int32)
    gate = np.array([[-12.0, -1.0, 0.0, 1.0, 12.0][i % 5] for i in range(q.size)], np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    qs, ks, vs, gs, ps = (gpu.upload(a) for a in (q, keys, values, gate, positions))
    scratch = gpu.buffer(rows * heads * 64 * (dim + 2) * 4)
    output = gpu.upload(np.full(q.size + 2 * GUARD, CANARY, np.float32))
    for gated in (False, True):
        gpu.attention(qs.pointer, ks.pointer, vs.pointer, context, ps.pointer, rows, heads, kv_heads, dim, scale,
                      gs.pointer if gated else None, scratch, output.at(GUARD * 4))
        actual = gpu.read(output, np.float32, (q.size + 2 * GUARD,))
        assert np.all(actual[:GUARD] == CANARY) and np.all(actual[GUARD + q.size:] == CANARY), "output guard"
        _, want, bound = oracle.op_attention(q, keys, values, context, positions, rows, heads, kv_heads, dim, scale,
                                             gate if gated else None, want64=True)
        got = actual[GUARD:GUARD + q.size].astype(np.float64)
        error = np.abs(got - want.ravel())
        assert np.all(np.isfinite(got)) and np.all(error <= bound.ravel()), (rows, heads, dim, context, gated, float((error / bound.ravel()).max()))
    for b in (qs, ks, vs, gs, ps, scratch, output):
        gpu.release(b)


@pytest.mark.parametrize("shape", SHAPES)
def test_causal_gqa_prefill_and_split_match_f64_softmax(gpu, shape):
    check(gpu, *shape, zero_queries=False)


def test_zero_queries(gpu):
    check(gpu, 17, 4, 2, 256, 35, zero_queries=True)


def test_shapes_and_scratch_are_checked(gpu):
    from straydog_b200.backend import StraydogError
    b = gpu.buffer(1 << 20)
    p = gpu.buffer(64)
    with pytest.raises(StraydogError):
        gpu.attention(b.pointer, b.pointer, b.pointer, 16, p.pointer, 1, 3, 2, 64, 1.0, None, None, b.pointer)   # heads % kv_heads
    with pytest.raises(StraydogError):
        gpu.attention(b.pointer, b.pointer, b.pointer, 16, p.pointer, 1, 2, 1, 2048, 1.0, None, None, b.pointer)  # dim too large
    with pytest.raises(StraydogError, match="scratch too small"):
        gpu.attention(b.pointer, b.pointer, b.pointer, 16, p.pointer, 1, 2, 1, 64, 1.0, None, None, b.pointer)   # a split needs scratch
    with pytest.raises(StraydogError, match="outside this device's allocations"):
        gpu.attention(b.pointer, b.pointer, b.pointer, 1 << 20, p.pointer, 1, 2, 1, 64, 1.0, None, None, b.pointer)
    gpu.release(b)
    gpu.release(p)
