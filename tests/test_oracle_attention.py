"""The oracle's attention restatements against independent formulations: a numpy F64 softmax, the
reference's top-k rule written out in Python (tests/fused_gpu.rs:325-357), and its own F64 variants."""
import numpy as np

import oracle
from util import XorShift, bf16_round, q8_state, queries_f16, tie_scores


def numpy_attention(q, k, v, scale):
    s = (q.astype(np.float64) @ k.astype(np.float64).T) * scale
    p = np.exp(s - s.max(-1, keepdims=True))
    return (p @ v.astype(np.float64)) / p.sum(-1, keepdims=True)


def test_gqa_decode_q8_matches_numpy_f64():
    rng = np.random.default_rng(11)
    context, length, heads, kv_heads = 300, 257, 16, 2
    state = q8_state(rng, context, kv_heads)
    q = queries_f16(rng, heads, 256)
    planes = oracle.q8_decode_rows(state.reshape(-1, 272)).reshape(2 * kv_heads, context, 256)
    got32 = oracle.gqa_decode_q8(state, context, length, heads, kv_heads, q, 1 / 16)
    got64 = oracle.gqa_decode_q8(state, context, length, heads, kv_heads, q, 1 / 16, f64=True)
    for h in range(heads):
        kv = h // (heads // kv_heads)
        want = numpy_attention(q[h:h + 1].astype(np.float32), planes[kv, :length], planes[kv_heads + kv, :length], 1 / 16)[0]
        assert np.abs(got64[h] - want).max() < 1e-6
        assert np.abs(got32[h] - want).max() < 1e-4


def test_attention_sequence_matches_dense_decode_on_identity_selection():
    rng = np.random.default_rng(12)
    context, base, heads, kv_heads, selected = 64, 40, 24, 2, 41
    state = q8_state(rng, context, kv_heads, filled=base)
    q = rng.normal(0, 1, (1, heads, 256)).astype(np.float16).astype(np.float32)
    k = rng.normal(0, 1, (1, kv_heads, 256)).astype(np.float32)
    v = rng.normal(0, 1, (1, kv_heads, 256)).astype(np.float32)
    packed = np.concatenate([q.ravel(), k.ravel(), v.ravel(), np.arange(selected, dtype=np.float32), [np.float32(selected)]])
    out = oracle.attention_sequence(state, context, heads, kv_heads, base, 1, selected, packed)
    dense = oracle.gqa_decode_q8(state, context, base + 1, heads, kv_heads, q[0].astype(np.float16), 0.0625)
    assert np.abs(out[0] - dense).max() < 2e-5
    # the new row was written before attending
    assert np.array_equal(state[0, base], oracle.q8_encode_rows(k[0, 0][None])[0])


def test_attention_sequence_masks_dead_slots():
    rng = np.random.default_rng(13)
    context, base, heads, kv_heads, selected = 32, 10, 24, 2, 8
    state = q8_state(rng, context, kv_heads, filled=base)
    q = rng.normal(0, 1, (heads, 256)).astype(np.float32)
    kv = rng.normal(0, 1, (2, kv_heads, 256)).astype(np.float32)
    # slots: a valid one, a future position, a negative, one past the count
    idx = np.array([3, 11, -1, 5, 10, 31, 2, 7], np.float32)
    packed = np.concatenate([q.ravel(), kv.ravel(), idx, [np.float32(6)]])
    out = oracle.attention_sequence(state.copy(), context, heads, kv_heads, base, 1, selected, packed)
    idx2 = np.array([3, 5, 10, 0, 0, 0, 0, 0], np.float32)
    packed2 = np.concatenate([q.ravel(), kv.ravel(), idx2, [np.float32(3)]])
    out2 = oracle.attention_sequence(state.copy(), context, heads, kv_heads, base, 1, selected, packed2)
    assert np.abs(out - out2).max() < 1e-6


def test_op_attention_f32_within_the_reference_bound_of_f64():
    # shapes of crates/straydog-engine/tests/attention_gpu.rs:135-142 (a subset that runs in seconds)
    for rows, heads, kv_heads, dim, context in [(15, 4, 2, 256, 33), (17, 4, 2, 256, 35), (16, 4, 2, 128, 35), (1, 2, 1, 256, 137), (17, 1, 1, 256, 1)]:
        random = XorShift(0x9E3779B97F4A7C15 ^ rows ^ (dim << 16))
        q = random.floats_unit(rows * heads * dim)
        keys = random.floats_unit(context * kv_heads * dim)
        values = random.floats_unit(context * kv_heads * dim)
        special = [0, 1, 15, 16, context - 1, context + 7]
        positions = np.array([special[r] if r < len(special) else (r * 17 + 3) % context for r in range(rows)], np.int32)
        gate = np.array([[-12.0, -1.0, 0.0, 1.0, 12.0][i % 5] for i in range(q.size)], np.float32)
        scale = np.float32(1.0) / np.sqrt(np.float32(dim))
        for g in (None, gate):
            out, out64, bound = oracle.op_attention(q, keys, values, context, positions, rows, heads, kv_heads, dim, float(scale), g, want64=True)
            assert np.all(np.abs(out.astype(np.float64) - out64) <= bound)
        # the F64 reference against numpy for row 0 (position 0: one key) and the last row
        r = rows - 1
        length = min(int(positions[r]) + 1, context)
        kk = keys.reshape(context, kv_heads, dim)[:length, 0]
        vv = values.reshape(context, kv_heads, dim)[:length, 0]
        want = numpy_attention(q.reshape(rows, heads, dim)[r, 0:1], kk, vv, float(scale))[0]
        _, out64, _ = oracle.op_attention(q, keys, values, context, positions, rows, heads, kv_heads, dim, float(scale), None, want64=True)
        assert np.abs(out64[r, 0] - want).max() < 1e-9


def python_top_k(scores, k):
    def key(v):
        v = np.float32(0.0) if v == 0 else np.float32(v)
        bits = int(np.array([v], np.float32).view(np.uint32)[0])
        return (~bits) & 0xFFFFFFFF if bits & 0x80000000 else bits | 0x80000000
    floor = key(-np.inf)
    keys = [key(s) for s in scores]
    live = [g for g in range(len(scores)) if keys[g] > floor]
    if len(live) <= k:
        out = list(live)
    else:
        threshold = sorted((keys[g] for g in live), reverse=True)[k - 1]
        need = k - sum(keys[g] > threshold for g in live)
        out = []
        for g in live:
            if keys[g] > threshold:
                out.append(g)
            elif keys[g] == threshold and need > 0:
                out.append(g)
                need -= 1
    return out + [-1] * (k - len(out))


def test_top_k_matches_the_reference_rule_with_many_ties():
    random = XorShift(0x2F6B91D3C0A54E77)
    k = 512
    for groups in [511, 512, 513, 600, 4096]:
        scores = tie_scores(random, 2, groups)
        got = oracle.top_k(scores, k)
        for row in range(2):
            assert list(got[row]) == python_top_k(list(scores[row]), k), groups


def test_sparse_attention_f32_close_to_f64_and_bf16_equals_widened():
    rng = np.random.default_rng(21)
    rows, heads, dim, window, raw_rows, compressed_rows, selections, rope_dims = 3, 4, 128, 16, 32, 50, 24, 32
    q = rng.normal(0, 1, (rows, heads, dim)).astype(np.float32)
    raw = rng.normal(0, 1, (raw_rows, dim)).astype(np.float32)
    halves, widened = bf16_round(rng.normal(0, 1, (compressed_rows, dim)).astype(np.float32))
    sinks = rng.normal(0, 2, heads).astype(np.float32)
    positions = np.array([3, 40, 100], np.int32)
    selected = rng.integers(0, compressed_rows, (rows, selections)).astype(np.int32)
    selected[:, 5] = -1
    freq = (10000.0 ** (-(2.0 * np.arange(rope_dims // 2)) / rope_dims)).astype(np.float32)
    args = (q, raw, raw_rows, positions, window)
    rest = (selected, selections, sinks, rows, heads, dim, 1 / np.sqrt(dim), rope_dims, freq)
    a = oracle.sparse_attention(*args, widened, *rest)
    b = oracle.sparse_attention(*args, halves, *rest)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    c = oracle.sparse_attention(*args, halves, *rest, f64=True)
    assert np.abs(a - c).max() < 2e-5
    # without rope and sinks at -inf a row is a plain softmax over its keys
    d = oracle.sparse_attention(q, raw, raw_rows, positions, window, halves, selected, selections, np.full(heads, -np.inf, np.float32),
                                rows, heads, dim, 1 / np.sqrt(dim), 0, None, f64=True)
    r, p = 1, 40
    keys = np.concatenate([raw[[(i % raw_rows) for i in range(p - window + 1, p + 1)]], widened[[s for s in selected[r] if s >= 0]]])
    want = numpy_attention(q[r], keys, keys, 1 / np.sqrt(dim))
    assert np.abs(d[r] - want).max() < 1e-6


def test_to_bf16_rounds_to_nearest_even():
    x = np.array([0.0, -0.0, np.inf, -np.inf, 3.4028235e38, 1.17549435e-38, 1 + 1 / 256, 1 + 3 / 256], np.float32)
    x = np.concatenate([x, np.array([0x3F808000, 0x3F818000], np.uint32).view(np.float32), np.random.default_rng(3).normal(0, 1e3, 1000).astype(np.float32)])
    got = oracle.to_bf16(x)
    want, _ = bf16_round(x)
    assert np.array_equal(got, want)
    assert np.isnan(oracle.bf16_to_f32(oracle.to_bf16(np.array([np.nan], np.float32)))[0])
