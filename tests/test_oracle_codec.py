"""The oracle's Q8_0 codec against the properties the reference's own unit tests pin
(crates/straydog-engine/src/gpu.rs:4060-4143, kv_format_tests) and IEEE half conversions."""
import numpy as np

import oracle


def xorshift_row(seed, magnitude):
    # gpu.rs:4087-4095: xorshift32 (13, 17, 5) seeded with seed * 2654435761 (at least 1)
    state = max((seed * 2_654_435_761) & 0xFFFFFFFF, 1)
    out = np.empty(256, np.float32)
    for i in range(256):
        state ^= (state << 13) & 0xFFFFFFFF
        state ^= state >> 17
        state ^= (state << 5) & 0xFFFFFFFF
        out[i] = (np.float32(state) / np.float32(0xFFFFFFFF) * np.float32(2.0) - np.float32(1.0)) * np.float32(magnitude)
    return out


def test_half_conversions_match_numpy():
    rng = np.random.default_rng(1)
    values = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-4, 2000), rng.normal(0, 3e4, 2000),
                             [0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e-8, 5.96e-8, 2.98e-8, 2.99e-8, np.inf, -np.inf, 6.1e-5]]).astype(np.float32)
    for v in values:
        expected = np.float32(v).astype(np.float16)
        assert oracle.f32_to_f16(float(v)) == int(expected.view(np.uint16)), v
    for h in range(0, 65536, 7):
        x = np.array([h], np.uint16).view(np.float16)[0]
        if np.isnan(x):
            continue
        assert oracle.f16_to_f32(h) == float(x)


def test_rows_are_sized_for_their_format():
    assert oracle.ROW_Q8 == 272 and oracle.ROW_Q8 % 16 == 0 and 4 * oracle.ROW_Q8 == 1088
    assert 13 * 262_144 * 4 * oracle.ROW_Q8 == 3_707_764_736


def test_a_q8_row_holds_its_values_then_its_scales():
    values = ((np.arange(256, dtype=np.float32) - 128.0) / 16.0).astype(np.float32)
    packed = oracle.q8_encode_rows(values[None])[0]
    for block in range(8):
        part = values[block * 32:(block + 1) * 32]
        top = np.abs(part).max()
        scale = int(packed[256 + 2 * block]) | int(packed[257 + 2 * block]) << 8
        assert scale == int(np.float32(top / np.float32(127.0)).astype(np.float16).view(np.uint16))
        largest = block * 32 + int(np.argmax(np.abs(part)))
        assert abs(int(packed[largest].view(np.int8))) == 127
        assert (int(packed[largest].view(np.int8)) < 0) == (values[largest] < 0)
    assert int(packed[128].view(np.int8)) == 0


def test_q8_rows_come_back_within_half_a_scale():
    for seed in range(1, 200):
        magnitude = [1e-3, 0.1, 1.0, 30.0, 600.0][seed % 5]
        values = xorshift_row(seed, magnitude)
        packed = oracle.q8_encode_rows(values[None])
        back = oracle.q8_decode_rows(packed)[0]
        scales = packed[0, 256:].view(np.float16).astype(np.float32)
        for block in range(8):
            error = np.abs(back[block * 32:(block + 1) * 32] - values[block * 32:(block + 1) * 32])
            assert np.all(error <= scales[block] * 0.5 * 1.001 + np.abs(values[block * 32:(block + 1) * 32]) * 1e-3), (seed, block)
    zero = oracle.q8_encode_rows(np.zeros((1, 256), np.float32))
    assert not zero.any() and not oracle.q8_decode_rows(zero).any()
    values = xorshift_row(7, 1.0)
    before = oracle.q8_encode_rows(values[None])[0]
    values[3] = 500.0
    after = oracle.q8_encode_rows(values[None])[0]
    assert np.array_equal(before[32:256], after[32:256]) and np.array_equal(before[258:272], after[258:272])
    assert int(after[3].view(np.int8)) == 127


def test_encode_matches_a_numpy_restatement():
    # an independent formulation: scale = f16(max/127); q = rint(v / f32(scale)) (numpy rint is ties-to-even)
    rng = np.random.default_rng(5)
    values = (rng.normal(0, 1, (64, 256)) * rng.choice([1e-4, 0.02, 1.0, 50.0], (64, 1))).astype(np.float32)
    packed = oracle.q8_encode_rows(values)
    blocks = values.reshape(64, 8, 32)
    scale_h = (np.abs(blocks).max(-1) / np.float32(127.0)).astype(np.float32).astype(np.float16)
    scale = scale_h.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(scale[..., None] > 0, np.rint(blocks / scale[..., None]), 0.0)
    q = np.clip(q, -127, 127).astype(np.int8)
    assert np.array_equal(packed[:, :256].view(np.int8), q.reshape(64, 256))
    assert np.array_equal(packed[:, 256:].view(np.float16), scale_h)


def test_kv_write_places_rows_in_their_planes():
    rng = np.random.default_rng(9)
    context, kv_heads, base, steps = 40, 2, 7, 3
    state = np.zeros((2 * kv_heads, context, 272), np.uint8)
    keys = rng.normal(0, 1, (steps, kv_heads, 256)).astype(np.float32)
    values = rng.normal(0, 2, (steps, kv_heads, 256)).astype(np.float32)
    oracle.kv_write(state, context, kv_heads, base, keys, values)
    for step in range(steps):
        for head in range(kv_heads):
            assert np.array_equal(state[head, base + step], oracle.q8_encode_rows(keys[step, head][None])[0])
            assert np.array_equal(state[kv_heads + head, base + step], oracle.q8_encode_rows(values[step, head][None])[0])
    untouched = np.ones(context, bool)
    untouched[base:base + steps] = False
    assert not state[:, untouched].any()
