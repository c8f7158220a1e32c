"""The oracle's restatement of qsa_normalize_rows (gpu/qsa_decode.hpp:86-111, gpu/sparse_attention.hpp:2-6, 55-71) against an
independent numpy statement of the same rule in float64. Parity unpinned: the reference's library reaches this kernel only inside
sd_qsa_sequence, which needs a layer's weights."""
import numpy as np

import oracle


def rope64(x, position):
    """x [..., width] float64: columns c < 64 turn with (c + 32) % 64 by position / 1e7^((c % 32) / 32)."""
    out = x.copy()
    c = np.arange(64)
    angle = position / np.power(1e7, (c % 32) / 32.0)
    partner = x[..., (c + 32) % 64]
    out[..., :64] = x[..., :64] * np.cos(angle) + np.where(c < 32, -partner, partner) * np.sin(angle)
    return out


def normalize64(x, norm, position):
    x = x.astype(np.float64)
    return rope64(x * norm / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6), position)


def test_rows_are_normalised_rotated_written_and_pooled():
    rng = np.random.default_rng(11)
    heads, kv_heads, context, selected = 6, 2, 64, 2052
    stride = heads * 512 + kv_heads * 512 + 640 + 8
    positions = np.array([9, 10, 11, 12, 13], np.uint32)      # position 11 completes block 2
    ropes = positions + 3                                     # (a sequence with an image before: rotation positions run ahead)
    rows = len(positions)
    proj = rng.normal(0, 1, (rows, stride)).astype(np.float32)
    before = proj.copy()
    qnorm, knorm = rng.normal(1, 0.1, 256).astype(np.float32), rng.normal(1, 0.1, 256).astype(np.float32)
    iqnorm, pool_norm = rng.normal(1, 0.1, 128).astype(np.float32), rng.normal(1, 0.1, 128).astype(np.float32)
    packed = np.zeros(rows * (heads * 256 + kv_heads * 512 + selected + 1), np.float32)
    state = np.zeros(context * 2 * kv_heads * 272, np.uint8)
    pool = context // 4 + 1
    index_state = np.zeros((pool + 16) * 128, np.float32)
    history0 = rng.normal(0, 1, (16, 128)).astype(np.float32)   # what the positions before the rows left in the ring
    index_state[pool * 128:] = history0.ravel()
    oracle.qsa_normalize_rows(proj, heads, kv_heads, qnorm, knorm, iqnorm, pool_norm, positions, ropes, packed, state, context, index_state)

    keys_at, values_at, index_at = heads * 512, heads * 512 + kv_heads * 256, heads * 512 + kv_heads * 512
    q = packed[:rows * heads * 256].reshape(rows, heads, 256)
    k = packed[rows * heads * 256:rows * (heads + kv_heads) * 256].reshape(rows, kv_heads, 256)
    planes = state.reshape(2 * kv_heads, context, 272)
    for r in range(rows):
        want_q = normalize64(before[r, :keys_at].reshape(heads, 512)[:, :256], qnorm, float(ropes[r]))
        want_k = normalize64(before[r, keys_at:values_at].reshape(kv_heads, 256), knorm, float(ropes[r]))
        want_iq = normalize64(before[r, index_at:index_at + 512].reshape(4, 128), iqnorm, float(ropes[r]))
        assert np.abs(q[r] - want_q).max() < 2e-5
        assert np.abs(k[r] - want_k).max() < 2e-5
        assert np.abs(proj[r, index_at:index_at + 512].reshape(4, 128) - want_iq).max() < 2e-5
        # the gate halves, the values and the index keys are left as they were
        assert np.array_equal(proj[r, :keys_at].reshape(heads, 512)[:, 256:], before[r, :keys_at].reshape(heads, 512)[:, 256:])
        assert np.array_equal(proj[r, values_at:index_at], before[r, values_at:index_at])
        # the K/V rows are the codec's encoding of the normalised keys and of the values, bit for bit
        for h in range(kv_heads):
            assert np.array_equal(planes[h, positions[r]], oracle.q8_encode_rows(k[r, h][None])[0])
            assert np.array_equal(planes[kv_heads + h, positions[r]], oracle.q8_encode_rows(before[r, values_at + 256 * h:values_at + 256 * (h + 1)][None])[0])
    assert not planes[:, :9].any() and not planes[:, 14:].any()
    # the ring holds the rows' index keys at position % 16; the other slots are untouched
    ring = index_state[pool * 128:].reshape(16, 128)
    for r in range(rows):
        assert np.array_equal(ring[positions[r] % 16], before[r, index_at + 512:index_at + 640])
    for slot in set(range(16)) - {int(p) % 16 for p in positions}:
        assert np.array_equal(ring[slot], history0[slot])
    # position 11 completed block 2 = positions 8..11: position 8 from the ring as it was, 9..11 from the rows
    taps = np.stack([history0[8], before[0, index_at + 512:index_at + 640], before[1, index_at + 512:index_at + 640],
                     before[2, index_at + 512:index_at + 640]]).astype(np.float64)
    want_block = normalize64(taps.mean(0), pool_norm, float(ropes[2]) - 3)
    blocks = index_state[:pool * 128].reshape(128, pool)
    assert np.abs(blocks[:, 2] - want_block).max() < 2e-5
    assert not blocks[:, :2].any() and not blocks[:, 3:].any()


def test_one_row_is_the_decode_steps_front():
    # rows = 1: what qsa_normalize_decode + qsa_pool_one + write_attention_kv do for one token (gpu/qsa_decode.hpp:28-44)
    rng = np.random.default_rng(12)
    heads, kv_heads, context = 4, 1, 32
    stride = heads * 512 + kv_heads * 512 + 640
    proj = rng.normal(0, 1, (1, stride)).astype(np.float32)
    norms = [np.ones(256, np.float32), np.ones(256, np.float32), np.ones(128, np.float32), np.ones(128, np.float32)]
    packed = np.zeros(heads * 256 + kv_heads * 512 + 2052 + 1, np.float32)
    state = np.zeros(context * 2 * kv_heads * 272, np.uint8)
    index_state = np.zeros((context // 4 + 1 + 16) * 128, np.float32)
    want = normalize64(proj[0, :256].copy(), norms[0], 5.0)
    oracle.qsa_normalize_rows(proj, heads, kv_heads, *norms, [5], [5], packed, state, context, index_state)
    assert np.abs(packed[:256] - want).max() < 2e-5
    assert not index_state[:(context // 4 + 1) * 128].any()   # position 5 completes no block
