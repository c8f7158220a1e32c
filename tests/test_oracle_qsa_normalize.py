"""The oracle's restatement of qsa_normalize_rows (gpu/qsa_decode.hpp:86-111, gpu/sparse_attention.hpp:2-6, 55-71) against an
independent numpy statement of the same rule in float64. (The pin to the reference's own library: tests/test_golden_oracle.py and
tests/test_gpu_qsa_layer.py, over what sd_qsa_sequence leaves behind when its weight matrices are selection matrices.)"""
import numpy as np
import pytest

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


def chunk_case(seed, heads, kv_heads, context, position, count):
    rng = np.random.default_rng(seed)
    c = dict(heads=heads, kv_heads=kv_heads, context=context, position=position, count=count, pool=context // 4 + 1)
    c["qgate"] = rng.normal(0, 1, (count, heads, 512)).astype(np.float32)
    c["key"], c["value"] = (rng.normal(0, 1, (count, kv_heads, 256)).astype(np.float32) for _ in range(2))
    c["iq"], c["ik"] = rng.normal(0, 1, (count, 4, 128)).astype(np.float32), rng.normal(0, 1, (count, 128)).astype(np.float32)
    c["norms"] = [rng.normal(1, 0.1, n).astype(np.float32) for n in (256, 256, 128, 128)]
    c["packed"] = np.zeros(count * (heads * 256 + kv_heads * 512 + 2052 + 1), np.float32)
    c["state"] = np.zeros(context * 2 * kv_heads * 272, np.uint8)
    c["index_state"] = np.zeros((c["pool"] + 16) * 128, np.float32)
    c["index_state"][c["pool"] * 128:] = rng.normal(0, 1, 16 * 128).astype(np.float32)
    return c


def as_rows(c):
    """The chunk's tokens as decode rows: one projections row a token, positions and rotation positions position + t."""
    heads, kv_heads, count = c["heads"], c["kv_heads"], c["count"]
    proj = np.concatenate([c["qgate"].reshape(count, -1), c["key"].reshape(count, -1), c["value"].reshape(count, -1),
                           c["iq"].reshape(count, -1), c["ik"]], axis=1).astype(np.float32)
    assert proj.shape[1] == heads * 512 + kv_heads * 512 + 640
    return np.ascontiguousarray(proj), np.arange(c["position"], c["position"] + count, dtype=np.uint32)


@pytest.mark.parametrize("position,count", [(0, 9), (6, 1), (7, 1), (10, 14), (13, 30), (21, 3)])
def test_a_prompt_chunks_front_equals_its_tokens_taken_as_rows(position, count):
    # qsa_pool takes a block's positions before the chunk from the ring and the rest from the chunk (gpu/sparse_attention.hpp:87-106);
    # the rows' form passes every token through the ring (gpu/qsa_decode.hpp:51-83): the same numbers, so the same bits
    c = chunk_case(position * 100 + count, 4, 2, 64, position, count)
    iq = c["iq"].copy()
    packed, state, index_state = c["packed"].copy(), c["state"].copy(), c["index_state"].copy()
    oracle.qsa_normalize_chunk(c["qgate"], c["key"], c["value"], iq, c["ik"], position, 4, 2, *c["norms"], packed, state, 64, index_state)
    proj, positions = as_rows(c)
    packed_r, state_r, index_r = c["packed"].copy(), c["state"].copy(), c["index_state"].copy()
    oracle.qsa_normalize_rows(proj, 4, 2, *c["norms"], positions, positions, packed_r, state_r, 64, index_r)
    live = count * (4 + 2) * 256
    assert np.array_equal(packed[:live].view(np.uint32), packed_r[:live].view(np.uint32))
    assert np.array_equal(packed[live:live + count * 512].reshape(count, 2, 256), c["value"]), "a chunk's values are copied into the packed rows"
    assert not packed_r[live:].any() and not packed[live + count * 512:].any()
    assert np.array_equal(state, state_r)
    assert np.array_equal(iq.reshape(count, 512).view(np.uint32), proj[:, 4 * 512 + 2 * 512:4 * 512 + 2 * 512 + 512].view(np.uint32))
    pool = c["pool"]
    assert np.array_equal(index_state[:pool * 128].view(np.uint32), index_r[:pool * 128].view(np.uint32)), "the pooled blocks"
    # the ring: a chunk saves its last four tokens, the rows every token; the slots both wrote agree and hold the index keys
    ring, ring_r = index_state[pool * 128:].reshape(16, 128), index_r[pool * 128:].reshape(16, 128)
    for t in range(max(0, count - 4), count):
        assert np.array_equal(ring[(position + t) % 16], c["ik"][t]) and np.array_equal(ring_r[(position + t) % 16], c["ik"][t])
    done = list(range(position // 4, (position + count) // 4))
    blocks = index_state[:pool * 128].reshape(128, pool)
    assert all(blocks[:, b].any() for b in done) and not np.delete(blocks, done, axis=1).any()


def test_a_rope_table_of_the_rows_own_positions_is_no_table_and_an_images_rows_turn_by_their_axes():
    # gpu/sparse_attention.hpp:27-32: text holds one position on all three axes, which is qsa_rope's angle; pair p turns by axis p % 3
    position, count = 13, 30
    c = chunk_case(7, 4, 2, 64, position, count)
    outs = []
    first = position // 4 * 4
    own = np.repeat(np.arange(first, position + count, dtype=np.uint32)[:, None], 3, axis=1)
    axes = own.copy()
    axes[5:25, 1] += 7          # an image's rows: other positions on the h and w axes
    axes[5:25, 2] += 11
    for table in (None, own, axes):
        iq, packed, state, index_state = c["iq"].copy(), c["packed"].copy(), c["state"].copy(), c["index_state"].copy()
        oracle.qsa_normalize_chunk(c["qgate"], c["key"], c["value"], iq, c["ik"], position, 4, 2, *c["norms"], packed, state, 64, index_state,
                                   rope_rows=table, rope_first=first)
        outs.append((iq, packed, state, index_state))
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
    queries = [o[1][:count * 4 * 256].reshape(count, 4, 256) for o in outs]
    turned = np.abs(queries[2] - queries[0]).max(axis=1)        # [token][column]
    rows = np.arange(5, 25) - (position - first)                # the table's rows 5..24 are tokens 4..23
    pairs = np.arange(32)
    assert not turned[:, 64:].any(), "columns from 64 on pass"
    assert not turned[:rows[0]].any() and not turned[rows[-1] + 1:].any(), "text rows turn as before"
    assert not turned[rows][:, pairs[pairs % 3 == 0]].any(), "the t axis kept its position"
    assert (turned[rows][:, pairs[pairs % 3 == 1]] > 0).any() and (turned[rows][:, pairs[pairs % 3 == 2]] > 0).any()
    # a pooled block turns by the table's row of its first position
    blocks = [o[3][:c["pool"] * 128].reshape(128, c["pool"]) for o in outs]
    changed = np.abs(blocks[2] - blocks[0]).max(axis=0) > 0
    begins = np.arange(c["pool"]) * 4
    inside = (begins >= first + 5) & (begins < first + 25) & (begins + 4 <= position + count)
    assert changed[inside].all() and not changed[~inside].any()
