"""sdx_qsa_normalize_rows (the fused front of Qwen's decode and verification attention: gpu/qsa_decode.hpp:86-111) against the
oracle's restatement. The normalised and rotated values go through powf, cosf and sinf, whose device and host forms differ in
the last place (and a last place of 1e7^(c/32) moves the angle by position * 6e-8), so they are compared within 2e-4 at positions
below 4096; everything behind them is integer or codec work and is held bit for bit: the K rows are the codec's encoding of the
keys the call itself wrote, the V rows and the history ring equal the oracle's. Then the call feeds the indexer and the attention
as the reference's qsa_decode_attend_rows chains them (gpu/qsa_decode.hpp:113-129)."""
import numpy as np
import pytest

import oracle
from straydog_b200.backend import StraydogError

pytestmark = pytest.mark.gpu
SELECTED = 2052


def case(seed, heads, kv_heads, context, positions, ropes=None, pad=0):
    rng = np.random.default_rng(seed)
    positions = np.asarray(positions, np.uint32)
    rows, stride, pool = len(positions), heads * 512 + kv_heads * 512 + 640 + pad, context // 4 + 1
    c = dict(heads=heads, kv_heads=kv_heads, context=context, rows=rows, stride=stride, pool=pool, positions=positions,
             ropes=positions.copy() if ropes is None else np.asarray(ropes, np.uint32))
    c["proj"] = rng.normal(0, 1, (rows, stride)).astype(np.float32)
    c["norms"] = [rng.normal(1, 0.1, n).astype(np.float32) for n in (256, 256, 128, 128)]
    c["packed"] = np.zeros(rows * (heads * 256 + kv_heads * 512 + SELECTED + 1), np.float32)
    c["state"] = rng.integers(0, 256, context * 2 * kv_heads * 272, dtype=np.uint8)
    index_state = np.zeros((pool + 16) * 128, np.float32)
    index_state[pool * 128:] = rng.normal(0, 1, 16 * 128).astype(np.float32)
    c["index_state"] = index_state
    return c


def run(gpu, c, mirror_rows=0):
    bufs = dict(proj=gpu.upload(c["proj"]), packed=gpu.upload(c["packed"]), state=gpu.upload(c["state"]), index=gpu.upload(c["index_state"]),
                positions=gpu.upload(c["positions"]), ropes=gpu.upload(c["ropes"]))
    norms = [gpu.upload(n) for n in c["norms"]]
    mirror = gpu.buffer(mirror_rows * 2 * c["kv_heads"] * 272) if mirror_rows else None
    gpu.qsa_normalize_rows(bufs["proj"].pointer, c["stride"], c["rows"], c["heads"], c["kv_heads"], *[n.pointer for n in norms],
                           bufs["positions"].pointer, bufs["ropes"].pointer, bufs["packed"].pointer, SELECTED, bufs["state"], c["context"],
                           bufs["index"].pointer, mirror.pointer if mirror else None, mirror_rows)
    got = dict(proj=gpu.read(bufs["proj"], np.float32, c["proj"].shape), packed=gpu.read(bufs["packed"], np.float32, c["packed"].shape),
               state=gpu.read(bufs["state"], np.uint8, c["state"].shape), index=gpu.read(bufs["index"], np.float32, c["index_state"].shape))
    if mirror:
        got["mirror"] = gpu.read(mirror, np.uint8, (2 * c["kv_heads"], mirror_rows, 272))
        gpu.release(mirror)
    for b in norms:
        gpu.release(b)
    return got, bufs


def reference(c):
    want = dict(proj=c["proj"].copy(), packed=c["packed"].copy(), state=c["state"].copy(), index=c["index_state"].copy())
    oracle.qsa_normalize_rows(want["proj"], c["heads"], c["kv_heads"], *c["norms"], c["positions"], c["ropes"], want["packed"], want["state"],
                              c["context"], want["index"])
    return want


@pytest.mark.parametrize("heads,kv_heads,context,positions,pad", [
    (24, 2, 4096, [2041, 2042, 2043, 2044, 2045, 2046, 2047, 2048], 0),    # the reference's layer, a full verification span
    (12, 1, 512, [7], 0),                                                  # half a layer (one GPU of two), one decode token that completes a block
    (16, 2, 1024, [0, 1, 2, 3, 4], 24),                                    # the benchmark's heads, the sequence's first rows, a padded stride
    (16, 2, 4096, [3001], 0),
])
def test_rows_equal_the_oracles(gpu, heads, kv_heads, context, positions, pad):
    c = case(1 + heads, heads, kv_heads, context, positions, pad=pad)
    want = reference(c)
    got, bufs = run(gpu, c)
    assert gpu.decode_status() == 0
    rows, pool = c["rows"], c["pool"]
    live = rows * (heads + kv_heads) * 256
    assert np.abs(got["packed"][:live] - want["packed"][:live]).max() < 2e-4
    assert np.array_equal(got["packed"][live:], c["packed"][live:]), "values, lists and counts stay"
    index_at = heads * 512 + kv_heads * 512
    assert np.abs(got["proj"][:, index_at:index_at + 512] - want["proj"][:, index_at:index_at + 512]).max() < 2e-4
    keep = np.ones(c["stride"], bool)
    keep[index_at:index_at + 512] = False
    for h in range(heads):
        keep[h * 512:h * 512 + 256] = True   # (the queries themselves are not rewritten, only read)
    assert np.array_equal(got["proj"][:, keep], c["proj"][:, keep])
    # K/V rows: positions of the rows only; V rows and the ring bit for bit; K rows = the codec over the keys the call wrote
    mine, theirs, before = (x.reshape(2 * kv_heads, context, 272) for x in (got["state"], want["state"], c["state"]))
    untouched = np.ones(context, bool)
    untouched[c["positions"]] = False
    assert np.array_equal(mine[:, untouched], before[:, untouched])
    keys = got["packed"][rows * heads * 256:live].reshape(rows, kv_heads, 256)
    for r, p in enumerate(c["positions"]):
        for h in range(kv_heads):
            assert np.array_equal(mine[kv_heads + h, p], theirs[kv_heads + h, p])
            assert np.array_equal(mine[h, p], oracle.q8_encode_rows(keys[r, h][None])[0])
            assert np.abs(oracle.q8_decode_rows(mine[h, p][None]) - oracle.q8_decode_rows(theirs[h, p][None])).max() < 0.05
    assert np.array_equal(got["index"][pool * 128:], want["index"][pool * 128:]), "the history ring"
    assert np.abs(got["index"][:pool * 128] - want["index"][:pool * 128]).max() < 2e-4
    done = [int(p) // 4 for p in c["positions"] if (int(p) + 1) % 4 == 0]
    others = np.ones(pool, bool)
    others[done] = False
    assert not got["index"][:pool * 128].reshape(128, pool)[:, others].any(), "only completed blocks are written"
    for b in bufs.values():
        gpu.release(b)


def test_rotation_positions_of_their_own_and_the_mirror(gpu):
    # a sequence with an image before the rows: the rotations run ahead of the K/V positions; the mirror ring takes the same rows
    c = case(5, 16, 2, 2048, [1030, 1031, 1032], ropes=[1100, 1101, 1102])
    want = reference(c)
    got, bufs = run(gpu, c, mirror_rows=64)
    live = c["rows"] * 18 * 256
    assert np.abs(got["packed"][:live] - want["packed"][:live]).max() < 2e-4
    planes = got["state"].reshape(4, 2048, 272)
    for p in c["positions"]:
        assert np.array_equal(got["mirror"][:, p % 64], planes[:, p])
    assert not got["mirror"][:, :6].any() and not got["mirror"][:, 9:].any()
    assert np.abs(got["index"][:c["pool"] * 128] - want["index"][:c["pool"] * 128]).max() < 2e-4
    for b in bufs.values():
        gpu.release(b)


def test_the_call_feeds_the_indexer_and_the_attention(gpu):
    # qsa_decode_attend_rows' chain (gpu/qsa_decode.hpp:113-129) out of this library's entries: front, block choice, attention with
    # the output gate; against the same chain through the oracle
    heads, kv_heads, context = 16, 2, 4096
    positions = np.arange(2300, 2306, dtype=np.uint32)
    c = case(9, heads, kv_heads, context, positions)
    rows, pool, row_floats = c["rows"], c["pool"], heads * 256 + kv_heads * 512
    rng = np.random.default_rng(10)
    from util import q8_state
    c["state"] = q8_state(rng, context, kv_heads).view(np.uint8).ravel().copy()
    c["index_state"][:pool * 128] = rng.normal(0, 1, pool * 128).astype(np.float32)   # the blocks pooled so far
    got, bufs = run(gpu, c)
    index_at = heads * 512 + kv_heads * 512
    gpu.qsa_index_select(bufs["proj"].pointer + index_at * 4, c["stride"], bufs["index"].pointer, pool, 0, bufs["positions"].pointer, rows, SELECTED,
                         heads, kv_heads, bufs["packed"].pointer)
    out = gpu.buffer(rows * heads * 256 * 4)
    gpu.qsa_attention_rows(bufs["state"], context, 0, bufs["positions"].pointer, rows, SELECTED, heads, kv_heads, 0.0625, bufs["packed"].pointer,
                           out.pointer, gates=(bufs["proj"].pointer, c["stride"]))
    mine = gpu.read(out, np.float32, (rows, heads, 256))
    packed = gpu.read(bufs["packed"], np.float32, c["packed"].shape)
    assert gpu.decode_status() == 0
    # the oracle's chain over the GPU's own front (the rotation's last places would otherwise move a block choice at a tie)
    state_np, proj_np = gpu.read(bufs["state"], np.uint8, c["state"].shape), gpu.read(bufs["proj"], np.float32, c["proj"].shape)
    blocks_np = gpu.read(bufs["index"], np.float32, c["index_state"].shape)[:pool * 128].reshape(128, pool)
    lists = oracle.qsa_index_select(proj_np[:, index_at:index_at + 512], blocks_np, 0, rows, SELECTED, row_floats, got["packed"].copy(),
                                    positions=positions)
    assert np.array_equal(packed, lists)
    start = rows * row_floats
    counts = packed[start + rows * SELECTED:]
    want = np.zeros((rows, heads, 256))
    planes = oracle.q8_decode_rows(state_np.reshape(-1, 272)).reshape(2 * kv_heads, context, 256).astype(np.float64)
    for r in range(rows):
        chosen = packed[start + r * SELECTED:start + r * SELECTED + int(counts[r])].astype(np.int64)
        assert chosen.max() == positions[r], "a row sees its own position, written by the front"
        for h in range(heads):
            kv = h // (heads // kv_heads)
            scores = planes[kv, chosen] @ packed[(r * heads + h) * 256:(r * heads + h + 1) * 256].astype(np.float64) * 0.0625
            w = np.exp(scores - scores.max())
            gate = proj_np[r, h * 512 + 256:h * 512 + 512].astype(np.float64)
            want[r, h] = (w / w.sum()) @ planes[kv_heads + kv, chosen] / (1 + np.exp(-gate))
    assert np.abs(mine - want).max() < 1e-4
    for b in list(bufs.values()) + [out]:
        gpu.release(b)


def test_a_position_past_the_state_writes_nothing_and_is_reported(gpu):
    c = case(3, 16, 2, 256, [100, 300])
    got, bufs = run(gpu, c)
    assert gpu.decode_status() == 5
    mine, before = got["state"].reshape(4, 256, 272), c["state"].reshape(4, 256, 272)
    untouched = np.ones(256, bool)
    untouched[100] = False
    assert np.array_equal(mine[:, untouched], before[:, untouched]) and not np.array_equal(mine[:, 100], before[:, 100])
    assert gpu.decode_status() == 0
    for b in bufs.values():
        gpu.release(b)


def test_invalid_front_shapes_are_refused(gpu):
    c = case(4, 16, 2, 256, [10, 11])
    bufs = dict(proj=gpu.upload(c["proj"]), packed=gpu.upload(c["packed"]), state=gpu.upload(c["state"]), index=gpu.upload(c["index_state"]),
                positions=gpu.upload(c["positions"]), ropes=gpu.upload(c["ropes"]))
    norms = [gpu.upload(n) for n in c["norms"]]

    def call(stride=c["stride"], rows=2, heads=16, kv_heads=2, context=256, mirror_rows=0, state=None):
        gpu.qsa_normalize_rows(bufs["proj"].pointer, stride, rows, heads, kv_heads, *[n.pointer for n in norms], bufs["positions"].pointer,
                               bufs["ropes"].pointer, bufs["packed"].pointer, SELECTED, state or bufs["state"], context, bufs["index"].pointer, None, mirror_rows)
    for kwargs in (dict(stride=c["stride"] - 1), dict(rows=0), dict(rows=257), dict(heads=0), dict(kv_heads=0), dict(context=0), dict(mirror_rows=8)):
        with pytest.raises(StraydogError, match="invalid Straydog attention dimensions"):
            call(**kwargs)
    for kwargs in (dict(context=260), dict(rows=3), dict(state=bufs["packed"].pointer + 4)):   # a state, rows or an index state the buffers do not hold
        with pytest.raises(StraydogError, match="outside|allocation|range"):
            call(**kwargs)
    call()
    assert gpu.decode_status() == 0
    for b in list(bufs.values()) + norms:
        gpu.release(b)


# ---- sdx_qsa_normalize_chunk: the same front for a prompt chunk (gpu/prefill_batch.hpp:342-370, gpu/sparse_attention.hpp:87-106, 135-139) ----
def chunk_case(seed, heads, kv_heads, context, position, count):
    rng = np.random.default_rng(seed)
    c = dict(heads=heads, kv_heads=kv_heads, context=context, position=position, count=count, pool=context // 4 + 1)
    c["qgate"] = rng.normal(0, 1, (count, heads, 512)).astype(np.float32)
    c["key"], c["value"] = (rng.normal(0, 1, (count, kv_heads, 256)).astype(np.float32) for _ in range(2))
    c["iq"], c["ik"] = rng.normal(0, 1, (count, 4, 128)).astype(np.float32), rng.normal(0, 1, (count, 128)).astype(np.float32)
    c["norms"] = [rng.normal(1, 0.1, n).astype(np.float32) for n in (256, 256, 128, 128)]
    c["packed"] = np.zeros(count * (heads * 256 + kv_heads * 512 + SELECTED + 1), np.float32)
    c["state"] = rng.integers(0, 256, context * 2 * kv_heads * 272, dtype=np.uint8)
    c["index_state"] = np.zeros((c["pool"] + 16) * 128, np.float32)
    c["index_state"][c["pool"] * 128:] = rng.normal(0, 1, 16 * 128).astype(np.float32)
    return c


def run_chunk(gpu, c):
    names = ("qgate", "key", "value", "iq", "ik", "packed", "state", "index_state")
    bufs = {n: gpu.upload(c[n]) for n in names}
    norms = [gpu.upload(n) for n in c["norms"]]
    try:
        gpu.qsa_normalize_chunk(bufs["qgate"].pointer, bufs["key"].pointer, bufs["value"].pointer, bufs["iq"].pointer, bufs["ik"].pointer, c["count"],
                                c["position"], c["heads"], c["kv_heads"], *[n.pointer for n in norms], bufs["packed"].pointer, SELECTED, bufs["state"],
                                c["context"], bufs["index_state"].pointer)
        return {n: gpu.read(bufs[n], c[n].dtype, c[n].shape) for n in ("iq", "packed", "state", "index_state")}
    finally:
        for b in list(bufs.values()) + norms:
            gpu.release(b)


@pytest.mark.parametrize("heads,kv_heads,context,position,count", [(24, 2, 4096, 0, 300), (16, 2, 2048, 1021, 70), (12, 1, 512, 7, 1), (16, 2, 512, 6, 1),
                                                                   (16, 2, 1024, 509, 16)])
def test_a_chunks_front_equals_the_oracles_and_its_tokens_taken_as_rows(gpu, heads, kv_heads, context, position, count):
    c = chunk_case(position + count, heads, kv_heads, context, position, count)
    got = run_chunk(gpu, c)
    assert gpu.decode_status() == 0
    want = {n: c[n].copy() for n in ("iq", "packed", "state", "index_state")}
    oracle.qsa_normalize_chunk(c["qgate"], c["key"], c["value"], want["iq"], c["ik"], position, heads, kv_heads, *c["norms"], want["packed"],
                               want["state"], context, want["index_state"])
    live, pool = count * (heads + kv_heads) * 256, c["pool"]
    assert np.abs(got["packed"][:live] - want["packed"][:live]).max() < 2e-4
    assert np.array_equal(got["packed"][live:], want["packed"][live:]), "the values' copy; lists and counts stay"
    assert np.abs(got["iq"] - want["iq"]).max() < 2e-4
    assert np.abs(got["index_state"][:pool * 128] - want["index_state"][:pool * 128]).max() < 2e-4
    assert np.array_equal(got["index_state"][pool * 128:], want["index_state"][pool * 128:]), "the history ring"
    mine, theirs, before = (x.reshape(2 * kv_heads, context, 272) for x in (got["state"], want["state"], c["state"]))
    assert np.array_equal(mine[kv_heads:], theirs[kv_heads:]), "value rows"
    assert np.array_equal(mine[:, :position], before[:, :position]) and np.array_equal(mine[:, position + count:], before[:, position + count:])
    keys = got["packed"][count * heads * 256:live].reshape(count, kv_heads, 256)
    for h in range(kv_heads):
        assert np.array_equal(mine[h, position:position + count], oracle.q8_encode_rows(keys[:, h]))
    # the same tokens as decode rows (<= 256 a call): the same bits everywhere both forms write
    if count <= 256:
        proj = np.ascontiguousarray(np.concatenate([c["qgate"].reshape(count, -1), c["key"].reshape(count, -1), c["value"].reshape(count, -1),
                                                    c["iq"].reshape(count, -1), c["ik"]], axis=1))
        positions = np.arange(position, position + count, dtype=np.uint32)
        r = dict(heads=heads, kv_heads=kv_heads, context=context, rows=count, stride=proj.shape[1], pool=pool, positions=positions, ropes=positions,
                 proj=proj, norms=c["norms"], packed=c["packed"], state=c["state"], index_state=c["index_state"])
        rows, bufs = run(gpu, r)
        for b in bufs.values():
            gpu.release(b)
        assert np.array_equal(rows["packed"][:live].view(np.uint32), got["packed"][:live].view(np.uint32))
        assert np.array_equal(rows["state"], got["state"])
        index_at = heads * 512 + kv_heads * 512
        assert np.array_equal(rows["proj"][:, index_at:index_at + 512].view(np.uint32), got["iq"].reshape(count, 512).view(np.uint32))
        assert np.array_equal(rows["index"][:pool * 128].view(np.uint32), got["index_state"][:pool * 128].view(np.uint32))


def image_axes(rng, first, count, position):
    """Rope positions of a sequence with images: text before (one position on all three axes), then an image's grid (t fixed, h and w
    running), then text again: three positions a row from `first`."""
    axes = np.zeros((count, 3), np.uint32)
    for i in range(count):
        p = first + i
        if p < position + 3:
            axes[i] = p
        elif p < position + 3 + 48:
            g = p - (position + 3)
            axes[i] = (position + 3, position + 3 + g // 8, position + 3 + g % 8)
        else:
            axes[i] = p - 40
    return axes


@pytest.mark.parametrize("heads,kv_heads,context,position,count", [(16, 2, 2048, 1021, 70), (24, 2, 1024, 0, 64), (16, 2, 512, 6, 1)])
def test_a_chunk_of_a_sequence_with_images_turns_by_the_rope_table(gpu, heads, kv_heads, context, position, count):
    """sd_rope_rows (gpu/straydog_gpu.h:607-609): with a table set the chunk's tokens and pooled blocks turn by three positions a row
    (gpu/sparse_attention.hpp:27-50, 111-131). A table of the rows' own positions on all three axes gives the bits of no table at all
    (text: the reference's own remark); an image's table gives the oracle's restatement; a table that does not cover the chunk is refused."""
    c = chunk_case(position + count + 1, heads, kv_heads, context, position, count)
    plain = run_chunk(gpu, c)
    first = position // 4 * 4
    own = np.repeat(np.arange(first, position + count, dtype=np.uint32)[:, None], 3, axis=1)
    try:
        gpu.rope_rows(first, own)
        same = run_chunk(gpu, c)
        for name in ("iq", "packed", "state", "index_state"):
            assert np.array_equal(np.ascontiguousarray(same[name]).view(np.uint8), np.ascontiguousarray(plain[name]).view(np.uint8)), name
        axes = image_axes(np.random.default_rng(3), first, position + count - first, position)
        gpu.rope_rows(first, axes)
        got = run_chunk(gpu, c)
        want = {n: c[n].copy() for n in ("iq", "packed", "state", "index_state")}
        oracle.qsa_normalize_chunk(c["qgate"], c["key"], c["value"], want["iq"], c["ik"], position, heads, kv_heads, *c["norms"], want["packed"],
                                   want["state"], context, want["index_state"], rope_rows=axes, rope_first=first)
        live, pool = count * (heads + kv_heads) * 256, c["pool"]
        assert np.abs(got["packed"][:live] - want["packed"][:live]).max() < 2e-4
        assert np.abs(got["iq"] - want["iq"]).max() < 2e-4
        assert np.abs(got["index_state"][:pool * 128] - want["index_state"][:pool * 128]).max() < 2e-4
        assert np.array_equal(got["index_state"][pool * 128:], want["index_state"][pool * 128:]), "the history ring"
        if count > 8:
            assert np.abs(got["packed"][:live] - plain["packed"][:live]).max() > 1e-2, "the image's rows turn elsewhere"
        mine, theirs = (x.reshape(2 * kv_heads, context, 272) for x in (got["state"], want["state"]))
        assert np.array_equal(mine[kv_heads:], theirs[kv_heads:]), "value rows"
        keys = got["packed"][count * heads * 256:live].reshape(count, kv_heads, 256)
        for h in range(kv_heads):
            assert np.array_equal(mine[h, position:position + count], oracle.q8_encode_rows(keys[:, h]))
        # a table that starts behind the chunk's first row, or ends before its last
        gpu.rope_rows(position + 1, axes)
        with pytest.raises(StraydogError, match="rope table"):
            run_chunk(gpu, c)
        gpu.rope_rows(first, axes[:-1])
        with pytest.raises(StraydogError, match="rope table"):
            run_chunk(gpu, c)
        with pytest.raises(StraydogError, match="rope table"):
            gpu.rope_rows(0, np.zeros((4101, 3), np.uint32))
    finally:
        gpu.rope_rows(0, None)
    again = run_chunk(gpu, c)
    assert np.array_equal(again["packed"].view(np.uint32), plain["packed"].view(np.uint32)), "count 0: the rows' own positions again"


def test_invalid_chunk_shapes_are_refused(gpu):
    c = chunk_case(2, 16, 2, 256, 100, 8)
    for kwargs in (dict(count=0), dict(position=250), dict(heads=0), dict(context=0)):
        d = dict(c)
        d.update(kwargs)
        with pytest.raises(StraydogError, match="invalid Straydog attention dimensions"):
            run_chunk(gpu, d)
    d = dict(c)
    d["count"] = 9   # more tokens than the arrays hold
    with pytest.raises(StraydogError, match="outside"):
        run_chunk(gpu, d)


def test_fp16_rows_take_the_nearest_fp16_of_the_keys_and_values():
    # sd_kv_format(512): the front writes FP16 rows (gpu/kernels.cpp:70), both forms
    from straydog_b200.backend import Backend
    with Backend(0, 1 << 29) as fp16:
        fp16.kv_format(512)
        c = case(8, 16, 2, 128, [60, 61, 62, 63])
        c["state"] = np.zeros(128 * 4 * 512, np.uint8)
        got, bufs = run(fp16, c)
        rows = got["state"].view(np.float16).reshape(4, 128, 256)
        keys = got["packed"][4 * 16 * 256:4 * 18 * 256].reshape(4, 2, 256)
        values = c["proj"][:, 16 * 512 + 512:16 * 512 + 1024].reshape(4, 2, 256)
        assert np.array_equal(rows[:2, 60:64].view(np.uint16), keys.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
        assert np.array_equal(rows[2:, 60:64].view(np.uint16), values.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
        assert not rows[:, :60].any() and not rows[:, 64:].any()
