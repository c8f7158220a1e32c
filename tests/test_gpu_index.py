"""The indexer's entries (sd_op_rope, sd_op_index_scores, sd_op_top_k, sd_op_index_select, sd_op_index_select_proj, sd_op_index_candidates, sd_op_compress) in the
manner of the reference's own tests (crates/straydog-engine/tests/fused_gpu.rs:391-431 and :477-545): the fused call gives the separate
calls' scores and indices bit for bit and leaves q as it was; the two-level pick is the top k over every group with the groups outside
the candidate blocks at -inf; and each against the reference library's own outputs and the CPU oracle."""
import os

import numpy as np
import pytest

import oracle
from straydog_b200.backend import StraydogError
from util import INDEX_CASES, INDEX_PROJ_CASES, TWO_LEVEL_CASES, compress_case, index_case, index_proj_case

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz"))
K = 512


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


class Case:
    def __init__(self, gpu, c, keys=None):
        self.gpu, self.c = gpu, c
        self.bufs = {name: gpu.upload(c[name]) for name in ("q", "weights", "visible", "positions", "frequencies")}
        self.bufs["keys"] = keys if keys is not None else gpu.upload(c["keys"])
        self.owned_keys = keys is None

    def select(self, k=K, candidates=None, keys=None):
        gpu, c, b = self.gpu, self.c, self.bufs
        scored = c["groups"] if candidates is None else candidates[1] * candidates[2]
        scores, picked = gpu.buffer(c["rows"] * max(scored, c["groups"]) * 4), gpu.buffer(c["rows"] * k * 4)
        gpu.index_select(b["q"].pointer, keys or b["keys"].pointer, b["weights"].pointer, b["visible"].pointer, c["rows"], c["groups"], c["heads"],
                         c["dim"], c["scale"], (c["rope_dims"], b["positions"].pointer, b["frequencies"].pointer), scores.pointer, k, picked.pointer,
                         candidates)
        got = gpu.read(scores, np.float32, (c["rows"], scored)), gpu.read(picked, np.int32, (c["rows"], k))
        gpu.release(picked)
        return got + (scores,)

    def apart(self, k=K):
        gpu, c, b = self.gpu, self.c, self.bufs
        q = gpu.upload(c["q"])
        scores, picked = gpu.buffer(c["rows"] * c["groups"] * 4), gpu.buffer(c["rows"] * k * 4)
        gpu.rope(q.pointer, c["rows"], c["heads"], c["dim"], c["rope_dims"], b["positions"].pointer, b["frequencies"].pointer)
        gpu.index_scores(q.pointer, b["keys"].pointer, b["weights"].pointer, b["visible"].pointer, c["rows"], c["groups"], c["heads"], c["dim"],
                         c["scale"], scores.pointer)
        gpu.top_k(scores.pointer, c["rows"], c["groups"], k, picked.pointer)
        got = gpu.read(scores, np.float32, (c["rows"], c["groups"])), gpu.read(picked, np.int32, (c["rows"], k))
        for x in (q, scores, picked):
            gpu.release(x)
        return got

    def close(self):
        for name, b in self.bufs.items():
            if name != "keys" or self.owned_keys:
                self.gpu.release(b)


@pytest.mark.parametrize("rows,groups", INDEX_CASES)
def test_an_index_select_matches_rope_scores_and_top_k(gpu, rows, groups):
    c = index_case(rows, groups)
    case = Case(gpu, c)
    scores_1, picked_1 = case.apart()
    for run in range(2):
        scores_2, picked_2, held = case.select()
        gpu.release(held)
        assert np.array_equal(bits(scores_1), bits(scores_2)), f"run {run}: scores"
        assert np.array_equal(picked_1, picked_2), f"run {run}: indices"
    assert np.array_equal(bits(gpu.read(case.bufs["q"], np.float32, c["q"].shape)), bits(c["q"])), "q unchanged"
    # the reference library's outputs for the same inputs, bit for bit; the CPU oracle within its sin and cos
    assert np.array_equal(bits(scores_2), bits(GOLDEN[f"index_scores_{rows}_{groups}"]))
    assert np.array_equal(picked_2, GOLDEN[f"index_top_{rows}_{groups}"])
    want, _ = oracle.index_select(c["q"], c["keys"], c["weights"], c["visible"], c["scale"], c["positions"], c["frequencies"], K)
    seen = np.isfinite(want)
    assert np.array_equal(seen, np.isfinite(scores_2))
    assert np.abs(scores_2[seen] - want[seen]).max() <= 1e-5
    assert np.array_equal(picked_2, oracle.top_k(scores_2, K))
    for row in range(rows):   # -inf from the row's visible count on
        assert np.all(np.isneginf(scores_2[row, c["visible"][row]:])) and np.all(seen[row, :c["visible"][row]])
    case.close()


def test_bf16_tagged_keys_score_as_their_widened_rows(gpu):
    c = index_case(2, 1500)
    halves = oracle.to_bf16(c["keys"])
    c["keys"] = oracle.bf16_to_f32(halves)
    case = Case(gpu, c)
    plain, picked, held = case.select()
    gpu.release(held)
    tagged_rows = gpu.upload(halves)
    tagged, picked_tagged, held = case.select(keys=tagged_rows.tagged_bf16())
    assert np.array_equal(bits(plain), bits(tagged)) and np.array_equal(picked, picked_tagged)
    rotated = oracle.rope(c["q"], c["positions"], c["frequencies"])
    assert np.abs(plain[:, :1400] - oracle.index_scores(rotated, halves, c["weights"], c["visible"], c["scale"])[:, :1400]).max() <= 1e-5
    for b in (held, tagged_rows):
        gpu.release(b)
    case.close()


@pytest.mark.parametrize("rows,groups,blocks,block", TWO_LEVEL_CASES + [(2, 20000, 2048, 8)])
def test_the_two_level_indexer_matches_its_reference(gpu, rows, groups, blocks, block):
    source = index_case(rows, groups, spread=13)
    first = Case(gpu, source)
    scores_np, _, scores = first.select()
    chosen, scratch = gpu.buffer(rows * blocks * 4), gpu.buffer(rows * -(-groups // block) * 4)
    gpu.index_candidates(scores.pointer, first.bufs["visible"].pointer, rows, groups, blocks, block, chosen.pointer, scratch)
    got = gpu.read(chosen, np.int32, (rows, blocks))
    assert np.array_equal(got, oracle.index_candidates(scores_np, source["visible"], blocks, block))
    key = f"candidates_{rows}_{groups}_{blocks}_{block}"
    if key in GOLDEN:
        assert np.array_equal(got, GOLDEN[key])
    keep = np.zeros((rows, groups), bool)
    for row in range(rows):
        newest = (source["visible"][row] - 1) // block
        assert newest in got[row], "the block of the last visible group is always kept"
        for b in got[row][got[row] >= 0]:
            keep[row, b * block:(b + 1) * block] = True
    # a later indexer: its choice among the candidates against the top k of its every-group scores with the rest at -inf
    later = index_case(rows, groups, spread=13, seed=1)
    later["keys"] = source["keys"]
    second = Case(gpu, later, keys=first.bufs["keys"])
    every, _, held = second.select()
    gpu.release(held)
    masked = np.where(keep, every, -np.inf).astype(np.float32)
    for run in range(2):
        within_scores, picked, held = second.select(candidates=(chosen.pointer, blocks, block))
        gpu.release(held)
        assert np.array_equal(picked, oracle.top_k(masked, K)), f"run {run}"
        # the scores in candidate order: those of the groups the slots stand for
        for row in range(rows):
            for slot in (0, len(got[row][got[row] >= 0]) - 1):
                b = got[row][slot]
                assert np.array_equal(bits(within_scores[row, slot * block:(slot + 1) * block][:max(0, min(block, groups - b * block))]),
                                      bits(every[row, b * block:(b + 1) * block]))
            assert np.all(np.isneginf(within_scores[row, np.repeat(got[row] < 0, block)]))
    if key in GOLDEN:
        assert np.array_equal(picked, GOLDEN[f"index_within_{rows}_{groups}_{blocks}_{block}"])
    want_scores, want = oracle.index_select(later["q"], later["keys"], later["weights"], later["visible"], later["scale"], later["positions"],
                                            later["frequencies"], K, candidates=got, block=block)
    assert want_scores.shape == within_scores.shape
    for b in (scores, chosen, scratch):
        gpu.release(b)
    first.close()
    second.close()


def test_compress_and_rope_against_the_reference_library_and_the_oracle(gpu):
    c = compress_case()
    kv, gate, out = gpu.upload(c["kv"]), gpu.upload(c["gate"]), gpu.buffer(c["groups"] * c["dim"] * 4)
    gpu.compress(kv.pointer, gate.pointer, c["groups"], c["ratio"], c["dim"], out.pointer)
    got = gpu.read(out, np.float32, (c["groups"], c["dim"]))
    assert np.array_equal(bits(got), bits(GOLDEN["compress"]))
    assert np.abs(got - oracle.compress(c["kv"], c["gate"], c["ratio"])).max() <= 1e-6
    gpu.compress(kv.pointer, None, c["groups"], 1, c["dim"], out.pointer)   # no gate: the rows themselves
    assert np.array_equal(bits(gpu.read(out, np.float32, (c["groups"], c["dim"]))), bits(c["kv"][:c["groups"]]))
    r = index_case(3, 1)
    x, at, fr = gpu.upload(r["q"]), gpu.upload(r["positions"]), gpu.upload(r["frequencies"])
    gpu.rope(x.pointer, 3, r["heads"], r["dim"], r["rope_dims"], at.pointer, fr.pointer)
    turned = gpu.read(x, np.float32, r["q"].shape)
    assert np.array_equal(bits(turned), bits(GOLDEN["rope"]))
    assert np.abs(turned - oracle.rope(r["q"], r["positions"], r["frequencies"])).max() <= 1e-6
    assert np.array_equal(bits(turned[..., :64]), bits(r["q"][..., :64])), "the columns before the rope stay"
    gpu.rope(x.pointer, 3, r["heads"], r["dim"], r["rope_dims"], at.pointer, fr.pointer, inverse=True)
    assert np.abs(gpu.read(x, np.float32, r["q"].shape) - r["q"]).max() <= 1e-6
    for b in (kv, gate, out, x, at, fr):
        gpu.release(b)


@pytest.mark.parametrize("kind,cols,heads,groups,off", INDEX_PROJ_CASES)
def test_index_select_proj_equals_the_reference_librarys(gpu, kind, cols, heads, groups, off):
    # sd_op_index_select_proj (gpu/kernels.cpp:5620-5667): the head weights projected from the row's input in the reference GEMV's order, then
    # sd_op_index_select; weights, scores and indices bit for bit those the reference's own library gave on a B200 (tests/golden/make_golden.py --proj)
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200_proj.npz"))
    c = index_proj_case(kind, cols, heads, groups)
    bufs = {name: gpu.upload(c[name]) for name in ("q", "keys", "visible", "positions", "frequencies", "proj")}
    x = gpu.buffer(cols * 4 + 16)
    gpu.write_buffer(x, off, c["x"])
    weights, scores, picked = gpu.buffer(heads * 4), gpu.buffer(groups * 4), gpu.buffer(512 * 4)
    gpu.index_select_proj(bufs["proj"].pointer, kind, cols, x.pointer + off, bufs["q"].pointer, bufs["keys"].pointer, weights.pointer,
                          bufs["visible"].pointer, groups, heads, c["dim"], c["scale"],
                          (c["rope_dims"], bufs["positions"].pointer, bufs["frequencies"].pointer), scores.pointer, 512, picked.pointer)
    key = f"proj_{kind}_{cols}_{heads}_{groups}_{off}"
    got_weights = gpu.read(weights, np.float32, (heads,))
    assert np.array_equal(bits(got_weights), bits(golden[key + "_weights"]))
    assert np.array_equal(bits(gpu.read(scores, np.float32, (groups,))), bits(golden[key + "_scores"]))
    assert np.array_equal(gpu.read(picked, np.int32, (512,)), golden[key + "_top"])
    # the same call as sd_op_index_select over the projected weights
    scores_2, picked_2 = gpu.buffer(groups * 4), gpu.buffer(512 * 4)
    gpu.index_select(bufs["q"].pointer, bufs["keys"].pointer, weights.pointer, bufs["visible"].pointer, 1, groups, heads, c["dim"], c["scale"],
                     (c["rope_dims"], bufs["positions"].pointer, bufs["frequencies"].pointer), scores_2.pointer, 512, picked_2.pointer)
    assert np.array_equal(gpu.read(picked_2, np.int32, (512,)), golden[key + "_top"])
    for b in list(bufs.values()) + [x, weights, scores, picked, scores_2, picked_2]:
        gpu.release(b)


def test_a_quantised_projection_kind_is_refused_by_name(gpu):
    c = index_proj_case(30, 256, 32, 600)
    bufs = {name: gpu.upload(c[name]) for name in ("q", "keys", "visible", "positions", "frequencies", "proj", "x")}
    weights, scores, picked = gpu.buffer(32 * 4), gpu.buffer(600 * 4), gpu.buffer(512 * 4)

    def call(kind=30, cols=256):
        gpu.index_select_proj(bufs["proj"].pointer, kind, cols, bufs["x"].pointer, bufs["q"].pointer, bufs["keys"].pointer, weights.pointer,
                              bufs["visible"].pointer, 600, 32, c["dim"], c["scale"], (c["rope_dims"], bufs["positions"].pointer, bufs["frequencies"].pointer),
                              scores.pointer, 512, picked.pointer)
    for kind in (8, 12, 13, 42):   # GGML's quantised kinds: the reference's GEMV family, not this library's
        with pytest.raises(StraydogError, match="unsupported Straydog GPU matrix format"):
            call(kind=kind)
    with pytest.raises(StraydogError, match="invalid Straydog index shape"):
        call(cols=8200)
    with pytest.raises(StraydogError, match="outside"):
        call(cols=512)      # a matrix and an input the buffers do not hold
    call()
    for b in list(bufs.values()) + [weights, scores, picked]:
        gpu.release(b)


def test_invalid_index_shapes_are_refused(gpu):
    c = index_case(1, 300)
    case = Case(gpu, c)
    b = case.bufs
    scores, picked = gpu.buffer(300 * 4 * 8), gpu.buffer(K * 4)
    rope = (64, b["positions"].pointer, b["frequencies"].pointer)
    with pytest.raises(StraydogError, match="invalid Straydog index shape"):   # more than 64 heads
        gpu.index_scores(b["q"].pointer, b["keys"].pointer, b["weights"].pointer, b["visible"].pointer, 1, 300, 65, 60, c["scale"], scores.pointer)
    with pytest.raises(StraydogError, match="invalid Straydog index shape"):   # an odd rope
        gpu.index_select(b["q"].pointer, b["keys"].pointer, b["weights"].pointer, b["visible"].pointer, 1, 300, 32, 128, c["scale"],
                         (63, rope[1], rope[2]), scores.pointer, K, picked.pointer)
    with pytest.raises(StraydogError, match="invalid Straydog index candidates"):   # candidates without a block size
        gpu.index_select(b["q"].pointer, b["keys"].pointer, b["weights"].pointer, b["visible"].pointer, 1, 300, 32, 128, c["scale"], rope,
                         scores.pointer, K, picked.pointer, (picked.pointer, 4, 0))
    small = gpu.buffer(16)
    with pytest.raises(StraydogError, match="need more scratch"):
        gpu.index_candidates(scores.pointer, b["visible"].pointer, 1, 300, 8, 8, picked.pointer, small)
    with pytest.raises(StraydogError, match="outside"):   # keys shorter than groups x dim
        gpu.index_scores(b["q"].pointer, b["keys"].pointer, b["weights"].pointer, b["visible"].pointer, 1, 301, 32, 128, c["scale"], scores.pointer)
    for x in (scores, picked, small):
        gpu.release(x)
    case.close()


@pytest.mark.parametrize("heads,dim,half_keys", [(32, 128, False), (64, 128, True), (20, 72, False), (20, 72, True), (7, 16, True), (64, 100, False)])
def test_scores_of_either_kernel_equal_the_oracle(gpu, heads, dim, half_keys):
    """Widths that are whole 16-column steps take the 8 x 8 register-tile kernel, the others the general one; F32 and BF16-tagged keys; a
    number of places that fills no whole tile; rows that see fewer groups than there are."""
    c = index_case(3, 1000, heads=heads, dim=dim, rope_dims=0, spread=129)
    keys = c["keys"]
    if half_keys:
        keys = oracle.to_bf16(keys)
    q, weights, visible = gpu.upload(c["q"]), gpu.upload(c["weights"]), gpu.upload(c["visible"])
    held = gpu.upload(keys)
    scores = gpu.buffer(3 * 1000 * 4)
    gpu.index_scores(q.pointer, held.tagged_bf16() if half_keys else held.pointer, weights.pointer, visible.pointer, 3, 1000, heads, dim, c["scale"], scores.pointer)
    got = gpu.read(scores, np.float32, (3, 1000))
    want = oracle.index_scores(c["q"], keys, c["weights"], c["visible"], c["scale"])
    assert np.array_equal(bits(got), bits(want))
    for x in (q, weights, visible, held, scores):
        gpu.release(x)
