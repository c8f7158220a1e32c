"""Generates tests/golden/*.npz by running the REFERENCE's own GPU library (oracle/_ref/libstraydog_ref.so,
built from the reference's unmodified sources by oracle/Makefile.ref) through its C ABI on a B200.

    python tests/golden/make_golden.py          # on a machine with a GPU and oracle/_ref built
    python tests/golden/make_golden.py --proj   # reference_b200_proj.npz alone: sd_op_index_select_proj over plain weight kinds
    python tests/golden/make_golden.py --qsa    # reference_b200_qsa.npz alone: sd_qsa_sequence (a whole Qwen attention layer) over selection matrices

Inputs are rebuilt from seeds by straydog_b200.synthetic (the fixtures hold outputs only, plus the few
state rows a call writes), so the fixtures stay small. The tests compare the CPU oracle and this
library's kernels against them.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from straydog_b200 import _lib, synthetic  # noqa: E402
from straydog_b200.backend import Backend  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(ROOT, "oracle", "_ref", "libstraydog_ref.so")

SEQUENCE_CASES = [(4, 2052, 3000, 4096, "sparse"), (3, 64, 100, 256, "dense"), (8, 513, 20, 64, "sparse")]
ATTENTION_CASES = [(15, 16, 2, 256, 137), (1, 2, 1, 256, 137), (17, 4, 2, 256, 35), (16, 4, 2, 128, 35)]
SPARSE_CASES = [(1, 32), (4, 32)]
LATENT_CASES = [(11, 2, 16, 576, 1024, 256)]
DSPARK_CASES = [(1, 0, 0), (5, 37, 149), (3, 128, 389)]
TOPK_GROUPS = [511, 512, 513, 600, 4096, 30000]


def proj_main():
    """sd_op_index_select_proj of the reference's library for synthetic.INDEX_PROJ_CASES: the projected head weights, the scores and the
    chosen indices (k = 512) of one row each."""
    gpu = Backend(0, 2 << 30, library=_lib.load(REF, reference_abi_only=True))
    out = {}
    for kind, cols, heads, groups, off in synthetic.INDEX_PROJ_CASES:
        c = synthetic.index_proj_case(kind, cols, heads, groups)
        bufs = {name: gpu.upload(c[name]) for name in ("q", "keys", "visible", "positions", "frequencies", "proj")}
        x = gpu.buffer(cols * 4 + 16)
        gpu.write_buffer(x, off, c["x"])
        weights, scores, picked = gpu.buffer(heads * 4), gpu.buffer(groups * 4), gpu.buffer(512 * 4)
        gpu.index_select_proj(bufs["proj"].pointer, kind, cols, x.pointer + off, bufs["q"].pointer, bufs["keys"].pointer, weights.pointer,
                              bufs["visible"].pointer, groups, heads, c["dim"], c["scale"],
                              (c["rope_dims"], bufs["positions"].pointer, bufs["frequencies"].pointer), scores.pointer, 512, picked.pointer)
        key = f"proj_{kind}_{cols}_{heads}_{groups}_{off}"
        out[key + "_weights"] = gpu.read(weights, np.float32, (heads,))
        out[key + "_scores"] = gpu.read(scores, np.float32, (groups,))
        out[key + "_top"] = gpu.read(picked, np.int32, (512,))
        for b in list(bufs.values()) + [x, weights, scores, picked]:
            gpu.release(b)
    gpu.close()
    target = os.environ.get("GOLDEN_OUT", os.path.join(HERE, "reference_b200_proj.npz"))
    np.savez_compressed(target, **out)
    print(f"wrote {target}: {len(out)} arrays, {os.path.getsize(target)} bytes")


def qsa_main():
    """sd_qsa_sequence of the reference's library (gpu/sparse_attention.hpp:441-512: projections, normalisation, pooling, block scores, block
    choice, K/V write, selection attention, gate, output projection) for synthetic.QSA_SEQUENCE_CASES. The six weight matrices are F32
    selection matrices (a 1 a row), so the projections are exact copies of input columns and the output is the first ten heads' gated
    attention: what the fixture holds is the reference's kernels' arithmetic behind the projections: the K/V rows the call wrote, the indexer
    state's new columns and its ring, the block scores of the rows (where the choice ran) and the output."""
    import ctypes as C
    lib = _lib.load(REF, reference_abi_only=True)
    lib.sd_qsa_sequence.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64,
                                    C.c_uint64, C.c_void_p, C.c_void_p]
    lib.sd_qsa_sequence.restype = C.c_int
    gpu = Backend(0, 6 << 30, library=lib)
    gpu.kv_format(272)
    matrices = [gpu.upload(synthetic.qsa_selection_matrix(name)) for name in ("qgate", "key", "value", "iq", "ik")] + [gpu.upload(synthetic.qsa_output_matrix())]
    out = {}
    for context, position, steps, seed in synthetic.QSA_SEQUENCE_CASES:
        c = synthetic.qsa_sequence_case(context, position, steps, seed)
        norms = [gpu.upload(n) for n in c["norms"]]
        state = gpu.allocate(c["state"].nbytes)
        gpu.write(state, c["state"])
        index, scratch = gpu.upload(c["index_state"]), gpu.buffer(256 * c["pool"] * 4)
        pointers = (C.c_void_p * 10)(*[b.pointer for b in matrices + norms])
        kinds = (C.c_int * 10)(*([0] * 10))
        result = np.empty((steps, synthetic.QSA_HIDDEN), np.float32)
        gpu._c(lib.sd_qsa_sequence(gpu.handle, pointers, kinds, state.pointer, index.pointer, scratch.pointer, context, position, steps,
                                   c["x"].ctypes.data_as(C.c_void_p), result.ctypes.data_as(C.c_void_p)))
        key = f"qsa_{context}_{position}_{steps}_{seed}"
        after = gpu.download(state, np.empty_like(c["state"])).reshape(4, context, 272)
        out[key + "_rows"] = after[:, position:position + steps].copy()
        untouched = np.ones(context, bool)
        untouched[position:position + steps] = False
        assert np.array_equal(after[:, untouched], c["state"].reshape(4, context, 272)[:, untouched])
        index_after = gpu.read(index, np.float32, c["index_state"].shape)
        first, last = position // 4, (position + steps) // 4
        out[key + "_blocks"] = index_after[:c["pool"] * 128].reshape(128, c["pool"])[:, first:last].copy()
        out[key + "_ring"] = index_after[c["pool"] * 128:].copy()
        if (position + steps) // 4 > 512:   # the block choice ran: the rows' block scores (a row's first (its position + 1) / 4 entries count)
            out[key + "_scores"] = gpu.read(scratch, np.float32, (steps, c["pool"]))[:, :(position + steps) // 4].copy()
        out[key + "_out"] = result
        for b in norms + [state, index, scratch]:
            gpu.release(b)
    gpu.close()
    target = os.environ.get("GOLDEN_OUT", os.path.join(HERE, "reference_b200_qsa.npz"))
    np.savez_compressed(target, **out)
    print(f"wrote {target}: {len(out)} arrays, {os.path.getsize(target)} bytes")


def main():
    gpu = Backend(0, 2 << 30, library=_lib.load(REF, reference_abi_only=True))
    gpu.kv_format(272)   # the reference defaults to FP16 rows until told otherwise (gpu/core.hpp:837)
    out = {}
    for steps, selected, base, context, kind in SEQUENCE_CASES:
        rng = np.random.default_rng(steps * 1000 + selected)
        state_np = synthetic.q8_state(rng, context, 2, filled=base)
        inp = synthetic.attention_sequence_input(rng, steps, selected, base, context, kind)
        state = gpu.allocate(state_np.nbytes)
        gpu.write(state, state_np)
        got = gpu.attention_sequence(state, context, base, steps, selected, inp)
        after = gpu.download(state, np.empty_like(state_np))
        key = f"sequence_{steps}_{selected}_{base}_{context}_{kind}"
        out[key] = got
        out[key + "_rows"] = after[:, base:base + steps].copy()
        gpu.release(state)
    for rows, heads, kv_heads, dim, context in ATTENTION_CASES:
        c = synthetic.op_attention_case(rows, heads, kv_heads, dim, context)
        qs, ks, vs, gs, ps = (gpu.upload(c[k]) for k in ("q", "keys", "values", "gate", "positions"))
        scratch = gpu.buffer(rows * heads * 64 * (dim + 2) * 4)
        o = gpu.buffer(c["q"].size * 4)
        for gated in (False, True):
            gpu.attention(qs.pointer, ks.pointer, vs.pointer, context, ps.pointer, rows, heads, kv_heads, dim, c["scale"],
                          gs.pointer if gated else None, scratch, o.pointer)
            out[f"attention_{rows}_{heads}_{kv_heads}_{dim}_{context}_{int(gated)}"] = gpu.read(o, np.float32, (rows, heads, dim))
        for b in (qs, ks, vs, gs, ps, scratch, o):
            gpu.release(b)

    def sparse(c, compressed_np, tagged):
        bufs = {k: gpu.upload(c[k]) for k in ("q", "raw", "sinks", "freq", "positions", "selected")}
        comp = gpu.upload(compressed_np)
        o = gpu.buffer(c["rows"] * c["heads"] * c["dim"] * 4)
        scratch = gpu.buffer(256 << 20)
        gpu.attention_turns_reserve(c["rows"], c["rope_dims"])
        gpu.sparse_attention(bufs["q"].pointer, bufs["raw"].pointer, c["raw_rows"], bufs["positions"].pointer, c["window"],
                             (comp.tagged_bf16() if tagged else comp.pointer, c["compressed_rows"]), (bufs["selected"].pointer, c["selections"]),
                             bufs["sinks"].pointer, c["rows"], c["heads"], c["dim"], c["scale"],
                             (c["rope_dims"], bufs["freq"].pointer) if c["rope_dims"] else None, scratch, o.pointer)
        got = gpu.read(o, np.float32, (c["rows"], c["heads"], c["dim"]))
        for b in list(bufs.values()) + [comp, o, scratch]:
            gpu.release(b)
        return got
    for rows, heads in SPARSE_CASES:
        c = synthetic.sparse_attention_case(rows, heads)
        tagged = sparse(c, c["halves"], True)
        plain = sparse(c, c["widened"], False)
        assert np.array_equal(tagged.view(np.uint32), plain.view(np.uint32)), "the reference's own BF16 = F32 contract"
        out[f"sparse_{rows}_{heads}"] = tagged
    for seed, rows, heads, dim, context, selections in LATENT_CASES:
        c = synthetic.latent_decode_case(seed, rows, heads, dim, context, selections)
        c["sinks"] = np.full(heads, -1e30, np.float32)   # exp(sink - top) = 0 either way
        out[f"latent_{seed}_{rows}_{heads}_{dim}_{context}_{selections}"] = sparse(c, c["halves"], True)
    random = synthetic.XorShift(0x2F6B91D3C0A54E77)
    for groups in TOPK_GROUPS:
        scores = synthetic.tie_scores(random, 2, groups)
        dev = gpu.upload(scores)
        o = gpu.buffer(2 * 512 * 4)
        gpu.top_k(dev.pointer, 2, groups, 512, o.pointer)
        out[f"topk_{groups}"] = gpu.read(o, np.int32, (2, 512))
        gpu.release(dev)
        gpu.release(o)
    c = synthetic.dspark_case()
    q, ring, block, sinks = (gpu.upload(c[k]) for k in ("q", "ring", "block", "sinks"))
    o = gpu.buffer(c["q"].nbytes)
    for slots, history, anchor in DSPARK_CASES:
        gpu.dspark_attention(q.pointer, ring, block.pointer, sinks, 64, slots, anchor, None, history, o.pointer)
        out[f"dspark_{slots}_{history}_{anchor}"] = gpu.read(o, np.float32, (slots, 64, 512))[:, ::8].copy()   # every eighth head keeps the file small
    for b in (q, ring, block, sinks, o):
        gpu.release(b)

    def index_select(c, k, candidates=None):
        bufs = {name: gpu.upload(c[name]) for name in ("q", "keys", "weights", "visible", "positions", "frequencies")}
        scored = c["groups"] if candidates is None else candidates[1] * candidates[2]
        scores, picked = gpu.buffer(c["rows"] * max(scored, c["groups"]) * 4), gpu.buffer(c["rows"] * k * 4)
        gpu.index_select(bufs["q"].pointer, bufs["keys"].pointer, bufs["weights"].pointer, bufs["visible"].pointer, c["rows"], c["groups"],
                         c["heads"], c["dim"], c["scale"], (c["rope_dims"], bufs["positions"].pointer, bufs["frequencies"].pointer),
                         scores.pointer, k, picked.pointer, candidates)
        got = gpu.read(scores, np.float32, (c["rows"], scored)), gpu.read(picked, np.int32, (c["rows"], k))
        for b in list(bufs.values()) + [picked]:
            gpu.release(b)
        return got + (scores,)
    for rows, groups in synthetic.INDEX_CASES:
        c = synthetic.index_case(rows, groups)
        scores, picked, held = index_select(c, 512)
        gpu.release(held)
        out[f"index_scores_{rows}_{groups}"], out[f"index_top_{rows}_{groups}"] = scores, picked
    for rows, groups, blocks, block in synthetic.TWO_LEVEL_CASES:
        source = synthetic.index_case(rows, groups, spread=13)
        _, _, scores = index_select(source, 512)
        visible, chosen = gpu.upload(source["visible"]), gpu.buffer(rows * blocks * 4)
        scratch = gpu.buffer(rows * -(-groups // block) * 4)
        gpu.index_candidates(scores.pointer, visible.pointer, rows, groups, blocks, block, chosen.pointer, scratch)
        out[f"candidates_{rows}_{groups}_{blocks}_{block}"] = gpu.read(chosen, np.int32, (rows, blocks))
        later = synthetic.index_case(rows, groups, spread=13, seed=1)
        later["keys"] = source["keys"]
        _, picked, held = index_select(later, 512, (chosen.pointer, blocks, block))
        out[f"index_within_{rows}_{groups}_{blocks}_{block}"] = picked
        for b in (scores, visible, chosen, scratch, held):
            gpu.release(b)
    c = synthetic.compress_case()
    kv, gate, o = gpu.upload(c["kv"]), gpu.upload(c["gate"]), gpu.buffer(c["groups"] * c["dim"] * 4)
    gpu.compress(kv.pointer, gate.pointer, c["groups"], c["ratio"], c["dim"], o.pointer)
    out["compress"] = gpu.read(o, np.float32, (c["groups"], c["dim"]))
    c = synthetic.index_case(3, 1)
    x, at, fr = gpu.upload(c["q"]), gpu.upload(c["positions"]), gpu.upload(c["frequencies"])
    gpu.rope(x.pointer, 3, c["heads"], c["dim"], c["rope_dims"], at.pointer, fr.pointer)
    out["rope"] = gpu.read(x, np.float32, c["q"].shape)
    values = synthetic.XorShift(0x243F6A8885A308D3).floats_scaled(10_000, 1e3)
    dev = gpu.upload(values)
    o = gpu.buffer(values.size * 2)
    gpu.to_bf16(dev.pointer, values.size, o.pointer)
    out["to_bf16"] = gpu.read(o, np.uint16, (values.size,))
    gpu.close()
    target = os.environ.get("GOLDEN_OUT", os.path.join(HERE, "reference_b200.npz"))
    np.savez_compressed(target, **out)
    print(f"wrote {target}: {len(out)} arrays, {os.path.getsize(target)} bytes")


if __name__ == "__main__":
    proj_main() if "--proj" in sys.argv else qsa_main() if "--qsa" in sys.argv else main()
