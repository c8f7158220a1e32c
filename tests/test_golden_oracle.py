"""Pins the CPU oracle to outputs of the reference's own GPU library (tests/golden/reference_b200.npz, made by
tests/golden/make_golden.py on a B200): byte and index work bit for bit, attention within FP32 rounding."""
import os

import numpy as np
import pytest

import oracle
from util import (XorShift, attention_sequence_input, bf16_round, latent_decode_case, op_attention_case, q8_state,
                  sparse_attention_case, tie_scores)

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz"))
SEQUENCE_CASES = [(4, 2052, 3000, 4096, "sparse"), (3, 64, 100, 256, "dense"), (8, 513, 20, 64, "sparse")]
ATTENTION_CASES = [(15, 16, 2, 256, 137), (1, 2, 1, 256, 137), (17, 4, 2, 256, 35), (16, 4, 2, 128, 35)]


def worst(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max())


@pytest.mark.parametrize("steps,selected,base,context,kind", SEQUENCE_CASES)
def test_attention_sequence(steps, selected, base, context, kind):
    rng = np.random.default_rng(steps * 1000 + selected)
    state = q8_state(rng, context, 2, filled=base)
    inp = attention_sequence_input(rng, steps, selected, base, context, kind)
    got = oracle.attention_sequence(state, context, 24, 2, base, steps, selected, inp)
    key = f"sequence_{steps}_{selected}_{base}_{context}_{kind}"
    assert np.array_equal(state[:, base:base + steps], GOLDEN[key + "_rows"]), "the Q8_0 rows the call writes: bit for bit"
    assert worst(got, GOLDEN[key]) < 2e-5


@pytest.mark.parametrize("rows,heads,kv_heads,dim,context", ATTENTION_CASES)
def test_op_attention(rows, heads, kv_heads, dim, context):
    c = op_attention_case(rows, heads, kv_heads, dim, context)
    for gated in (0, 1):
        out, out64, bound = oracle.op_attention(c["q"], c["keys"], c["values"], context, c["positions"], rows, heads, kv_heads, dim, c["scale"],
                                                c["gate"] if gated else None, want64=True)
        ref = GOLDEN[f"attention_{rows}_{heads}_{kv_heads}_{dim}_{context}_{gated}"]
        # the reference's own kernels sit inside the bound its test derives around the oracle's F64 values
        assert np.all(np.abs(ref.astype(np.float64) - out64) <= bound)
        assert worst(out, ref) < 1e-5


@pytest.mark.parametrize("rows,heads", [(1, 32), (4, 32)])
def test_sparse_attention(rows, heads):
    c = sparse_attention_case(rows, heads)
    got = oracle.sparse_attention(c["q"], c["raw"], c["raw_rows"], c["positions"], c["window"], c["halves"], c["selected"], c["selections"],
                                  c["sinks"], rows, heads, c["dim"], c["scale"], c["rope_dims"], c["freq"])
    assert worst(got, GOLDEN[f"sparse_{rows}_{heads}"]) < 2e-5


def test_latent_decode_shape():
    seed, rows, heads, dim, context, selections = 11, 2, 16, 576, 1024, 256
    c = latent_decode_case(seed, rows, heads, dim, context, selections)
    got = oracle.sparse_attention(c["q"], c["raw"], c["raw_rows"], c["positions"], c["window"], c["halves"], c["selected"], selections,
                                  c["sinks"], rows, heads, dim, c["scale"], 0, None)
    assert worst(got, GOLDEN[f"latent_{seed}_{rows}_{heads}_{dim}_{context}_{selections}"]) < 2e-6


def test_top_k_and_bf16_bit_for_bit():
    random = XorShift(0x2F6B91D3C0A54E77)
    for groups in [511, 512, 513, 600, 4096, 30000]:
        scores = tie_scores(random, 2, groups)
        assert np.array_equal(oracle.top_k(scores, 512), GOLDEN[f"topk_{groups}"]), groups
    values = XorShift(0x243F6A8885A308D3).floats_scaled(10_000, 1e3)
    assert np.array_equal(oracle.to_bf16(values), GOLDEN["to_bf16"])
    assert np.array_equal(bf16_round(values)[0], GOLDEN["to_bf16"])


def test_dspark_attention():
    from util import dspark_case
    c = dspark_case()
    for slots, history, anchor in [(1, 0, 0), (5, 37, 149), (3, 128, 389)]:
        got = oracle.dspark_attention(c["q"][:slots], c["ring"], c["block"], c["sinks"], 64, slots, anchor, history)
        assert worst(got[:, ::8], GOLDEN[f"dspark_{slots}_{history}_{anchor}"]) < 2e-6   # (the fixture holds every eighth head)


def test_the_indexer():
    """Scores within the rope's sin and cos of the reference library's (the CPU's libm against the device's); everything after the scores
    (the choice of indices, the candidate blocks, the choice among them) bit for bit from the library's own scores."""
    from util import INDEX_CASES, TWO_LEVEL_CASES, compress_case, index_case
    for rows, groups in INDEX_CASES:
        c = index_case(rows, groups)
        scores, picked = oracle.index_select(c["q"], c["keys"], c["weights"], c["visible"], c["scale"], c["positions"], c["frequencies"], 512)
        want = GOLDEN[f"index_scores_{rows}_{groups}"]
        seen = np.isfinite(want)
        assert np.array_equal(seen, np.isfinite(scores)) and worst(scores[seen], want[seen]) <= 1e-5
        assert np.array_equal(oracle.top_k(want, 512), GOLDEN[f"index_top_{rows}_{groups}"])
    for rows, groups, blocks, block in TWO_LEVEL_CASES:
        source = index_case(rows, groups, spread=13)
        scores, _ = oracle.index_select(source["q"], source["keys"], source["weights"], source["visible"], source["scale"], source["positions"],
                                        source["frequencies"], 512)
        chosen = GOLDEN[f"candidates_{rows}_{groups}_{blocks}_{block}"]
        mine = oracle.index_candidates(scores, source["visible"], blocks, block)
        # a block's highest score an ulp apart could swap two blocks at the cut: allow a few, demand the rest
        assert np.mean(mine == chosen) > 0.99
        later = index_case(rows, groups, spread=13, seed=1)
        _, picked = oracle.index_select(later["q"], source["keys"], later["weights"], later["visible"], later["scale"], later["positions"],
                                        later["frequencies"], 512, candidates=chosen, block=block)
        want = GOLDEN[f"index_within_{rows}_{groups}_{blocks}_{block}"]
        assert np.mean(picked == want) > 0.98
        assert np.all(np.diff(picked.astype(np.int64), axis=1)[picked[:, 1:] >= 0] > 0), "ascending group indices"
    c = compress_case()
    assert worst(oracle.compress(c["kv"], c["gate"], c["ratio"]), GOLDEN["compress"]) <= 1e-6
    r = index_case(3, 1)
    assert worst(oracle.rope(r["q"], r["positions"], r["frequencies"]), GOLDEN["rope"]) <= 1e-6


def test_the_projection_of_index_select_proj():
    # the head weights sd_op_index_select_proj projects (the reference GEMV's order of summation), bit for bit the reference library's
    # on a B200; then the scores and indices from them as in test_the_indexer
    from straydog_b200.synthetic import INDEX_PROJ_CASES, index_proj_case
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200_proj.npz"))
    for kind, cols, heads, groups, off in INDEX_PROJ_CASES:
        c = index_proj_case(kind, cols, heads, groups)
        key = f"proj_{kind}_{cols}_{heads}_{groups}_{off}"
        got = oracle.index_proj(c["proj"], kind, c["x"], units=(cols % (4 if kind == 0 else 8) == 0 and off == 0))
        assert np.array_equal(got.view(np.uint32), golden[key + "_weights"].view(np.uint32)), key
        assert np.array_equal(oracle.top_k(golden[key + "_scores"][None], 512)[0], golden[key + "_top"]), key


def test_the_qwen_layer_behind_its_projections():
    # tests/golden/reference_b200_qsa.npz: what the reference's sd_qsa_sequence left behind over selection matrices (make_golden.py --qsa).
    # The oracle's restatement of the front and of the indexer against it: the value rows and the ring bit for bit; the key rows and the
    # pooled blocks through the host's powf / cosf / sinf (a last place of theirs moves a rotated value by position * 6e-8); the lists the
    # rule gives over the reference's block scores equal the oracle's
    from straydog_b200.synthetic import QSA_SEQUENCE_CASES, qsa_sequence_case
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200_qsa.npz"))
    for context, position, steps, seed in QSA_SEQUENCE_CASES:
        c = qsa_sequence_case(context, position, steps, seed)
        key = f"qsa_{context}_{position}_{steps}_{seed}"
        selected, row_floats = 2052, 24 * 256 + 2 * 512
        packed = np.zeros(steps * (row_floats + selected + 1), np.float32)
        state, index_state, iq = c["state"].view(np.uint8).ravel().copy(), c["index_state"].copy(), c["iq"].copy()
        oracle.qsa_normalize_chunk(c["qgate"], c["key"], c["value"], iq, c["ik"], position, 24, 2, *c["norms"], packed, state, context, index_state)
        rows, want = state.reshape(4, context, 272)[:, position:position + steps], golden[key + "_rows"]
        assert np.array_equal(rows[2:], want[2:]), "value rows"
        mine = oracle.q8_decode_rows(np.ascontiguousarray(rows[:2]).reshape(-1, 272))
        theirs = oracle.q8_decode_rows(np.ascontiguousarray(want[:2]).reshape(-1, 272))
        assert np.abs(mine - theirs).max() < 0.06, "key rows: a quantisation step apart at most"
        pool = c["pool"]
        assert np.array_equal(index_state[pool * 128:].view(np.uint32), golden[key + "_ring"].view(np.uint32))
        blocks = index_state[:pool * 128].reshape(128, pool)[:, position // 4:(position + steps) // 4]
        assert blocks.shape == golden[key + "_blocks"].shape and (not blocks.size or np.abs(blocks - golden[key + "_blocks"]).max() < 5e-3)
        if key + "_scores" in golden:
            # the oracle's choice over the reference's own blocks (so that the scores are the same numbers): its lists are the rule's over the
            # reference's scores
            index_ref = c["index_state"].copy()
            index_ref[:pool * 128].reshape(128, pool)[:, position // 4:(position + steps) // 4] = golden[key + "_blocks"]
            queries_ref = iq.reshape(steps, 512)
            lists = oracle.qsa_index_select(queries_ref, index_ref[:pool * 128].reshape(128, pool), position, steps, selected, row_floats, packed.copy())
            start = steps * row_floats
            for t in range(steps):
                complete = (position + t + 1) // 4
                scores = golden[key + "_scores"][t, :complete].astype(np.float64)
                kept = np.sort(np.argsort(-scores, kind="stable")[:512])
                listed = np.concatenate([(kept[:, None] * 4 + np.arange(4)).ravel(), np.arange(complete * 4, position + t + 1)])
                count = int(lists[start + steps * selected + t])
                got = lists[start + t * selected:start + t * selected + count]
                # (the oracle's index queries went through the host's cosf: a block at the 512th score may change places with its neighbour)
                assert count == len(listed) and len(set(got.astype(np.int64)) ^ set(listed)) <= 16, t
