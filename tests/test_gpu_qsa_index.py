"""sdx_qsa_index_select (Qwen's indexer: block scores and the exact top-512 block choice) against the oracle's restatement of
gpu/sparse_attention.hpp:141-243, bit for bit: the scores are chains of fused multiply-adds in column order on both sides and the
choice is integer work. Then the lists it writes drive sdx_qsa_attention_rows."""
import numpy as np
import pytest

import oracle
from straydog_b200.backend import StraydogError
from util import q8_state, qsa_index_case

pytestmark = pytest.mark.gpu


def run(gpu, c, positions=None):
    q, blocks, packed = gpu.upload(c["queries"]), gpu.upload(c["blocks"]), gpu.upload(c["packed"])
    pos = gpu.upload(np.asarray(positions, np.uint32)) if positions is not None else None
    gpu.qsa_index_select(q.pointer, 512, blocks.pointer, c["pool"], c["base"], pos.pointer if pos else None, c["steps"], c["selected"],
                         c["heads"], c["kv_heads"], packed.pointer)
    got = gpu.read(packed, np.float32, c["packed"].shape)
    for b in (q, blocks, pos):
        if b:
            gpu.release(b)
    return got, packed


@pytest.mark.parametrize("steps,base,pool,integers", [(1, 2046, 520, False), (3, 2049, 600, True), (9, 30000, 7600, False), (40, 2000, 1024, True),
                                                      (5, 100, 64, False), (2, 131000, 32800, False)])
def test_lists_and_counts_equal_the_oracles(gpu, steps, base, pool, integers):
    c = qsa_index_case(steps, base, pool, integers=integers)
    want = oracle.qsa_index_select(c["queries"], c["blocks"], base, steps, c["selected"], c["row_floats"], c["packed"].copy())
    got, packed = run(gpu, c)
    start = steps * c["row_floats"]
    assert np.array_equal(got[:start].view(np.uint32), c["packed"][:start].view(np.uint32)), "queries, keys and values stay"
    counts = got[start + steps * c["selected"]:]
    assert np.array_equal(counts, want[start + steps * c["selected"]:])
    for r in range(steps):
        n = int(counts[r])
        at = start + r * c["selected"]
        assert np.array_equal(got[at:at + n], want[at:at + n]), r
        assert np.array_equal(got[at + n:at + c["selected"]].view(np.uint32), c["packed"][at + n:at + c["selected"]].view(np.uint32)), "slots past the count stay"
    gpu.release(packed)


def test_positions_per_row_and_the_lists_feed_the_attention(gpu):
    # verification rows at their own positions; the lists written by the indexer are then attended (the count and every listed
    # position are live by construction), and the result equals the attention over the oracle's lists bit for bit
    steps, pool, context, heads, kv_heads = 4, 1200, 4800, 16, 2
    positions = np.array([4700, 4701, 2047, 4790], np.uint32)
    c = qsa_index_case(steps, 0, pool, heads, kv_heads)
    want = oracle.qsa_index_select(c["queries"], c["blocks"], 0, steps, c["selected"], c["row_floats"], c["packed"].copy(), positions=positions)
    got, packed = run(gpu, c, positions)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    rng = np.random.default_rng(1)
    state = gpu.upload(q8_state(rng, context, kv_heads))
    pos, out = gpu.upload(positions), gpu.buffer(steps * heads * 256 * 4)
    gpu.qsa_attention_rows(state, context, 0, pos.pointer, steps, c["selected"], heads, kv_heads, 0.0625, packed.pointer, out.pointer)
    mine = gpu.read(out, np.uint32, (steps * heads * 256,))
    theirs = gpu.upload(want)
    gpu.qsa_attention_rows(state, context, 0, pos.pointer, steps, c["selected"], heads, kv_heads, 0.0625, theirs.pointer, out.pointer)
    assert np.array_equal(mine, gpu.read(out, np.uint32, (steps * heads * 256,)))
    assert gpu.decode_status() == 0
    for b in (packed, state, pos, out, theirs):
        gpu.release(b)


def test_invalid_indexer_shapes_are_refused(gpu):
    c = qsa_index_case(1, 3000, 800)
    q, blocks, packed = gpu.upload(c["queries"]), gpu.upload(c["blocks"]), gpu.upload(c["packed"])
    for kwargs in (dict(selected=2051), dict(pool=700), dict(query_stride=256), dict(steps=0)):   # a short list, a pool the row outgrows, ...
        a = dict(query_stride=512, pool=800, base=3000, steps=1, selected=2052)
        a.update(kwargs)
        with pytest.raises(StraydogError, match="invalid Straydog indexer dimensions"):
            gpu.qsa_index_select(q.pointer, a["query_stride"], blocks.pointer, a["pool"], a["base"], None, a["steps"], a["selected"], 16, 2, packed.pointer)
    with pytest.raises(StraydogError, match="outside"):
        gpu.qsa_index_select(q.pointer, 512, blocks.pointer, 801, 3000, None, 1, 2052, 16, 2, packed.pointer)
    for b in (q, blocks, packed):
        gpu.release(b)
