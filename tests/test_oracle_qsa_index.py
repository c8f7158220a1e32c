"""The oracle's restatement of Qwen's indexer (orc_qsa_index_select) against an independent numpy statement of the rule, on inputs of
small whole numbers (every sum exact whatever its order, equal scores everywhere: the tie rule decides most of the list)."""
import numpy as np

import oracle
from straydog_b200.synthetic import qsa_index_case


def expected_list(queries, blocks, position):
    complete = (position + 1) // 4
    if complete <= 512:
        return list(range(position + 1))
    dots = np.einsum("hc,cb->hb", queries.reshape(4, 128).astype(np.float64), blocks[:, :complete].astype(np.float64))
    scores = np.maximum(dots, 0).sum(0)
    kept = np.sort(np.argsort(-scores, kind="stable")[:512])   # highest first, equal scores by lowest block
    return [int(b) * 4 + tap for b in kept for tap in range(4)] + list(range(complete * 4, position + 1))


def test_lists_and_counts_follow_the_rule():
    for steps, base, pool in [(3, 2040, 600), (5, 2051, 4000), (2, 30001, 7600), (4, 100, 64)]:
        c = qsa_index_case(steps, base, pool, integers=True)
        before = c["packed"].copy()
        got = oracle.qsa_index_select(c["queries"], c["blocks"], base, steps, c["selected"], c["row_floats"], c["packed"])
        start = steps * c["row_floats"]
        assert np.array_equal(got[:start], before[:start]), "queries, keys and values stay"
        for r in range(steps):
            want = expected_list(c["queries"][r], c["blocks"], base + r)
            count = int(got[start + steps * c["selected"] + r])
            assert count == len(want), (steps, base, r)
            assert np.array_equal(got[start + r * c["selected"]:start + r * c["selected"] + count], np.array(want, np.float32))


def test_positions_may_be_given_per_row():
    c = qsa_index_case(3, 0, 3000, integers=True)
    positions = np.array([2047, 9000, 2052], np.uint32)
    got = oracle.qsa_index_select(c["queries"], c["blocks"], 0, 3, c["selected"], c["row_floats"], c["packed"], positions=positions)
    start = 3 * c["row_floats"]
    for r in range(3):
        want = expected_list(c["queries"][r], c["blocks"], int(positions[r]))
        assert int(got[start + 3 * c["selected"] + r]) == len(want)
        assert np.array_equal(got[start + r * c["selected"]:start + r * c["selected"] + len(want)], np.array(want, np.float32))
