"""The oracle's indexer functions against independent numpy restatements (F64 where the arithmetic is floating point)."""
import numpy as np

import oracle
from straydog_b200.synthetic import compress_case, index_case


def test_scores_follow_the_formula_and_stop_at_the_visible_count():
    c = index_case(3, 700, spread=50)
    rotated = oracle.rope(c["q"], c["positions"], c["frequencies"])
    got = oracle.index_scores(rotated, c["keys"], c["weights"], c["visible"], c["scale"])
    dots = np.einsum("rhd,gd->rhg", rotated.astype(np.float64), c["keys"].astype(np.float64))
    want = (np.maximum(dots, 0) * c["weights"].astype(np.float64)[:, :, None]).sum(1) * c["scale"]
    for row in range(3):
        seen = c["visible"][row]
        assert np.abs(got[row, :seen] - want[row, :seen]).max() < 1e-5
        assert np.all(np.isneginf(got[row, seen:]))
    halves = oracle.to_bf16(c["keys"])
    assert np.array_equal(oracle.index_scores(rotated, halves, c["weights"], c["visible"], c["scale"]).view(np.uint32),
                          oracle.index_scores(rotated, oracle.bf16_to_f32(halves), c["weights"], c["visible"], c["scale"]).view(np.uint32))


def test_rope_turns_the_last_columns_in_pairs():
    c = index_case(2, 1)
    got = oracle.rope(c["q"], c["positions"], c["frequencies"])
    assert np.array_equal(got[..., :64], c["q"][..., :64])
    angle = c["positions"].astype(np.float64)[:, None] * c["frequencies"].astype(np.float64)[None, :]
    a, b = c["q"][..., 64::2].astype(np.float64), c["q"][..., 65::2].astype(np.float64)
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    assert np.array_equal(got[..., 64::2], (a * cos - b * sin).astype(np.float32))
    assert np.array_equal(got[..., 65::2], (a * sin + b * cos).astype(np.float32))
    assert np.abs(oracle.rope(got, c["positions"], c["frequencies"], inverse=True) - c["q"]).max() < 1e-6


def test_candidates_keep_the_newest_block_and_the_best_of_the_rest():
    rng = np.random.default_rng(3)
    scores = rng.normal(size=(2, 1001)).astype(np.float32)
    visible = np.array([1001, 640], np.int32)
    scores[1, 640:] = -np.inf
    got = oracle.index_candidates(scores, visible, 16, 8)
    for row in range(2):
        tops = np.array([scores[row, b * 8:(b + 1) * 8].max() for b in range(126)])
        newest = (visible[row] - 1) // 8
        tops[newest] = np.inf
        want = np.sort(np.argsort(-tops, kind="stable")[:16])
        assert np.array_equal(got[row], want)
        assert newest in got[row]
    # fewer blocks with a finite score than slots: every one kept, -1 after them
    few = oracle.index_candidates(scores[1:, :64], np.array([64], np.int32), 16, 8)
    assert np.array_equal(few[0], np.r_[np.arange(8), np.full(8, -1)])


def test_a_choice_among_candidates_is_the_masked_top_k():
    c = index_case(2, 900, spread=13)
    scores, _ = oracle.index_select(c["q"], c["keys"], c["weights"], c["visible"], c["scale"], c["positions"], c["frequencies"], 64)
    chosen = oracle.index_candidates(scores, c["visible"], 20, 8)
    within, picked = oracle.index_select(c["q"], c["keys"], c["weights"], c["visible"], c["scale"], c["positions"], c["frequencies"], 64,
                                         candidates=chosen, block=8)
    assert within.shape == (2, 160)
    keep = np.zeros_like(scores, bool)
    for row in range(2):
        for b in chosen[row][chosen[row] >= 0]:
            keep[row, b * 8:(b + 1) * 8] = True
    assert np.array_equal(picked, oracle.top_k(np.where(keep, scores, -np.inf).astype(np.float32), 64))


def test_compress_is_a_softmax_pool():
    c = compress_case()
    got = oracle.compress(c["kv"], c["gate"], c["ratio"])
    g = c["gate"].reshape(c["groups"], c["ratio"], c["dim"]).astype(np.float64)
    w = np.exp(g - g.max(1, keepdims=True))
    want = (w * c["kv"].reshape(g.shape)).sum(1) / w.sum(1)
    assert np.abs(got - want).max() < 1e-6
    assert np.array_equal(oracle.compress(c["kv"][:c["groups"]], None, 1), c["kv"][:c["groups"]])
