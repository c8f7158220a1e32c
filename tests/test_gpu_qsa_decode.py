"""Split-K Q8_0 GQA decode (sdx_qsa_decode, sdx_qsa_plan*, sdx_attention_batch) against the oracle."""
import numpy as np
import pytest

import oracle
from util import close, q8_state, queries_f16

pytestmark = pytest.mark.gpu
CANARY = np.float32(12345.125)
GUARD = 7


def run_decode(gpu, states_np, contexts, lengths, heads, kv_heads, q, scale=1 / 16, plan=False):
    n = len(states_np)
    states = [gpu.upload(s) for s in states_np]
    q_dev = gpu.upload(q)
    out = gpu.upload(np.full(n * heads * 256 + 2 * GUARD, CANARY, np.float32))
    if plan:
        p = gpu.qsa_plan(states, contexts, lengths, heads, kv_heads)
        gpu.qsa_plan_run(p, scale, q_dev.pointer, out.at(GUARD * 4))
        gpu.qsa_plan_run(p, scale, q_dev.pointer, out.at(GUARD * 4))   # a plan replays
        gpu.qsa_plan_release(p)
    else:
        gpu.qsa_decode(states, contexts, lengths, heads, kv_heads, scale, q_dev.pointer, out.at(GUARD * 4))
    got = gpu.read(out, np.float32, (n * heads * 256 + 2 * GUARD,))
    assert gpu.decode_status() == 0
    assert np.all(got[:GUARD] == CANARY) and np.all(got[-GUARD:] == CANARY), "output guard"
    for b in states + [q_dev, out]:
        gpu.release(b)
    return got[GUARD:-GUARD].reshape(n, heads, 256)


def expect_decode(states_np, contexts, lengths, heads, kv_heads, q, scale=1 / 16, f64=True):
    return np.stack([oracle.gqa_decode_q8(states_np[s], contexts[s], lengths[s], heads, kv_heads, q[s], scale, f64=f64)
                     for s in range(len(states_np))])


def test_config0_single_sequence_4096(gpu):
    rng = np.random.default_rng(100)
    state = q8_state(rng, 4096, 2)
    q = queries_f16(rng, 1, 16, 256)
    got = run_decode(gpu, [state], [4096], [4096], 16, 2, q)
    want = expect_decode([state], [4096], [4096], 16, 2, q)
    ok, worst = close(got, want)
    assert ok, worst
    # much tighter than the stated tolerance: FP32 accumulation of exact products
    assert worst < 2e-4, worst
    want32 = expect_decode([state], [4096], [4096], 16, 2, q, f64=False)
    assert close(got, want32)[0]


@pytest.mark.parametrize("length", [1, 2, 15, 16, 17, 31, 32, 33, 127, 128, 129, 1000])
def test_edge_lengths(gpu, length):
    rng = np.random.default_rng(200 + length)
    context = 1024
    state = q8_state(rng, context, 2)
    # rows past the length hold bytes that must not leak in (scales that are NaN/Inf as FP16)
    state[:, length:, :] = 0xFF
    q = queries_f16(rng, 1, 16, 256)
    got = run_decode(gpu, [state], [context], [length], 16, 2, q)
    want = expect_decode([state], [context], [length], 16, 2, q)
    ok, worst = close(got, want)
    assert ok, (length, worst)


@pytest.mark.parametrize("heads,kv_heads", [(1, 1), (2, 2), (4, 2), (8, 1), (16, 2), (12, 3), (32, 4)])
def test_head_groupings(gpu, heads, kv_heads):
    rng = np.random.default_rng(300 + heads)
    state = q8_state(rng, 400, kv_heads)
    q = queries_f16(rng, 1, heads, 256)
    got = run_decode(gpu, [state], [400], [333], heads, kv_heads, q, scale=0.05)
    want = expect_decode([state], [400], [333], heads, kv_heads, q, scale=0.05)
    ok, worst = close(got, want)
    assert ok, worst


def test_ragged_batch_and_plan_replay(gpu):
    rng = np.random.default_rng(400)
    lengths = [int(x) for x in rng.integers(1, 3000, 12)]
    contexts = [l + int(x) for l, x in zip(lengths, rng.integers(0, 50, 12))]
    states = [q8_state(rng, c, 2) for c in contexts]
    q = queries_f16(rng, 12, 16, 256)
    want = expect_decode(states, contexts, lengths, 16, 2, q)
    got = run_decode(gpu, states, contexts, lengths, 16, 2, q)
    ok, worst = close(got, want)
    assert ok, worst
    got_plan = run_decode(gpu, states, contexts, lengths, 16, 2, q, plan=True)
    assert np.array_equal(got_plan.view(np.uint32), got.view(np.uint32)), "a plan's run equals the direct call"


def test_a_sequence_result_does_not_depend_on_its_batch(gpu):
    # the reference's verification contract (lines 40-41 of the reference's own design notes under docs/) asks a row's bits to be those of a one-token decode. With the
    # default moving cuts the split points move with the batch, so the value is the same to FP32 rounding; with fixed cuts
    # (sdx_decode_cuts) a sequence is cut by its own length alone and the bits are the same in any batch.
    rng = np.random.default_rng(500)
    lengths = [700, 64, 9000, 333, 1]
    states = [q8_state(rng, l, 2) for l in lengths]
    q = queries_f16(rng, len(lengths), 16, 256)
    want = expect_decode(states, lengths, lengths, 16, 2, q)
    for fixed in (False, True):
        gpu.decode_cuts(fixed)
        try:
            together = run_decode(gpu, states, lengths, lengths, 16, 2, q)
            ok, worst = close(together, want)
            assert ok and worst < 5e-4, (fixed, worst)
            for s in range(len(lengths)):
                alone = run_decode(gpu, [states[s]], [lengths[s]], [lengths[s]], 16, 2, q[s:s + 1])
                pair = run_decode(gpu, [states[s], states[2]], [lengths[s], lengths[2]], [lengths[s], lengths[2]], 16, 2, q[[s, 2]], plan=True)
                if fixed:
                    assert np.array_equal(alone[0].view(np.uint32), together[s].view(np.uint32)), s
                    assert np.array_equal(pair[0].view(np.uint32), together[s].view(np.uint32)), s
                else:
                    ok, worst = close(alone[0], together[s], atol=5e-4, rtol=1e-3)
                    assert ok, (s, worst)
        finally:
            gpu.decode_cuts(False)


@pytest.mark.parametrize("fixed", [False, True])
def test_the_benchmarks_longest_contexts(gpu, fixed):
    # the metric is quoted at 32 K context: sequences at and just under it, beside the shortest the batch may hold
    rng = np.random.default_rng(501)
    lengths = [32768, 32767, 1024, 20001]
    contexts = [32768, 32768, 1024, 20480]
    states = [q8_state(rng, c, 2) for c in contexts]
    q = queries_f16(rng, len(lengths), 16, 256)
    gpu.decode_cuts(fixed)
    try:
        got = run_decode(gpu, states, contexts, lengths, 16, 2, q, plan=True)
    finally:
        gpu.decode_cuts(False)
    want = expect_decode(states, contexts, lengths, 16, 2, q)
    ok, worst = close(got, want)
    assert ok and worst < 5e-4, worst


def test_large_scales_and_peaked_softmax(gpu):
    rng = np.random.default_rng(600)
    state = q8_state(rng, 256, 2)
    state[:, :, 256:] = np.full((4, 256, 8), 3.0, np.float16).view(np.uint8).reshape(4, 256, 16)   # values up to 381
    q = queries_f16(rng, 1, 16, 256)
    got = run_decode(gpu, [state], [256], [256], 16, 2, q, scale=1 / 16)
    want = expect_decode([state], [256], [256], 16, 2, q, scale=1 / 16)
    ok, worst = close(got, want, atol=2e-3 * 150, rtol=1e-2)   # outputs are O(300) here
    assert ok, worst


@pytest.mark.parametrize("heads,kv_heads,plan", [(24, 2, False), (24, 2, True), (12, 1, False), (16, 1, False), (20, 2, True)])
def test_groups_of_more_than_eight_heads_are_taken_as_two_halves(gpu, heads, kv_heads, plan):
    # the reference's own layer has 24 query heads on 2 K/V heads (gpu/core.hpp:384-392; 12 on 1 for a GPU's half): an even group of up
    # to 16 is two segments a (sequence, K/V head), each streaming the head's rows for half of its query heads
    rng = np.random.default_rng(heads * 7 + kv_heads)
    lengths, contexts = [1, 17, 700, 2049], [16, 64, 1024, 4096]
    states = [q8_state(rng, c, kv_heads) for c in contexts]
    q = queries_f16(rng, len(lengths), heads, 256)
    got = run_decode(gpu, states, contexts, lengths, heads, kv_heads, q, plan=plan)
    want = expect_decode(states, contexts, lengths, heads, kv_heads, q)
    ok, worst = close(got, want)
    assert ok and worst < 1e-3, worst   # (a sequence of a few keys has nothing to average the FP16 rounding of its weights over)


def test_an_odd_group_of_more_than_eight_heads_is_refused(gpu):
    from straydog_b200.backend import StraydogError
    state, q, out = gpu.buffer(2 * 64 * 272), gpu.buffer(18 * 256 * 2), gpu.buffer(18 * 256 * 4)
    for heads in (9, 11, 17, 18):
        with pytest.raises(StraydogError, match="invalid Straydog attention dimensions"):
            gpu.qsa_decode([state], [64], [10], heads, 1, 1 / 16, q.pointer, out.pointer)
    gpu.qsa_decode([state], [64], [10], 10, 1, 1 / 16, q.pointer, out.pointer)
    for b in (state, q, out):
        gpu.release(b)


def test_attention_batch_from_host_buffers(gpu):
    rng = np.random.default_rng(700)
    n, heads, kv_heads = 5, 16, 2
    bases = [0, 15, 16, 200, 1023]
    contexts = [64, 64, 64, 512, 1024]
    states_np = [q8_state(rng, c, kv_heads, filled=b) for c, b in zip(contexts, bases)]
    states = [gpu.upload(s) for s in states_np]
    q = queries_f16(rng, n, heads, 256)
    k = rng.normal(0, 1, (n, kv_heads, 256)).astype(np.float32)
    v = rng.normal(0, 1, (n, kv_heads, 256)).astype(np.float32)
    out = np.empty((n, heads, 256), np.float32)
    gpu.attention_batch(states, contexts, bases, heads, kv_heads, 1 / 16, q, k, v, out)
    for s in range(n):
        oracle.kv_write(states_np[s], contexts[s], kv_heads, bases[s], k[s:s + 1], v[s:s + 1])
        got_state = gpu.read(states[s], np.uint8, states_np[s].shape)
        assert np.array_equal(got_state, states_np[s]), "the new row is written bit for bit"
        want = oracle.gqa_decode_q8(states_np[s], contexts[s], bases[s] + 1, heads, kv_heads, q[s], 1 / 16, f64=True)
        ok, worst = close(out[s], want)
        assert ok, (s, worst)
    for b in states:
        gpu.release(b)


def test_page_locked_host_buffers_are_used_in_place_with_the_bits_of_the_copied_ones(gpu):
    # page-locked buffers: the append reads the new rows and the merge writes the outputs in place (no copies of theirs); pageable
    # buffers take the copies. The same states, rows and outputs either way, bit for bit; a mix of the two kinds as well.
    import torch
    rng = np.random.default_rng(701)
    n, heads, kv_heads = 7, 16, 2
    bases = [0, 15, 16, 200, 1023, 31, 700]
    contexts = [64, 64, 64, 512, 1024, 64, 1024]
    states_np = [q8_state(rng, c, kv_heads, filled=b) for c, b in zip(contexts, bases)]
    q = queries_f16(rng, n, heads, 256)
    k = rng.normal(0, 1, (n, kv_heads, 256)).astype(np.float32)
    v = rng.normal(0, 1, (n, kv_heads, 256)).astype(np.float32)

    def locked(a, off=0):
        # (off: the view starts `off` elements into the page-locked allocation: an address that is not 16-byte aligned)
        t = torch.empty(a.size + off, dtype=torch.from_numpy(a).dtype).pin_memory()
        view = t.numpy()[off:].reshape(a.shape)
        view[...] = a
        return t, view
    results = []
    for kinds in ("pageable", "locked", "mixed", "off"):
        states = [gpu.upload(s) for s in states_np]
        keep = []
        def pick(a, lock):
            if not lock:
                return a.copy()
            t, view = locked(a, 1 if kinds == "off" else 0)
            keep.append(t)
            return view
        qq = pick(q, kinds == "locked")
        kk = pick(k, kinds != "pageable")
        vv = pick(v, kinds in ("locked", "off"))
        out = pick(np.full((n, heads, 256), -7.0, np.float32), kinds != "pageable")
        gpu.attention_batch(states, contexts, bases, heads, kv_heads, 1 / 16, qq, kk, vv, out)
        results.append((out.copy(), [gpu.read(s, np.uint8, sn.shape) for s, sn in zip(states, states_np)]))
        for b in states:
            gpu.release(b)
    for out, rows in results[1:]:
        assert np.array_equal(out.view(np.uint32), results[0][0].view(np.uint32))
        assert all(np.array_equal(a, b) for a, b in zip(rows, results[0][1]))
    for s in range(n):
        want_state = states_np[s].copy()
        oracle.kv_write(want_state, contexts[s], kv_heads, bases[s], k[s:s + 1], v[s:s + 1])
        assert np.array_equal(results[1][1][s], want_state)
        want = oracle.gqa_decode_q8(want_state, contexts[s], bases[s] + 1, heads, kv_heads, q[s], 1 / 16, f64=True)
        ok, worst = close(results[1][0][s], want)
        assert ok, (s, worst)


def test_batch_steps_reuse_the_work_list_until_a_sequence_enters_a_new_tile(gpu):
    # a run of decode steps: the entry keeps the step before's work list while no sequence crosses into a new 16-key tile and builds a
    # new one when one does (positions 15 -> 16, 31 -> 32 ...); another batch, another entry of the handle and a changed batch in
    # between must not leave a stale list behind. Every step is held to the oracle and to the rows the codec writes.
    rng = np.random.default_rng(702)
    heads, kv_heads = 16, 2
    contexts = [96, 2048, 512]
    bases = [12, 1000, 29]
    states_np = [q8_state(rng, c, kv_heads, filled=b) for c, b in zip(contexts, bases)]
    states = [gpu.upload(s) for s in states_np]
    other_np = q8_state(rng, 64, kv_heads, filled=40)
    other, q_dev, out_dev = gpu.upload(other_np), gpu.buffer(heads * 256 * 2), gpu.buffer(heads * 256 * 4)

    def step(order):
        n = len(order)
        q = queries_f16(rng, n, heads, 256)
        k, v = (rng.normal(0, 1, (n, kv_heads, 256)).astype(np.float32) for _ in range(2))
        out = np.empty((n, heads, 256), np.float32)
        gpu.attention_batch([states[i] for i in order], [contexts[i] for i in order], [bases[i] for i in order], heads, kv_heads, 1 / 16, q, k, v, out)
        for j, i in enumerate(order):
            oracle.kv_write(states_np[i], contexts[i], kv_heads, bases[i], k[j:j + 1], v[j:j + 1])
            want = oracle.gqa_decode_q8(states_np[i], contexts[i], bases[i] + 1, heads, kv_heads, q[j], 1 / 16, f64=True)
            ok, worst = close(out[j], want)
            assert ok, (i, bases[i], worst)
            bases[i] += 1

    for _ in range(7):           # positions 12..18, 1000..1006, 29..35: two tile crossings on the way
        step([0, 1, 2])
    step([2, 0])                 # a different batch
    gpu.qsa_decode([other], [64], [41], heads, kv_heads, 1 / 16, q_dev.pointer, out_dev.pointer)   # another entry of the handle, not waited for
    for _ in range(3):
        step([0, 1, 2])
    for i in range(3):
        assert np.array_equal(gpu.read(states[i], np.uint8, states_np[i].shape), states_np[i]), "every appended row, bit for bit"
    assert gpu.decode_status() == 0
    for b in states + [other, q_dev, out_dev]:
        gpu.release(b)


def test_a_refused_batch_step_leaves_the_states_untouched(gpu):
    # every check runs before the new rows are written: too many heads a group, and one state listed twice
    from straydog_b200.backend import StraydogError
    rng = np.random.default_rng(701)
    state_np = q8_state(rng, 64, 2, filled=10)
    a, b = gpu.upload(state_np), gpu.upload(state_np)
    q = queries_f16(rng, 2, 18, 256)
    k = rng.normal(0, 1, (2, 1, 256)).astype(np.float32)
    out = np.empty((2, 18, 256), np.float32)
    with pytest.raises(StraydogError):
        gpu.attention_batch([a, b], [64, 64], [10, 10], 18, 1, 1 / 16, q, k, k, out)       # 18 heads on one K/V head
    q16, k2, out16 = queries_f16(rng, 2, 16, 256), rng.normal(0, 1, (2, 2, 256)).astype(np.float32), np.empty((2, 16, 256), np.float32)
    with pytest.raises(StraydogError, match="listed twice"):
        gpu.attention_batch([a, a], [64, 64], [10, 10], 16, 2, 1 / 16, q16, k2, k2, out16)
    for buffer in (a, b):
        assert np.array_equal(gpu.read(buffer, np.uint8, state_np.shape), state_np)
        gpu.release(buffer)


def test_invalid_batches_are_refused(gpu):
    from straydog_b200.backend import StraydogError
    state = gpu.buffer(4 * 64 * 272)
    q = gpu.buffer(16 * 256 * 2)
    out = gpu.buffer(16 * 256 * 4)
    for args in [([state], [64], [65], 16, 2),      # length past the context
                 ([state], [64], [0], 16, 2),       # no key
                 ([state], [128], [10], 16, 2),     # state smaller than the context says
                 ([state], [64], [10], 18, 1),      # more than 16 heads a group
                 ([state], [64], [10], 16, 3)]:     # heads not a multiple of kv_heads
        with pytest.raises(StraydogError):
            gpu.qsa_decode(args[0], args[1], args[2], args[3], args[4], 1 / 16, q.pointer, out.pointer)
    with pytest.raises(StraydogError):
        gpu.qsa_decode([state], [64], [10], 16, 2, 1 / 16, q.pointer + 4096 * 2, out.pointer)   # queries outside their buffer
    for b in (state, q, out):
        gpu.release(b)
