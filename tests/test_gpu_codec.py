"""Q8_0 write and decode on the GPU against the oracle: bit for bit."""
import numpy as np
import pytest

import oracle
from util import q8_state

pytestmark = pytest.mark.gpu


def test_kv_write_is_bit_exact(gpu):
    rng = np.random.default_rng(31)
    context, kv_heads = 96, 2
    for base, steps in [(0, 1), (5, 8), (40, 56), (95, 1)]:
        keys = (rng.normal(0, 1, (steps, kv_heads, 256)) * rng.choice([1e-5, 0.02, 1.0, 40.0, 6e4], (steps, kv_heads, 1))).astype(np.float32)
        values = rng.normal(0, 3, (steps, kv_heads, 256)).astype(np.float32)
        keys[0, 0, 32:64] = 0.0            # an all-zero block: zero scale, zero bytes
        values[0, 0, :3] = [np.float32(0.5), np.float32(1.5), np.float32(2.5)]   # ties
        expect = np.zeros((2 * kv_heads, context, 272), np.uint8)
        oracle.kv_write(expect, context, kv_heads, base, keys, values)
        state = gpu.buffer(expect.nbytes)
        k_dev, v_dev = gpu.upload(keys), gpu.upload(values)
        gpu.kv_write(state, context, kv_heads, base, steps, k_dev, v_dev)
        got = gpu.read(state, np.uint8, expect.shape)
        assert np.array_equal(got, expect), (base, steps)
        for b in (state, k_dev, v_dev):
            gpu.release(b)


def test_q8_decode_is_bit_exact(gpu):
    rng = np.random.default_rng(32)
    state = q8_state(rng, 500, 2)
    rows = state.reshape(-1, 272)
    dev = gpu.upload(rows)
    out = gpu.buffer(rows.shape[0] * 256 * 4)
    gpu.kv_decode_rows(dev.pointer, rows.shape[0], out)
    got = gpu.read(out, np.float32, (rows.shape[0], 256))
    want = oracle.q8_decode_rows(rows)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    gpu.release(dev)
    gpu.release(out)


def test_kv_write_rejects_bad_shapes(gpu):
    from straydog_b200.backend import StraydogError
    state = gpu.buffer(4 * 16 * 272)
    rows = gpu.buffer(2 * 256 * 4)
    with pytest.raises(StraydogError):
        gpu.kv_write(state, 16, 2, 16, 1, rows, rows)      # past the context
    with pytest.raises(StraydogError):
        gpu.kv_write(state, 32, 2, 0, 1, rows, rows)       # state too small for the context
    gpu.release(state)
    gpu.release(rows)


def test_kv_stage_registration_is_validated(gpu):
    # gpu/kernels.cpp:4277-4290: the stage is one allocation of exactly rows * 4096 bytes; it is dropped when that allocation is released
    from straydog_b200.backend import StraydogError
    stage = gpu.buffer(8 * 4096)
    gpu.kv_stage(stage, 8)
    for rows in (0, 7, 9):
        with pytest.raises(StraydogError, match="K/V stage"):
            gpu.kv_stage(stage, rows)
    other = gpu.buffer(64)
    with pytest.raises(StraydogError):
        gpu.kv_stage(other, 8)
    gpu.release(other)
    gpu.release(stage)


def test_fp16_rows_are_written_decoded_and_attended_by_the_check_path():
    # gpu/kernels.cpp:4266-4275 takes 512 (FP16 rows) and 272 (Q8_0 rows). FP16 rows (a value's nearest FP16, gpu/kernels.cpp:42, 70)
    # are written, decoded and attended by sd_attention_sequence, the path Q8_0 results are checked against (the selection-list kernel
    # reads them too: test_gpu_qsa_select.py); the dense batch decode and the prompt kernel read Q8_0 rows only and say so at the call
    # instead of misreading FP16 rows
    from straydog_b200.backend import Backend, StraydogError
    from util import attention_sequence_input
    rng = np.random.default_rng(21)
    with Backend(0, 1 << 28) as gpu:
        with pytest.raises(StraydogError, match="K/V format"):
            gpu.kv_format(100)
        gpu.kv_format(512)
        context, base, steps, selected = 96, 40, 5, 64
        filled = rng.normal(0, 1, (4, context, 256)).astype(np.float16)
        filled[:, base:] = 0
        state = gpu.allocate(filled.nbytes)
        gpu.write(state, filled)
        inp = attention_sequence_input(rng, steps, selected, base, context, "sparse")
        got = gpu.attention_sequence(state, context, base, steps, selected, inp)
        rows = gpu.download(state, np.empty_like(filled))
        q = inp[:steps * 24 * 256].reshape(steps, 24, 256).astype(np.float64)
        k = inp[steps * 24 * 256:steps * 26 * 256].reshape(steps, 2, 256)
        v = inp[steps * 26 * 256:steps * 28 * 256].reshape(steps, 2, 256)
        want_rows = filled.copy()
        want_rows[:2, base:base + steps] = k.transpose(1, 0, 2).astype(np.float16)
        want_rows[2:, base:base + steps] = v.transpose(1, 0, 2).astype(np.float16)
        assert np.array_equal(rows.view(np.uint16), want_rows.view(np.uint16)), "rows base.. hold the nearest FP16 of the new keys and values"
        lists = inp[steps * 28 * 256:steps * 28 * 256 + steps * selected].reshape(steps, selected)
        counts = inp[steps * 28 * 256 + steps * selected:]
        planes = want_rows.astype(np.float64)
        for r in range(steps):
            live = [int(x) for x in lists[r, :int(counts[r])] if 0 <= x <= base + r and x < context]
            for h in range(24):
                scores = planes[h // 12, live] @ q[r, h] * 0.0625
                w = np.exp(scores - scores.max())
                assert np.abs(got[r, h] - (w / w.sum()) @ planes[2 + h // 12, live]).max() < 1e-4
        # the codec's two entries in the same format
        keys, values = rng.normal(0, 2, (3, 2, 256)).astype(np.float32), rng.normal(0, 2, (3, 2, 256)).astype(np.float32)
        kb, vb = gpu.upload(keys), gpu.upload(values)
        gpu.kv_write(state, context, 2, 7, 3, kb, vb)
        out = gpu.buffer(3 * 256 * 4)
        gpu._c(gpu.lib.sdx_kv_decode_rows(gpu.handle, state.pointer + (1 * context + 7) * 512, 3, out.pointer))
        assert np.array_equal(gpu.read(out, np.float32, (3, 256)), keys[:, 1].astype(np.float16).astype(np.float32))
        q16, o = gpu.buffer(16 * 256 * 2), gpu.buffer(16 * 256 * 4)
        with pytest.raises(StraydogError, match="Q8_0"):
            gpu.qsa_decode([state], [context], [16], 16, 2, 1 / 16, q16.pointer, o.pointer)
        with pytest.raises(StraydogError, match="Q8_0"):
            gpu.qsa_prompt(state, context, 0, 4, 16, 2, 1 / 16, q16.pointer, o.pointer)
        gpu.kv_format(272)
        small = gpu.buffer(4 * 16 * 272)
        gpu.qsa_decode([small], [16], [16], 16, 2, 1 / 16, q16.pointer, o.pointer)
