"""sd_attention_sequence at the reference's own shapes (24 query / 2 K/V heads, <= 2052 selected keys)."""
import numpy as np
import pytest

import oracle
from util import attention_sequence_input, close, q8_state

pytestmark = pytest.mark.gpu


def packed_input(rng, steps, selected, base, context, kind):
    return attention_sequence_input(rng, steps, selected, base, context, kind)


@pytest.mark.parametrize("steps,selected,base,context,kind", [
    (1, 1, 0, 16, "dense"), (1, 64, 100, 256, "dense"), (4, 2052, 3000, 4096, "sparse"),
    (8, 513, 20, 64, "sparse"), (3, 2052, 2500, 2600, "dense"), (17, 100, 0, 300, "sparse")])
def test_matches_the_oracle(gpu, steps, selected, base, context, kind):
    rng = np.random.default_rng(steps * 1000 + selected)
    state_np = q8_state(rng, context, 2, filled=base)
    inp = packed_input(rng, steps, selected, base, context, kind)
    state = gpu.allocate(state_np.nbytes)
    gpu.write(state, state_np)
    got = gpu.attention_sequence(state, context, base, steps, selected, inp)
    want_state = state_np.copy()
    want = oracle.attention_sequence(want_state, context, 24, 2, base, steps, selected, inp)
    ok, worst = close(got, want, atol=1e-4, rtol=1e-3)   # FP32 on both sides: only summation order differs
    assert ok, worst
    got_state = gpu.download(state, np.empty_like(state_np))
    assert np.array_equal(got_state, want_state), "rows base.. are written bit for bit"
    gpu.release(state)


def test_validation_follows_the_reference(gpu):
    from straydog_b200.backend import StraydogError, lib
    import ctypes as C
    context = 64
    state = gpu.allocate(context * 4 * 272)
    good = packed_input(np.random.default_rng(1), 1, 8, 10, context, "dense")
    out = np.empty(24 * 256, np.float32)

    def call(st, ctx, base, steps, selected, inp, in_count, out_count):
        return lib().sd_attention_sequence(gpu.handle, st, ctx, base, steps, selected, inp.ctypes.data_as(C.c_void_p), in_count,
                                           out.ctypes.data_as(C.c_void_p), out_count)
    assert call(state.pointer, context, 10, 1, 8, good, good.size, out.size) == 0
    assert call(state.pointer, context, 10, 1, 2053, good, good.size, out.size) < 0            # selected > 2052
    assert b"attention dimensions" in lib().sd_error()
    assert call(state.pointer, context, 64, 1, 8, good, good.size, out.size) < 0               # no room past base
    assert call(state.pointer, context * 2, 10, 1, 8, good, good.size, out.size) < 0           # state size mismatch
    assert b"state size mismatch" in lib().sd_error()
    assert call(state.pointer, context, 10, 1, 8, good, good.size - 1, out.size) < 0           # workspace mismatch
    bad = good.copy()
    bad[-1] = 0.0
    assert call(state.pointer, context, 10, 1, 8, bad, bad.size, out.size) < 0                 # count < 1
    assert b"selection count" in lib().sd_error()
    bad[-1] = 2.5
    assert call(state.pointer, context, 10, 1, 8, bad, bad.size, out.size) < 0                 # not an integer
    gpu.release(state)
