"""sdx_qsa_decode_static: the decode whose scratch is a fixed array inside the library, for hosts that may not
allocate while they serve. Collected last on purpose (a failure here stops nothing before it).

Checks, through the C ABI: two calls in a row (different batches, so the second must not see the first one's
leftovers in the shared array) give what sdx_qsa_decode gives for the same inputs, and what the CPU oracle
gives within the decode tests' tolerance; a batch beyond the stated limits is refused with an error; once a
first call has made the library's device image resident, a further call on a new batch shape leaves the
GPU's free memory where it was.
"""
import numpy as np
import pytest

import oracle
from util import close, q8_state, queries_f16

pytestmark = pytest.mark.gpu


def decode_both(gpu, lengths, seed):
    rng = np.random.default_rng(seed)
    states_np = [q8_state(rng, l, 2) for l in lengths]
    q = queries_f16(rng, len(lengths), 16, 256)
    states = [gpu.upload(s) for s in states_np]
    q_dev = gpu.upload(q)
    out_static = gpu.upload(np.full((len(lengths), 16, 256), np.nan, np.float32))
    out_plain = gpu.buffer(len(lengths) * 16 * 256 * 4)
    gpu.qsa_decode_static(states, lengths, lengths, 16, 2, 1 / 16, q_dev.pointer, out_static.pointer)
    got_static = gpu.read(out_static, np.float32, (len(lengths), 16, 256))
    gpu.qsa_decode(states, lengths, lengths, 16, 2, 1 / 16, q_dev.pointer, out_plain.pointer)
    got_plain = gpu.read(out_plain, np.float32, (len(lengths), 16, 256))
    want = np.stack([oracle.gqa_decode_q8(states_np[s], lengths[s], lengths[s], 16, 2, q[s], 1 / 16, f64=True) for s in range(len(lengths))])
    for b in states + [q_dev, out_static, out_plain]:
        gpu.release(b)
    return got_static, got_plain, want


def test_two_calls_in_a_row_match_the_allocating_entry(gpu):
    for lengths, seed in [([3000, 17, 901, 2048, 1], 1), ([64, 5000], 2)]:
        got_static, got_plain, want = decode_both(gpu, lengths, seed)
        ok, worst = close(got_static, got_plain)
        assert ok, worst
        assert np.array_equal(got_static.view(np.uint32), got_plain.view(np.uint32)), "the same kernels over the same work list"
        ok, worst = close(got_static, want)
        assert ok, worst
    assert gpu.decode_status() == 0


def test_a_batch_beyond_the_static_scratch_is_refused(gpu):
    from straydog_b200.backend import StraydogError
    state = gpu.buffer(4 * 16 * 272)
    q = gpu.buffer(65 * 16 * 256 * 2)
    out = gpu.buffer(65 * 16 * 256 * 4)
    with pytest.raises(StraydogError, match="at most 64 sequences"):
        gpu.qsa_decode_static([state] * 65, [16] * 65, [16] * 65, 16, 2, 1 / 16, q.pointer, out.pointer)
    for b in (state, q, out):
        gpu.release(b)


def test_the_largest_batch_the_limits_allow_fits_the_static_scratch(gpu):
    # 64 sequences on 8 K/V heads is the most segments a call may hold (512); its work list has at most one piece per warp of the
    # GPU plus one per segment, 8 * 148 + 512 = 1696 on a B200, inside the 2048 the scratch holds (the refusal beyond 2048 pieces
    # guards a GPU with more SMs): the call is accepted and gives the allocating entry's bits
    rng = np.random.default_rng(10)
    length = 3001
    state_np = q8_state(rng, length, 8)
    state = gpu.upload(state_np)
    q = gpu.upload(queries_f16(rng, 64, 8, 256))
    out_static, out_plain = gpu.buffer(64 * 8 * 256 * 4), gpu.buffer(64 * 8 * 256 * 4)
    gpu.qsa_decode_static([state] * 64, [length] * 64, [length] * 64, 8, 8, 1 / 16, q.pointer, out_static.pointer)
    gpu.qsa_decode([state] * 64, [length] * 64, [length] * 64, 8, 8, 1 / 16, q.pointer, out_plain.pointer)
    a, b = gpu.read(out_static, np.uint32, (64 * 8 * 256,)), gpu.read(out_plain, np.uint32, (64 * 8 * 256,))
    assert np.array_equal(a, b)
    assert gpu.decode_status() == 0
    for buffer in (state, q, out_static, out_plain):
        gpu.release(buffer)


def test_after_the_first_call_a_call_leaves_free_memory_unchanged(gpu):
    import torch
    rng = np.random.default_rng(9)
    states = [gpu.upload(q8_state(rng, l, 2)) for l in (700, 1300, 90)]
    q = gpu.upload(queries_f16(rng, 3, 16, 256))
    out = gpu.buffer(3 * 16 * 256 * 4)
    gpu.qsa_decode_static(states[:1], [700], [700], 16, 2, 1 / 16, q.pointer, out.pointer)   # the first call: the image is resident after it
    free_before = torch.cuda.mem_get_info(0)[0]
    gpu.qsa_decode_static(states, [700, 1300, 90], [700, 1300, 90], 16, 2, 1 / 16, q.pointer, out.pointer)   # a batch shape not seen before
    assert torch.cuda.mem_get_info(0)[0] == free_before
    for b in states + [q, out]:
        gpu.release(b)
