"""sd_op_dspark_attention in the manner of the reference's own test (crates/straydog-engine/tests/dspark_attention_gpu.rs): its seeded
inputs, its F64 oracle's bound (error <= 2e-5 / (1 + |reference|)), the anchor read from device memory, the observable cases with
constant keys, every invalid shape refused."""
import numpy as np
import pytest

import oracle
from util import dspark_case

pytestmark = pytest.mark.gpu
HEADS, DIM = 64, 512


def check(actual, expected):
    error = np.abs(actual.astype(np.float64) - expected) / (1.0 + np.abs(expected))
    assert error.max() <= 2e-5, error.max()


def test_blocks_of_1_to_5_slots_and_histories_0_37_128(gpu):
    c = dspark_case()
    q, ring, block, sinks = (gpu.upload(c[k]) for k in ("q", "ring", "block", "sinks"))
    out = gpu.buffer(c["q"].nbytes)
    for slots in range(1, 6):
        for history, anchor in [(0, 0), (37, 149), (128, 389)]:
            gpu.dspark_attention(q.pointer, ring, block.pointer, sinks, HEADS, slots, anchor, None, history, out.pointer)
            want = oracle.dspark_attention(c["q"][:slots], c["ring"], c["block"], c["sinks"], HEADS, slots, anchor, history, f64=True)
            check(gpu.read(out, np.float32, (slots, HEADS, DIM)), want)
    for slots in (1, 4):   # a device's half of the heads: q [slots][32][512] and its sinks
        half = HEADS // 2
        gpu.dspark_attention(q.pointer, ring, block.pointer, sinks, half, slots, 149, None, 37, out.pointer)
        q_half = c["q"].reshape(-1, DIM)[:slots * half].reshape(slots, half, DIM)
        check(gpu.read(out, np.float32, (slots, half, DIM)), oracle.dspark_attention(q_half, c["ring"], c["block"], c["sinks"], half, slots, 149, 37, f64=True))
    # the anchor from a device int32: the same launch follows it as it moves
    anchor_at = gpu.upload(np.array([389], np.int32))
    for at in (389, 200, 128):
        gpu.write_buffer(anchor_at, 0, np.array([at], np.int32))
        gpu.dspark_attention(q.pointer, ring, block.pointer, sinks, HEADS, 3, 389, anchor_at.pointer, 128, out.pointer)
        check(gpu.read(out, np.float32, (3, HEADS, DIM)), oracle.dspark_attention(c["q"][:3], c["ring"], c["block"], c["sinks"], HEADS, 3, at, 128, f64=True))
    from straydog_b200.backend import StraydogError
    for heads, slots, anchor, history in [(64, 0, 0, 0), (64, 6, 0, 0), (64, 1, 129, 129), (64, 1, 36, 37), (64, 1, 2 ** 32 - 1, 0), (0, 1, 0, 0), (65, 1, 0, 0)]:
        with pytest.raises(StraydogError, match="DSpark"):
            gpu.dspark_attention(q.pointer, ring, block.pointer, sinks, heads, slots, anchor, None, history, out.pointer)
    for b in (q, ring, block, sinks, out, anchor_at):
        gpu.release(b)


def test_future_keys_and_the_sinks_mass_are_observable(gpu):
    q = gpu.upload(np.zeros((5, HEADS, DIM), np.float32))
    ring = gpu.upload(np.full((128, DIM), 23.0, np.float32))   # no history: must never be attended
    block_np = np.repeat(np.arange(1, 6, dtype=np.float32)[:, None], DIM, 1)
    block, sinks = gpu.upload(block_np), gpu.upload(np.zeros(HEADS, np.float32))
    out = gpu.buffer(5 * HEADS * DIM * 4)

    def run():
        gpu.dspark_attention(q.pointer, ring, block.pointer, sinks, HEADS, 5, 0, None, 0, out.pointer)
        return gpu.read(out, np.float32, (5, HEADS, DIM))
    check(run(), np.full((5, HEADS, DIM), 2.5))          # every query, the first included, sees five keys and one sink
    block_np[4] = 11.0
    gpu.write_buffer(block, 0, block_np)
    check(run(), np.full((5, HEADS, DIM), 3.5))
    for sink, expected in [(1000.0, 0.0), (-1000.0, 4.2)]:
        gpu.write_buffer(sinks, 0, np.full(HEADS, sink, np.float32))
        check(run(), np.full((5, HEADS, DIM), expected))
    for b in (q, ring, block, sinks, out):
        gpu.release(b)


def test_the_reference_librarys_own_outputs(gpu):
    import os
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz"))
    c = dspark_case()
    q, ring, block, sinks = (gpu.upload(c[k]) for k in ("q", "ring", "block", "sinks"))
    out = gpu.buffer(c["q"].nbytes)
    for slots, history, anchor in [(1, 0, 0), (5, 37, 149), (3, 128, 389)]:
        gpu.dspark_attention(q.pointer, ring, block.pointer, sinks, HEADS, slots, anchor, None, history, out.pointer)
        want = golden[f"dspark_{slots}_{history}_{anchor}"]
        got = gpu.read(out, np.float32, (slots, HEADS, DIM))
        assert np.abs(got[:, ::8] - want).max() <= 2e-5   # (the fixture holds every eighth head)
    for b in (q, ring, block, sinks, out):
        gpu.release(b)
