"""Selection-list decode attention on the tensor cores (sdx_qsa_attention_rows: the reference's qsa_attention / qsa_attention_rows,
gpu/sparse_attention_compute.hpp:609-647) against outputs of the reference's own library and against the oracle."""
import os

import numpy as np
import pytest

import oracle
from util import attention_sequence_input, close, q8_state

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz"))
GUARD, CANARY = 8, np.float32(-7777.5)


def attend(gpu, state, context, base, steps, selected, heads, kv_heads, packed, positions=None, mirror=None, gates=None, scale=0.0625):
    """Appends the rows' keys and values as the reference's span does (write_attention_kv), then attends; returns [steps][heads][256]."""
    inp = gpu.upload(packed)
    keys_at, values_at = steps * heads * 256 * 4, steps * (heads + kv_heads) * 256 * 4
    if positions is None:
        gpu._c(gpu.lib.sdx_kv_write(gpu.handle, state.pointer, context, kv_heads, base, steps, inp.at(keys_at), inp.at(values_at)))
    pos = gpu.upload(np.asarray(positions, np.uint32)) if positions is not None else None
    out = gpu.upload(np.full(steps * heads * 256 + 2 * GUARD, CANARY, np.float32))
    gate_buffer = gpu.upload(gates) if gates is not None else None
    gpu.qsa_attention_rows(state, context, base, pos.pointer if pos else None, steps, selected, heads, kv_heads, scale, inp.pointer,
                           out.at(GUARD * 4), mirror=mirror, gates=(gate_buffer.pointer, heads * 512) if gate_buffer else None)
    got = gpu.read(out, np.float32, (steps * heads * 256 + 2 * GUARD,))
    assert gpu.decode_status() == 0
    assert np.all(got[:GUARD] == CANARY) and np.all(got[-GUARD:] == CANARY), "output guard"
    for b in (inp, pos, out, gate_buffer):
        if b:
            gpu.release(b)
    return got[GUARD:-GUARD].reshape(steps, heads, 256)


@pytest.mark.parametrize("steps,selected,base,context,kind", [(4, 2052, 3000, 4096, "sparse"), (3, 64, 100, 256, "dense"), (8, 513, 20, 64, "sparse")])
def test_the_reference_librarys_own_outputs(gpu, steps, selected, base, context, kind):
    # the inputs of sd_attention_sequence's golden cases (24 query / 2 K/V heads, unsorted lists with dead slots) through the
    # tensor-core kernel: the outputs the reference's library gave on a B200
    rng = np.random.default_rng(steps * 1000 + selected)
    state_np = q8_state(rng, context, 2, filled=base)
    packed = attention_sequence_input(rng, steps, selected, base, context, kind)
    state = gpu.allocate(state_np.nbytes)
    gpu.write(state, state_np)
    got = attend(gpu, state, context, base, steps, selected, 24, 2, packed)
    after = gpu.download(state, np.empty_like(state_np))
    key = f"sequence_{steps}_{selected}_{base}_{context}_{kind}"
    assert np.array_equal(after[:, base:base + steps], GOLDEN[key + "_rows"])
    ok, worst = close(got, GOLDEN[key], atol=1e-4, rtol=1e-3)
    assert ok and worst < 1e-4, worst
    gpu.release(state)


@pytest.mark.parametrize("heads,kv_heads", [(16, 2), (24, 2), (12, 1), (4, 4)])
def test_a_rows_bits_do_not_depend_on_the_rows_beside_it(gpu, heads, kv_heads):
    # the verification contract: row r of an 8-row launch has the bits of a one-row launch of the same token
    rng = np.random.default_rng(heads * 10 + kv_heads)
    steps, selected, base, context = 8, 700, 1500, 2048
    state_np = q8_state(rng, context, kv_heads, filled=base)
    packed = attention_sequence_input(rng, steps, selected, base, context, "sparse", heads, kv_heads)
    state = gpu.allocate(state_np.nbytes)
    gpu.write(state, state_np)
    together = attend(gpu, state, context, base, steps, selected, heads, kv_heads, packed)
    want = oracle.attention_sequence(gpu.download(state, np.empty_like(state_np)), context, heads, kv_heads, base, steps, selected, packed)
    ok, worst = close(together, want, atol=1e-4, rtol=1e-3)
    assert ok, worst
    q_n, kv_n = steps * heads * 256, steps * kv_heads * 256
    for r in (0, 3, 7):
        one = np.concatenate([packed[r * heads * 256:(r + 1) * heads * 256], packed[q_n + r * kv_heads * 256:q_n + (r + 1) * kv_heads * 256],
                              packed[q_n + kv_n + r * kv_heads * 256:q_n + kv_n + (r + 1) * kv_heads * 256],
                              packed[q_n + 2 * kv_n + r * selected:q_n + 2 * kv_n + (r + 1) * selected],
                              packed[q_n + 2 * kv_n + steps * selected + r:q_n + 2 * kv_n + steps * selected + r + 1]]).astype(np.float32)
        alone = attend(gpu, state, context, base + r, 1, selected, heads, kv_heads, one, positions=[base + r])
        assert np.array_equal(alone[0].view(np.uint32), together[r].view(np.uint32)), r
    gpu.release(state)


def test_recent_rows_come_from_the_ring_mirror(gpu):
    # a host-resident state's newest rows are read from the mirror slot position % mirror_rows when
    # position + mirror_rows > last + 8: the state's copies of those rows are scrambled here, the result must not change
    rng = np.random.default_rng(3)
    steps, selected, base, context, mirror_rows = 4, 300, 1000, 1100, 128
    state_np = q8_state(rng, context, 2, filled=base + steps)
    packed = attention_sequence_input(rng, steps, selected, base, context, "sparse")
    state = gpu.upload(state_np)
    positions = [base + r for r in range(steps)]
    want = attend(gpu, state, context, base, steps, selected, 24, 2, packed, positions=positions)
    last = base + steps - 1
    mirror_np = np.zeros((4, mirror_rows, 272), np.uint8)
    scrambled = state_np.copy()
    for position in range(context):
        if position + mirror_rows > last + 8 and position <= last:
            mirror_np[:, position % mirror_rows] = state_np[:, position]
            scrambled[:, position] = 0x55
    state2, mirror = gpu.upload(scrambled), gpu.upload(mirror_np)
    got = attend(gpu, state2, context, base, steps, selected, 24, 2, packed, positions=positions, mirror=(mirror.pointer, mirror_rows))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    for b in (state, state2, mirror):
        gpu.release(b)


def test_the_merge_applies_the_output_gate(gpu):
    rng = np.random.default_rng(4)
    steps, selected, base, context = 2, 130, 200, 256
    state_np = q8_state(rng, context, 2, filled=base + steps)
    packed = attention_sequence_input(rng, steps, selected, base, context, "dense")
    state = gpu.upload(state_np)
    positions = [base, base + 1]
    plain = attend(gpu, state, context, base, steps, selected, 24, 2, packed, positions=positions)
    gates = rng.normal(0, 4, (steps, 24, 512)).astype(np.float32)
    gated = attend(gpu, state, context, base, steps, selected, 24, 2, packed, positions=positions, gates=gates)
    x = gates[:, :, 256:].astype(np.float64)
    want = plain * (1.0 / (1.0 + np.exp(-x)))
    assert np.abs(gated - want).max() < 1e-6
    gpu.release(state)


def test_invalid_shapes_are_refused(gpu):
    from straydog_b200.backend import StraydogError
    state = gpu.buffer(4 * 64 * 272)
    packed = gpu.buffer(2 * (24 * 256 + 1024 + 64 + 1) * 4)
    out = gpu.buffer(2 * 24 * 256 * 4)
    for context, steps, selected, heads, kv_heads in [(0, 1, 64, 24, 2), (64, 0, 64, 24, 2), (64, 257, 64, 24, 2), (64, 2, 0, 24, 2),
                                                      (64, 2, 8193, 24, 2), (64, 2, 64, 24, 5), (64, 2, 64, 40, 2), (128, 2, 64, 24, 2),
                                                      (64, 3, 64, 24, 2)]:
        with pytest.raises(StraydogError):
            gpu.qsa_attention_rows(state, context, 0, None, steps, selected, heads, kv_heads, 0.0625, packed.pointer, out.pointer)
    for b in (state, packed, out):
        gpu.release(b)


@pytest.mark.parametrize("stage_rows,expect_passes", [(4096, 1), (700, None), (24, 0)])
def test_a_host_resident_state_is_attended_through_the_gathered_union(gpu, stage_rows, expect_passes):
    # the K/V lies in page-locked host memory (sd_host_state); the union of the rows' selected 4-position blocks is copied into the
    # VRAM stage and the selections renumbered to it: the bits of the plain entry over a VRAM copy of the same state. Stages that hold
    # the whole batch's union, a few rows' at a time, and not even one row's (refused).
    rng = np.random.default_rng(77)
    steps, selected, base, context, heads, kv_heads = 8, 600, 3000, 4096, 16, 2
    state_np = q8_state(rng, context, kv_heads, filled=base + steps)
    packed = attention_sequence_input(rng, steps, selected, base, context, "sparse", heads, kv_heads)
    positions = np.arange(base, base + steps, dtype=np.uint32)
    device_state = gpu.allocate(state_np.nbytes)
    gpu.write(device_state, state_np)
    want = attend(gpu, device_state, context, base, steps, selected, heads, kv_heads, packed, positions=positions)
    assert gpu.lib.sd_host_state_supported(gpu.handle) == 1
    host_state = gpu.host_state(state_np.nbytes)
    gpu.write(host_state, state_np)
    assert np.array_equal(gpu.download(host_state, np.empty_like(state_np)), state_np)
    stage = gpu.allocate(stage_rows * 4096)
    gpu.kv_stage(stage, stage_rows)
    inp, pos = gpu.upload(packed), gpu.upload(positions)
    out = gpu.upload(np.full(steps * heads * 256 + 2 * GUARD, CANARY, np.float32))
    if expect_passes == 0:   # a stage that does not hold even one row's selection
        from straydog_b200.backend import StraydogError
        with pytest.raises(StraydogError, match="too small for one row"):
            gpu.qsa_attention_gathered(host_state, context, base, pos.pointer, steps, selected, heads, kv_heads, 0.0625, inp.pointer, out.at(GUARD * 4))
    for run in range(2 if expect_passes != 0 else 0):
        passes = gpu.qsa_attention_gathered(host_state, context, base, pos.pointer, steps, selected, heads, kv_heads, 0.0625, inp.pointer, out.at(GUARD * 4))
        got = gpu.read(out, np.float32, (steps * heads * 256 + 2 * GUARD,))
        assert np.all(got[:GUARD] == CANARY) and np.all(got[-GUARD:] == CANARY), "output guard"
        assert np.array_equal(got[GUARD:-GUARD].view(np.uint32), want.reshape(-1).view(np.uint32)), run
        assert passes == expect_passes if expect_passes else passes > 1
    assert gpu.decode_status() == 0
    assert np.array_equal(gpu.read(inp, np.float32, packed.shape), packed), "the caller's rows stay as they are"
    for b in (device_state, inp, pos, out, stage, host_state):   # (releasing the stage unregisters it)
        gpu.release(b)
    from straydog_b200.backend import StraydogError
    with pytest.raises(StraydogError, match="no Straydog K/V stage"):
        gpu.qsa_attention_gathered(device_state.pointer, context, base, None, steps, selected, heads, kv_heads, 0.0625, inp.pointer, out.pointer)


def dense_f64(planes, packed, steps, selected, heads, kv_heads, base, context, scale=0.0625):
    """The definition in float64 over FP16 rows' values: softmax of q . k over the row's live slots, times v."""
    group = heads // kv_heads
    q = packed[:steps * heads * 256].reshape(steps, heads, 256).astype(np.float64)
    at = steps * (heads + 2 * kv_heads) * 256
    lists, counts = packed[at:at + steps * selected].reshape(steps, selected), packed[at + steps * selected:]
    out = np.zeros((steps, heads, 256))
    for r in range(steps):
        live = [int(x) for x in lists[r, :int(counts[r])] if 0 <= x <= base + r and x < context]
        for h in range(heads):
            scores = planes[h // group, live] @ q[r, h] * scale
            w = np.exp(scores - scores.max())
            out[r, h] = (w / w.sum()) @ planes[kv_heads + h // group, live]
    return out


@pytest.mark.parametrize("steps,selected,base,context,heads,kv_heads,kind", [(5, 64, 40, 96, 24, 2, "sparse"), (4, 2052, 3000, 4096, 24, 2, "sparse"),
                                                                             (8, 700, 1500, 2048, 16, 2, "sparse"), (3, 130, 200, 256, 12, 1, "dense")])
def test_fp16_rows_are_attended_on_the_tensor_cores(steps, selected, base, context, heads, kv_heads, kind):
    """sd_kv_format(512): the selection-list kernel reads FP16 rows (256 halves) as the tensor cores' operands. Held to the float64
    definition over the rows' values, to the FP32 check path (sd_attention_sequence, at its own 24 / 2 heads) and to the contract that a
    row's bits do not depend on the rows beside it; dead slots (lists with -1, positions past the row's own) carry no weight."""
    from straydog_b200.backend import Backend
    rng = np.random.default_rng(steps * 100 + selected)
    with Backend(0, 1 << 29) as gpu:
        gpu.kv_format(512)
        filled = rng.normal(0, 1, (2 * kv_heads, context, 256)).astype(np.float16)
        filled[:, base:] = 0
        packed = attention_sequence_input(rng, steps, selected, base, context, kind, heads, kv_heads)
        state = gpu.allocate(filled.nbytes)
        gpu.write(state, filled)
        got = attend(gpu, state, context, base, steps, selected, heads, kv_heads, packed)   # (writes the rows' keys and values first)
        rows = gpu.download(state, np.empty_like(filled))
        k = packed[steps * heads * 256:steps * (heads + kv_heads) * 256].reshape(steps, kv_heads, 256)
        assert np.array_equal(rows[:kv_heads, base:base + steps].view(np.uint16), k.transpose(1, 0, 2).astype(np.float16).view(np.uint16))
        want = dense_f64(rows.astype(np.float64), packed, steps, selected, heads, kv_heads, base, context)
        assert np.abs(got - want).max() < 5e-5, np.abs(got - want).max()
        if (heads, kv_heads) == (24, 2):
            check = gpu.attention_sequence(state, context, base, steps, selected, packed)
            assert np.abs(got - check).max() < 1e-4
        positions = np.arange(base, base + steps, dtype=np.uint32)
        for r in (0, steps - 1):
            width = heads * 256 + kv_heads * 512
            q_at, k_at, v_at = r * heads * 256, steps * heads * 256 + r * kv_heads * 256, steps * (heads + kv_heads) * 256 + r * kv_heads * 256
            at = steps * (heads + 2 * kv_heads) * 256
            one = np.concatenate([packed[q_at:q_at + heads * 256], packed[k_at:k_at + kv_heads * 256], packed[v_at:v_at + kv_heads * 256],
                                  packed[at + r * selected:at + (r + 1) * selected], packed[at + steps * selected + r:at + steps * selected + r + 1]])
            alone = attend(gpu, state, context, base, 1, selected, heads, kv_heads, one, positions=positions[r:r + 1])
            assert np.array_equal(alone[0].view(np.uint32), got[r].view(np.uint32)), r
        gpu.release(state)


def test_fp16_rows_of_a_host_resident_state_go_through_the_gathered_union():
    from straydog_b200.backend import Backend
    rng = np.random.default_rng(78)
    steps, selected, base, context, heads, kv_heads = 8, 600, 3000, 4096, 16, 2
    with Backend(0, 1 << 29) as gpu:
        gpu.kv_format(512)
        filled = rng.normal(0, 1, (2 * kv_heads, context, 256)).astype(np.float16)
        packed = attention_sequence_input(rng, steps, selected, base, context, "sparse", heads, kv_heads)
        positions = np.arange(base, base + steps, dtype=np.uint32)
        device_state = gpu.allocate(filled.nbytes)
        gpu.write(device_state, filled)
        want = attend(gpu, device_state, context, base, steps, selected, heads, kv_heads, packed, positions=positions)
        host_state = gpu.host_state(filled.nbytes)
        gpu.write(host_state, filled)
        stage = gpu.allocate(1400 * 4096)
        gpu.kv_stage(stage, 1400)
        inp, pos, out = gpu.upload(packed), gpu.upload(positions), gpu.buffer(steps * heads * 256 * 4)
        passes = gpu.qsa_attention_gathered(host_state, context, base, pos.pointer, steps, selected, heads, kv_heads, 0.0625, inp.pointer, out.pointer)
        assert passes > 1 and gpu.decode_status() == 0
        assert np.array_equal(gpu.read(out, np.float32, want.shape).view(np.uint32), want.view(np.uint32))
        for b in (device_state, inp, pos, out, stage, host_state):
            gpu.release(b)
