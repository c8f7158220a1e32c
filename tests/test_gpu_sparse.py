"""sd_op_sparse_attention: the reference's ds_state_bf16_gpu.rs shapes (BF16-tagged rows give the bits of
their F32 values), the oracle within tolerance, sinks, rope, empty selections, ring addressing."""
import numpy as np
import pytest

import oracle
from util import XorShift, bf16_round, close, sparse_attention_case

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["default", "mma3", "tc1"])
def form(request):
    """Which tensor-core kernel answers where several can: the library's own choice (at 128 heads and more, BF16 rows and short windows
    the pair-of-CTAs tcgen05 kernel), the mma.sync kernel for every shape, or the single-CTA tcgen05 kernel in the pair kernel's place."""
    import os
    if request.param != "default":
        os.environ["SDX_SPARSE_KERNEL"] = request.param
    yield request.param
    os.environ.pop("SDX_SPARSE_KERNEL", None)


def reference_case(rows, heads):
    return sparse_attention_case(rows, heads)


def run(gpu, c, compressed_np, tagged, scratch_bytes=64 << 20):
    bufs = {k: gpu.upload(c[k]) for k in ("q", "raw", "sinks", "freq", "positions", "selected")}
    comp = gpu.upload(compressed_np)
    out = gpu.buffer(c["rows"] * c["heads"] * c["dim"] * 4)
    scratch = gpu.buffer(scratch_bytes) if scratch_bytes else None
    gpu.attention_turns_reserve(c["rows"], c["rope_dims"])
    gpu.sparse_attention(bufs["q"].pointer, bufs["raw"].pointer, c["raw_rows"], bufs["positions"].pointer, c["window"],
                         (comp.tagged_bf16() if tagged else comp.pointer, c["compressed_rows"]),
                         (bufs["selected"].pointer, c["selections"]), bufs["sinks"].pointer, c["rows"], c["heads"], c["dim"],
                         float(np.float32(1.0) / np.sqrt(np.float32(c["dim"]))),
                         (c["rope_dims"], bufs["freq"].pointer) if c["rope_dims"] else None, scratch, out.pointer)
    got = gpu.read(out, np.float32, (c["rows"], c["heads"], c["dim"]))
    for b in list(bufs.values()) + [comp, out] + ([scratch] if scratch else []):
        gpu.release(b)
    return got


@pytest.mark.parametrize("rows,heads", [(1, 32), (4, 32), (64, 32), (16, 64)])
def test_the_attention_of_bf16_rows_is_that_of_their_f32_values(gpu, form, rows, heads):
    c = reference_case(rows, heads)
    from_f32 = run(gpu, c, c["widened"], tagged=False)
    from_bf16 = run(gpu, c, c["halves"], tagged=True)
    assert from_f32.any()
    assert np.array_equal(from_f32.view(np.uint32), from_bf16.view(np.uint32))
    want = oracle.sparse_attention(c["q"], c["raw"], c["raw_rows"], c["positions"], c["window"], c["halves"], c["selected"],
                                   c["selections"], c["sinks"], rows, heads, c["dim"], float(np.float32(1.0) / np.sqrt(np.float32(c["dim"]))),
                                   c["rope_dims"], c["freq"], f64=True)
    ok, worst = close(from_bf16, want)
    assert ok, worst


def test_benchmark_shape_small(gpu, form):
    # config 3's shape at a size the oracle finishes quickly: 576-wide BF16 rows N(0, 0.05), unique sorted indices,
    # window 1 (the query's own F32 row), sinks at -inf, no rope
    rng = np.random.default_rng(41)
    rows, heads, dim, ctx, sel = 4, 128, 576, 4096, 512
    halves, widened = bf16_round(rng.normal(0, 0.05, (rows * ctx, dim)).astype(np.float32))
    _, q = bf16_round(rng.normal(0, 1, (rows, heads, dim)).astype(np.float32))
    raw = widened.reshape(rows, ctx, dim)[:, -1].copy()
    selected = np.stack([np.sort(rng.choice(ctx, sel, replace=False)) + r * ctx for r in range(rows)]).astype(np.int32)
    c = dict(q=q, raw=raw, sinks=np.full(heads, -np.inf, np.float32), freq=np.zeros(1, np.float32), positions=np.arange(rows, dtype=np.int32),
             selected=selected, dim=dim, window=1, raw_rows=rows, compressed_rows=rows * ctx, selections=sel, rope_dims=0, rows=rows, heads=heads)
    got = run(gpu, c, halves, tagged=True)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    want = oracle.sparse_attention(q, raw, rows, c["positions"], 1, halves, selected, sel, c["sinks"], rows, heads, dim, scale, 0, None, f64=True)
    ok, worst = close(got, want)
    assert ok, worst


@pytest.mark.parametrize("rows,heads,dim,window,selections,rope_dims,exact_q", [
    (3, 16, 576, 8, 200, 0, True), (8, 16, 576, 8, 2048, 64, True), (2, 128, 576, 1, 96, 0, True), (5, 24, 512, 128, 31, 64, False),
    (1, 8, 512, 3, 0, 0, False), (2, 40, 576, 40, 65, 128, False), (4, 32, 576, 4, 300, 64, False), (2, 64, 512, 1, 128, 0, False),
    (3, 48, 576, 2, 100, 128, True), (2, 80, 576, 16, 64, 0, True), (1, 16, 512, 1, 4000, 0, True),
    # 128 heads and more: the shapes the tcgen05 kernel takes by the library's own choice (rope on F32 queries, a head tile that is
    # half padding, 512-wide rows, the longest window it accepts, a ragged last tile of selections)
    (2, 128, 576, 8, 200, 64, False), (1, 144, 512, 2, 100, 0, True), (3, 128, 512, 16, 1000, 128, False), (1, 192, 576, 1, 64, 64, True)])
def test_tensor_core_kernel_shapes(gpu, form, rows, heads, dim, window, selections, rope_dims, exact_q):
    """Head tiles of 16 and 32 with tails, spans with a causal window (config 4's layout), rope on BF16-exact and on F32 queries,
    partial tiles, no selection at all; each against the F64 oracle and against this library's FP32 kernel."""
    import os
    rng = np.random.default_rng(rows * 100 + heads)
    raw_rows, compressed_rows = max(window, 8), 5000
    q = rng.normal(0, 1, (rows, heads, dim)).astype(np.float32)
    if exact_q:
        _, q = bf16_round(q)
    raw = rng.normal(0, 0.05, (raw_rows, dim)).astype(np.float32)
    halves, _ = bf16_round(rng.normal(0, 0.05, (compressed_rows, dim)).astype(np.float32))
    selected = rng.integers(0, compressed_rows, (rows, max(selections, 1))).astype(np.int32)
    selected[:, ::9] = -1
    positions = (np.arange(rows) + (window - 1 if rows > 1 else 0)).astype(np.int32)
    sinks = rng.normal(0, 1, heads).astype(np.float32)
    freq = (10000.0 ** (-(2.0 * np.arange(max(rope_dims, 2) // 2)) / max(rope_dims, 2))).astype(np.float32)
    c = dict(q=q, raw=raw, sinks=sinks, freq=freq, positions=positions, selected=selected, dim=dim, window=window, raw_rows=raw_rows,
             compressed_rows=compressed_rows, selections=selections, rope_dims=rope_dims, rows=rows, heads=heads)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    want = oracle.sparse_attention(q, raw, raw_rows, positions, window, halves, selected if selections else None, selections, sinks, rows, heads,
                                   dim, scale, rope_dims, freq if rope_dims else None, f64=True)
    got = run(gpu, c, halves, tagged=True)
    ok, worst = close(got, want)
    assert ok, worst
    os.environ["SDX_SPARSE_SIMT"] = "1"
    try:
        simt = run(gpu, c, halves, tagged=True)
    finally:
        del os.environ["SDX_SPARSE_SIMT"]
    assert close(simt, want, atol=1e-4, rtol=1e-3)[0]
    assert close(got, simt)[0]


@pytest.mark.parametrize("heads,window,rope_dims", [(16, 8, 64), (32, 3, 0), (8, 20, 0)])
def test_spans_in_one_call_equal_one_call_a_span(gpu, form, heads, window, rope_dims):
    """sdx_sparse_attention_spans: several verify spans (their own window rings, one shared cache allocation) in one launch give
    the bits of one sd_op_sparse_attention call a span, and stay within tolerance of the oracle."""
    rng = np.random.default_rng(7 + heads)
    spans, span_rows, dim, selections, raw_rows, per_cache = 3, 8, 576, 96, 32, 700
    q = rng.normal(0, 1, (spans, span_rows, heads, dim)).astype(np.float32)
    raw = rng.normal(0, 0.05, (spans, raw_rows, dim)).astype(np.float32)
    halves, _ = bf16_round(rng.normal(0, 0.05, (spans * per_cache, dim)).astype(np.float32))
    selected = rng.integers(0, per_cache, (spans, span_rows, selections)).astype(np.int32)
    selected[:, :, ::7] = -1
    absolute = np.where(selected >= 0, selected + (np.arange(spans) * per_cache)[:, None, None], -1).astype(np.int32)
    positions = np.stack([np.arange(span_rows) + 5 * s for s in range(spans)]).astype(np.int32)   # (span s starts at ring row 5 s)
    sinks = rng.normal(0, 1, heads).astype(np.float32)
    freq = (10000.0 ** (-(2.0 * np.arange(max(rope_dims, 2) // 2)) / max(rope_dims, 2))).astype(np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    bufs = {k: gpu.upload(v) for k, v in dict(q=q, raw=raw, positions=positions, selected=absolute, sinks=sinks, freq=freq).items()}
    comp = gpu.upload(halves)
    out = gpu.buffer(q.nbytes)
    rope = (rope_dims, bufs["freq"].pointer) if rope_dims else None
    gpu.sparse_attention_spans(bufs["q"].pointer, bufs["raw"].pointer, raw_rows, bufs["positions"].pointer, window,
                               (comp.tagged_bf16(), spans * per_cache), (bufs["selected"].pointer, selections), bufs["sinks"].pointer,
                               spans, span_rows, heads, dim, scale, rope, out.pointer)
    together = gpu.read(out, np.float32, q.shape)
    one = gpu.buffer(q[0].nbytes)
    for s in range(spans):
        gpu.sparse_attention(bufs["q"].pointer + s * q[0].nbytes, bufs["raw"].pointer + s * raw[0].nbytes, raw_rows,
                             bufs["positions"].pointer + s * span_rows * 4, window, (comp.tagged_bf16(), spans * per_cache),
                             (bufs["selected"].pointer + s * span_rows * selections * 4, selections), bufs["sinks"].pointer,
                             span_rows, heads, dim, scale, rope, None, one.pointer)
        alone = gpu.read(one, np.float32, q[0].shape)
        assert np.array_equal(alone.view(np.uint32), together[s].view(np.uint32)), f"span {s}"
        want = oracle.sparse_attention(q[s], raw[s], raw_rows, positions[s], window, halves, absolute[s], selections, sinks, span_rows, heads,
                                       dim, scale, rope_dims, freq if rope_dims else None, f64=True)
        ok, worst = close(alone, want)
        assert ok, worst
    for b in list(bufs.values()) + [comp, out, one]:
        gpu.release(b)


def test_gathered_form_with_one_rank_equals_the_plain_call(gpu):
    """sdx_sparse_attention_gather at world = 1: slot 0 of the gathered buffer holds the bits of sd_op_sparse_attention; foreign
    pointers and bad ranks are refused. (Two ranks wait on each other's counters, so they never share one GPU: the N-GPU
    form is checked against the oracle by `bench.py --config 3` under torchrun.)"""
    from straydog_b200.backend import StraydogError
    rng = np.random.default_rng(11)
    rows, heads, dim, ctx, sel = 3, 16, 576, 2048, 256
    halves, widened = bf16_round(rng.normal(0, 0.05, (rows * ctx, dim)).astype(np.float32))
    _, q = bf16_round(rng.normal(0, 1, (rows, heads, dim)).astype(np.float32))
    raw = widened.reshape(rows, ctx, dim)[:, -1].copy()
    selected = np.stack([np.sort(rng.choice(ctx, sel, replace=False)) + r * ctx for r in range(rows)]).astype(np.int32)
    sinks = rng.normal(0, 1, heads).astype(np.float32)
    bufs = {k: gpu.upload(v) for k, v in dict(q=q, raw=raw, positions=np.arange(rows, dtype=np.int32), selected=selected, sinks=sinks).items()}
    comp = gpu.upload(halves)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    plain, full, flags = gpu.buffer(q.nbytes), gpu.buffer(q.nbytes), gpu.buffer(4)
    args = (bufs["q"].pointer, bufs["raw"].pointer, rows, bufs["positions"].pointer, 1, (comp.tagged_bf16(), rows * ctx),
            (bufs["selected"].pointer, sel), bufs["sinks"].pointer, rows, heads, dim, scale, None)
    gpu.sparse_attention(*args, None, plain.pointer)
    gpu.sparse_attention_gather(*args, 0, [full.pointer], [flags.pointer], 1)
    a, b = gpu.read(plain, np.float32, q.shape), gpu.read(full, np.float32, q.shape)
    assert a.any() and np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert gpu.decode_status() == 0
    with pytest.raises(StraydogError):
        gpu.sparse_attention_gather(*args, 1, [full.pointer], [flags.pointer], 2)          # rank outside the world
    with pytest.raises(StraydogError):
        gpu.sparse_attention_gather(*args, 0, [full.pointer + 4], [flags.pointer], 2)      # buffer too small from there, and misaligned
    with pytest.raises(StraydogError):
        gpu.ipc_close(full.pointer)                                                          # not a peer mapping
    assert len(gpu.ipc_export(full)) == 64
    for b_ in list(bufs.values()) + [comp, plain, full, flags]:
        gpu.release(b_)


def test_a_gather_whose_peer_never_arrives_gives_up_with_a_status(gpu):
    """The counter wait behind the gathered form is bounded: with a second 'rank' that nothing ever runs (both buffers on this
    GPU), the wait runs out after a second, the call returns, the status word says 4 and the handle stays usable."""
    import time
    rng = np.random.default_rng(12)
    rows, heads, dim, ctx, sel = 1, 16, 512, 512, 128
    halves, widened = bf16_round(rng.normal(0, 0.05, (ctx, dim)).astype(np.float32))
    _, q = bf16_round(rng.normal(0, 1, (rows, heads, dim)).astype(np.float32))
    raw = widened[-1:].copy()
    selected = np.sort(rng.choice(ctx, sel, replace=False)).astype(np.int32).reshape(1, sel)
    bufs = {k: gpu.upload(v) for k, v in dict(q=q, raw=raw, positions=np.zeros(1, np.int32), selected=selected,
                                              sinks=np.zeros(heads, np.float32)).items()}
    comp = gpu.upload(halves)
    mine, other = gpu.buffer(2 * q.nbytes), gpu.buffer(2 * q.nbytes)
    my_flags, other_flags = gpu.buffer(8), gpu.buffer(8)
    args = (bufs["q"].pointer, bufs["raw"].pointer, 1, bufs["positions"].pointer, 1, (comp.tagged_bf16(), ctx),
            (bufs["selected"].pointer, sel), bufs["sinks"].pointer, rows, heads, dim, float(dim) ** -0.5, None)
    assert gpu.decode_status() == 0
    started = time.perf_counter()
    gpu.sparse_attention_gather(*args, 0, [mine.pointer, other.pointer], [my_flags.pointer, other_flags.pointer], 1)
    gpu.synchronize()
    waited = time.perf_counter() - started
    assert 0.9 < waited < 5.0, waited
    assert gpu.decode_status() == 4
    # rank 0's slot is written in both copies, its counter raised in both; the absent rank's slot and counter are untouched
    a, b = gpu.read(mine, np.float32, (2, rows, heads, dim)), gpu.read(other, np.float32, (2, rows, heads, dim))
    assert a[0].any() and np.array_equal(a[0], b[0]) and not a[1].any() and not b[1].any()
    assert gpu.read(my_flags, np.int32, (2,)).tolist() == [1, 0] and gpu.read(other_flags, np.int32, (2,)).tolist() == [1, 0]
    plain = gpu.buffer(q.nbytes)
    gpu.sparse_attention(*args, None, plain.pointer)   # the handle still works
    assert np.array_equal(gpu.read(plain, np.float32, q.shape), a[0])
    for b_ in list(bufs.values()) + [comp, mine, other, my_flags, other_flags, plain]:
        gpu.release(b_)


def test_window_ring_empty_selections_and_no_selection_list(gpu):
    rng = np.random.default_rng(42)
    rows, heads, dim, window, raw_rows = 5, 8, 64, 6, 8
    q = rng.normal(0, 1, (rows, heads, dim)).astype(np.float32)
    raw = rng.normal(0, 1, (raw_rows, dim)).astype(np.float32)
    halves, _ = bf16_round(rng.normal(0, 1, (20, dim)).astype(np.float32))
    positions = np.array([0, 3, 7, 8, 21], np.int32)      # before the window fills, and wrapped around the ring
    selected = np.full((rows, 4), -1, np.int32)
    selected[2] = [3, -1, 19, 0]
    sinks = rng.normal(0, 1, heads).astype(np.float32)
    c = dict(q=q, raw=raw, sinks=sinks, freq=np.zeros(1, np.float32), positions=positions, selected=selected, dim=dim, window=window,
             raw_rows=raw_rows, compressed_rows=20, selections=4, rope_dims=0, rows=rows, heads=heads)
    got = run(gpu, c, halves, tagged=True, scratch_bytes=0)
    want = oracle.sparse_attention(q, raw, raw_rows, positions, window, halves, selected, 4, sinks, rows, heads, dim, 0.125, 0, None, f64=True)
    ok, worst = close(got, want)
    assert ok, worst


def test_invalid_shapes_are_refused(gpu):
    from straydog_b200.backend import StraydogError
    b = gpu.buffer(1 << 20)
    def call(**kw):
        a = dict(rows=1, heads=4, dim=64, window=4, rope=None, selections=4)
        a.update(kw)
        gpu.sparse_attention(b.pointer, b.pointer, 8, b.pointer, a["window"], (b.pointer, 16), (b.pointer, a["selections"]), b.pointer,
                             a["rows"], a["heads"], a["dim"], 1.0, a["rope"], None, b.pointer)
    call()
    for bad in (dict(rows=0), dict(rows=65536), dict(window=0), dict(rope=(3, b.pointer)), dict(rope=(130, b.pointer)), dict(dim=32, rope=(64, b.pointer)),
                dict(selections=1 << 30)):
        with pytest.raises(StraydogError):
            call(**bad)
    gpu.release(b)
