"""Cycle counters of the MMA-issuing threads of the two tcgen05 kernels, from a build with -DSDX_TRACE.

    python -m straydog_b200.trace prompt [context first rows]      # qsa_prompt_tc_kernel (default 16384 8192 8192)
    python -m straydog_b200.trace latent [heads rows context]      # sparse_tc2_kernel (default 128 32 16384; SDX_SPARSE_KERNEL=tc1: sparse_tc_kernel)

Builds the traced variant of the library beside the product one (libstraydog_gpu_b200_trace.so; the product build holds no
counters), runs a few calls on cuda:0 and prints, per 64-key (prompt) or 32-key (latent) tile, the cycles each issuing thread spent in
all and in each of its waits. A diagnostic: the figures the profile summaries of these kernels quote.
"""
import ctypes as C
import os
import sys
import time

import numpy as np

from . import _lib, build, synthetic
from .backend import Backend

TRACE_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libstraydog_gpu_b200_trace.so")


def counters(gpu, lib):
    buf = (C.c_int64 * (8 * 8192))()
    n = lib.sdx_trace_read(gpu.handle, buf, 8 * 8192)
    return np.array(buf[:8 * n], np.int64).reshape(n, 8)


def prompt(lib, context=16384, first=8192, rows=8192):
    gpu = Backend(0, 4 << 30, library=lib)
    rng = np.random.default_rng(3)
    state, q = gpu.upload(synthetic.q8_state(rng, context, 2)), gpu.upload(synthetic.queries_f16(rng, rows, 16, 256))
    out = gpu.buffer(rows * 16 * 256 * 4)
    times = []
    for _ in range(5):
        gpu.synchronize()
        t0 = time.perf_counter()
        gpu.qsa_prompt(state, context, first, rows, 16, 2, 1 / 16, q.pointer, out.pointer)
        gpu.synchronize()
        times.append(time.perf_counter() - t0)
    t = counters(gpu, lib)
    per = lambda i: float((t[:, i] / t[:, 5]).mean())   # noqa: E731
    print(f"qsa_prompt_tc_kernel, {rows} rows after {first}: {min(times) * 1e3:.3f} ms a call (traced build), {len(t)} CTAs")
    print(f"  per 64-key tile: scores thread {per(0):.0f} cycles (waiting for a tile {per(1):.0f}, for a free score buffer {per(3):.0f}); "
          f"values thread {per(6):.0f} (waiting for the weights {per(2):.0f}, for a tile {per(4):.0f}); softmax thread 0 waiting for the scores {per(7):.0f}")
    gpu.close()


def latent(lib, heads=128, rows=32, context=16384):
    dim, sel = 576, 2048
    gpu = Backend(0, 8 << 30, library=lib)
    rng = np.random.default_rng(3)
    halves = synthetic.bf16_round(rng.normal(0, 0.05, (rows * context, dim)).astype(np.float32))[0]
    _, q = synthetic.bf16_round(rng.normal(0, 1, (rows, heads, dim)).astype(np.float32))
    raw = rng.normal(0, 0.05, (rows, dim)).astype(np.float32)
    selected = np.stack([np.sort(rng.choice(context, sel, replace=False)) + (i % rows) * context for i in range(4 * rows)])
    selected = selected.astype(np.int32).reshape(4, rows, sel)
    comp, qb, rb = gpu.upload(halves), gpu.upload(q), gpu.upload(raw)
    lists = [gpu.upload(selected[v]) for v in range(4)]
    pb, kb = gpu.upload(np.arange(rows, dtype=np.int32)), gpu.upload(np.full(heads, -1e30, np.float32))
    out = gpu.buffer(rows * heads * dim * 4)
    for i in range(6):
        gpu.sparse_attention(qb.pointer, rb.pointer, rows, pb.pointer, 1, (comp.tagged_bf16(), rows * context), (lists[i % 4].pointer, sel),
                             kb.pointer, rows, heads, dim, float(dim) ** -0.5, None, None, out.pointer)
    t = counters(gpu, lib)
    if not len(t):
        print("the call did not take a tcgen05 kernel (it needs 128 heads or more): no counters")
    elif os.environ.get("SDX_SPARSE_KERNEL") == "tc1":
        per = lambda i: float((t[:, i] / t[:, 5]).mean())   # noqa: E731
        print(f"sparse_tc_kernel, {heads} heads, {rows} rows x {sel} selected: {len(t)} CTAs, {t[:, 5].mean():.0f} tiles each")
        print(f"  per 32-key tile: issuing thread {per(0):.0f} cycles (waiting for a tile {per(1):.0f}, for the weights {per(2):.0f}, "
              f"for a free score buffer {per(3):.0f}); a copy warp waiting for a free slot {per(4):.0f}")
    else:
        per = lambda i: float((t[:, i] / t[:, 5]).mean())   # noqa: E731
        print(f"sparse_tc2_kernel (pairs of CTAs), {heads} heads, {rows} rows x {sel} selected: {len(t)} CTAs, {t[:, 5].mean():.0f} tiles each")
        print(f"  a CTA: {t[:, 3].mean():.0f} cycles before the first tile (Q's preparation), {t[:, 7].mean():.0f} in the tiles, {t[:, 2].mean():.0f} after "
              f"(the last products, the partial's stores)")
        print(f"  per 32-key tile: score thread {per(0):.0f} cycles (waiting for a tile {per(1):.0f}); softmax thread {per(7):.0f} "
              f"(waiting for the two halves' rows {per(4):.0f})")
    gpu.close()


def main(argv):
    if not argv or argv[0] not in ("prompt", "latent"):
        raise SystemExit(__doc__)
    build.build(defines=("SDX_TRACE",), out=TRACE_LIB)
    lib = _lib.load(TRACE_LIB)
    (prompt if argv[0] == "prompt" else latent)(lib, *[int(x) for x in argv[1:]])


if __name__ == "__main__":
    main(sys.argv[1:])
