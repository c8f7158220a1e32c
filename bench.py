#!/usr/bin/env python
"""Benchmark of the attention path: the Q8_0 GQA decode of the ragged 64-sequence batch (the line's headline) and, as extra keys
of the same line, the other four configurations and the two curves that really scale.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu] [--config C] [--no-extras]

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE for N > 1). A step of the headline is one pass of the decode
attention over one batch: 64 sequences with context lengths uniform in [1024, 32768], 16 query / 2 K/V heads of 256, Q8_0 K/V
rows, FP16 queries, FP32 output. Sequences are independent, so ranks share no data: every rank decodes a 64-sequence batch of
the same seeded lengths and its own seeded contents (weak scaling).

Prints ONE JSON line (rank 0). `value` is K/V gigabytes streamed per second by the whole job with everything resident in HBM;
`e2e` is the same metric through sdx_attention_batch with host buffers (queries, new K/V rows and outputs copied inside the timed
call, a new position every step). `roofline` times the streaming kernel alone with CUDA events on its own stream. `cpu_baseline`
times the CPU oracle on a bounded sample. Extra keys: `configs` (configurations 0, 2, 3, 4, each with its own time, roofline,
clock record and error against the oracle), `step_ms_percentiles`, and under torchrun `config1_strong` (the one 64-sequence batch
dealt over the ranks) and `config3_head_sharded` (the 128 heads dealt over the ranks, outputs gathered inside the kernel).
`--impl reference` times the reference's scalar host path (the CPU oracle port); `--impl reference-gpu --config C` times the
reference's own kernels from oracle/_ref on the same GPU. `--config C` alone prints that configuration's entry only.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADS, KV_HEADS, DIM, ROW = 16, 2, 256, 272
SCALE = 1.0 / 16.0
SEED = 20261125
METRIC, UNIT = "decode_attn_kv_gbps", "GB/s"
TOLERANCE = (2e-3, 1e-2)   # max-abs or max-rel per element: the tests' tolerance


TENSOR_SUSTAINED = 1400.0   # dense BF16 over seconds under the power cap (the fallback; the measured file overrides it)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        global TENSOR_SUSTAINED
        TENSOR_SUSTAINED = float(peaks.get("bf16_tflops_sustained", TENSOR_SUSTAINED))
        return float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback (6.65 TB/s, 1.59 PFLOP/s: earlier measurements on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None
        try:
            self.process = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                             "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def count(self):
        try:
            with open(self.file.name) as f:
                return sum(1 for _ in f)
        except OSError:
            return 0

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.process is None:
            return out
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, reasons, power = [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                clocks.append(float(parts[0]))
                out["sm_max_mhz"] = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, state in zip(names, parts[4:8]):
                if state.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if clocks:
            out["sm_mhz"] = statistics.median(clocks)
            out["samples"] = len(clocks)
            out["power_w_max"] = max(power)
        out["reasons"] = sorted(reasons)
        return out


def within_tolerance(got, want):
    error = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    ok = (error <= TOLERANCE[0]) | (error <= TOLERANCE[1] * np.abs(want))
    return bool(np.all(ok) and np.all(np.isfinite(got))), float(error.max())


def batch_for(rank, world, scaling, sequences=64):
    """(lengths of this rank's sequences, their seeds)."""
    from straydog_b200.sharding import rank_batch
    return rank_batch(SEED, rank, world, scaling, sequences)


def make_states(lengths, seeds, slack=0):
    """Q8_0 states of `length + slack` positions with `length` rows filled."""
    from straydog_b200.synthetic import q8_state
    return [q8_state(np.random.default_rng(seed), length + slack, KV_HEADS, filled=length) for length, seed in zip(lengths, seeds)]


def workload_config(lengths):
    return {"workload": "config 1: ragged Q8_0 GQA decode batch, 64 sequences x 1 query token, context uniform in [1024, 32768], "
                        "16 query / 2 K/V heads, head_dim 256, FP16 queries, softmax scale 1/16, FP32 output",
            "sequences_per_gpu": len(lengths), "kv_bytes_per_gpu": sum(lengths) * 2 * KV_HEADS * ROW, "seed": SEED,
            "l2": "inputs larger than L2 (1.0 GB of K/V per step against 126 MB); the CPU arm reads host memory"}


def cpu_sample(lengths, seeds, budget_s):
    """Times the CPU oracle on the first sequences of the batch until about budget_s seconds are spent."""
    import oracle
    from straydog_b200.synthetic import queries_f16
    oracle.set_threads(os.cpu_count() or 1)   # (torchrun exports OMP_NUM_THREADS=1 to its ranks)
    spent, nbytes, used = 0.0, 0, 0
    rng = np.random.default_rng(SEED)
    for length, seed in zip(lengths, seeds):
        state = make_states([length], [seed])[0]
        q = queries_f16(rng, HEADS, DIM)
        t0 = time.perf_counter()
        oracle.gqa_decode_q8(state, length, length, HEADS, KV_HEADS, q, SCALE)
        spent += time.perf_counter() - t0
        nbytes += length * 2 * KV_HEADS * ROW
        used += 1
        if spent >= budget_s:
            break
    return nbytes / spent / 1e9, used, nbytes, spent, oracle.threads()


def run_reference(args, rank):
    """The reference's scalar host path (its CPU restatement: no part of the reference's CPU code covers attention on the host
    beyond the scalar definition the oracle restates), on all host threads, rank 0 only."""
    if rank != 0:
        return
    lengths, seeds = batch_for(0, 1, "weak")
    per_step = max(2.0, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_sample(lengths, seeds, per_step / 4)
    times, total_bytes, used, threads = [], 0, 0, 0
    for _ in range(args.steps):
        _, used, nbytes, spent, threads = cpu_sample(lengths, seeds, per_step)
        times.append(spent)
        total_bytes += nbytes
    total = sum(times)
    value = total_bytes / total / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (seeded)", "config": workload_config(lengths),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"first {used} of 64 sequences per step ({total_bytes // args.steps} K/V bytes)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tokens_per_s": used * args.steps / total}
    print(json.dumps(line), flush=True)


# ---- timing helpers ----
def timed(gpu, fn, steps, warmup):
    for _ in range(max(3, warmup)):
        fn()
    gpu.synchronize()
    start, stop = gpu.event(), gpu.event()
    gpu.record(start)
    for _ in range(steps):
        fn()
    gpu.record(stop)
    gpu.synchronize()
    return gpu.elapsed_ms(start, stop) / steps


def measured(gpu, fn, local, seconds=1.2, steps=None, warmup=3):
    """fn timed back to back for about `seconds` (device events on the library's stream) with the GPU's clocks sampled meanwhile."""
    pilot = timed(gpu, fn, 10, warmup)
    count = steps or int(max(20, min(50000, seconds * 1e3 / max(pilot, 1e-3))))
    sampler = ClockSampler(local)
    t0 = time.perf_counter()
    while sampler.count() < 1 and time.perf_counter() - t0 < 2.0:   # (the sampler's first line, under load)
        for _ in range(20):
            fn()
        gpu.synchronize()
    ms = timed(gpu, fn, count, 0)
    clocks = sampler.stop()
    clocks["note"] = "nvidia-smi every 100 ms while this configuration's timed steps ran"
    return ms, count, clocks


class DeviceArray:
    """A device buffer of this library seen by torch without a copy (the CUDA array interface)."""
    def __init__(self, pointer, count, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (int(pointer), False), "version": 3}


def reference_gpu_backend(budget):
    """The reference's own GPU library built for sm_100a (oracle/_ref): the same-box kernels to beat."""
    from straydog_b200 import _lib
    from straydog_b200.backend import Backend
    path = os.path.join(ROOT, "oracle", "_ref", "libstraydog_ref.so")
    if not os.path.exists(path):
        raise SystemExit("oracle/_ref/libstraydog_ref.so is missing: build it with `make -f oracle/Makefile.ref` where the reference's sources are")
    gpu = Backend(0, budget, library=_lib.load(path, reference_abi_only=True))
    gpu.kv_format(272)
    return gpu


def host_timed(gpu, step, probe_buffer, steps):
    """The reference queues on its own stream: its calls are timed on the host around a synchronising read."""
    probe = np.empty(4, np.float32)
    for _ in range(2):
        step()
    gpu.read_buffer(probe_buffer, 0, probe)
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    gpu.read_buffer(probe_buffer, 0, probe)
    return (time.perf_counter() - t0) * 1e3 / steps


# ---- configurations 0 and 2: one Q8_0 state, a one-token decode or a prompt chunk ----
def run_qsa_config(cfg, args, local, gpu=None):
    from straydog_b200.backend import Backend
    from straydog_b200 import synthetic
    import oracle
    peak_hbm, peak_tensor, peak_source = measured_peaks()
    ref = args.impl == "reference-gpu"
    context = 4096 if cfg == 0 else 16384
    first, rows = (4095, 1) if cfg == 0 else (8192, 8192)
    rng = np.random.default_rng(SEED + cfg)
    state_np = synthetic.q8_state(rng, context, KV_HEADS)
    q_np = synthetic.queries_f16(rng, rows, HEADS, DIM)
    kv_bytes = (first + rows) * 2 * KV_HEADS * ROW
    flops = 4.0 * DIM * HEADS * sum(first + r + 1 for r in range(rows))
    entry = {"workload": "config 0: 1 sequence x 4096 keys, one-token decode" if cfg == 0 else
                         "config 2: 8192-token chunk after 8192 cached, causal prompt attention", "impl": args.impl}
    own = gpu is None
    if not ref:
        gpu = gpu or Backend(local, 4 << 30)
        state, q = gpu.upload(state_np), gpu.upload(q_np)
        out = gpu.buffer(rows * HEADS * DIM * 4)
        if cfg == 0:
            plan = gpu.qsa_plan([state], [context], [context], HEADS, KV_HEADS)
            step = lambda: gpu.qsa_plan_run(plan, SCALE, q.pointer, out.pointer)
        else:
            step = lambda: gpu.qsa_prompt(state, context, first, rows, HEADS, KV_HEADS, SCALE, q.pointer, out.pointer)
        ms, count, clocks = measured(gpu, step, local, steps=args.steps if args.config == cfg and args.steps_given else None)
        got = gpu.read(out, np.float32, (rows, HEADS, DIM))
        if cfg == 0:
            want = oracle.gqa_decode_q8(state_np, context, context, HEADS, KV_HEADS, q_np[0], SCALE, f64=True)[None]
            ok, error = within_tolerance(got, want)
            gpu.qsa_plan_release(plan)
        else:
            sample = [0, 1, 15, 16, 4097, rows - 17, rows - 1]
            want = oracle.gqa_prompt_q8(state_np, context, first, HEADS, KV_HEADS, q_np, SCALE, rows=sample, f64=True)
            ok, error = within_tolerance(got[sample], want[sample])
            entry["rows_checked"] = sample
        if gpu.decode_status() != 0:
            raise SystemExit(f"config {cfg}: a bounded wait inside a kernel gave up: the result is invalid")
        if not ok:
            raise SystemExit(f"config {cfg}: the timed output differs from the oracle (max abs error {error})")
        entry.update({"steps": count, "clocks": clocks, "max_abs_error_vs_oracle": error})
        for b in (state, q, out):
            gpu.release(b)
    else:
        # the reference's generic GQA over the dequantised F32 K/V [context][kv_heads][dim] (gpu/token_mixing.hpp:652)
        gpu = reference_gpu_backend(8 << 30)
        planes = oracle.q8_decode_rows(state_np.reshape(-1, ROW)).reshape(2 * KV_HEADS, context, DIM)
        keys = np.ascontiguousarray(planes[:KV_HEADS].transpose(1, 0, 2))
        values = np.ascontiguousarray(planes[KV_HEADS:].transpose(1, 0, 2))
        kb, vb, qb = gpu.upload(keys), gpu.upload(values), gpu.upload(q_np.astype(np.float32))
        pb = gpu.upload(np.arange(first, first + rows, dtype=np.int32))
        scratch = gpu.buffer(max(1, rows * HEADS * 64 * (DIM + 2) * 4) if rows < 16 else 4096)
        out = gpu.buffer(rows * HEADS * DIM * 4)
        ms = host_timed(gpu, lambda: gpu.attention(qb.pointer, kb.pointer, vb.pointer, context, pb.pointer, rows, HEADS, KV_HEADS, DIM, SCALE,
                                                   None, scratch, out.pointer), out, args.steps)
        entry["steps"] = args.steps
    entry.update({"ms": ms, "kv_gbps": kv_bytes / ms / 1e6, "tflops": flops / ms / 1e9, "tokens_per_s": rows / ms * 1e3,
                  "roofline": ({"bound": "hbm", "achieved": kv_bytes / ms / 1e6, "peak": peak_hbm, "unit": "GB/s", "frac": kv_bytes / ms / 1e6 / peak_hbm,
                                "note": "two launches of a few microseconds: launch-bound, the state (4.5 MB) stays in L2"}
                               if cfg == 0 else
                               {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": TENSOR_SUSTAINED, "unit": "TFLOP/s",
                                "frac": flops / ms / 1e9 / TENSOR_SUSTAINED, "frac_of_burst_peak": flops / ms / 1e9 / peak_tensor, "burst_peak": peak_tensor,
                                "note": "algorithmic flops 4 * 256 * 16 * sum of visible keys; the kernel issues every product twice (FP16 hi and lo "
                                        "planes of K and V), which the figure does not count. The steps run back to back for about a second under the "
                                        "power cap, so the peak is the sustained cuBLAS figure; the burst one is beside it"}),
                  "peak_source": peak_source})
    if own or ref:
        gpu.close()
    return entry


# ---- the index producers: top-k of a row of scores, and the fused index select (scores + top-k) ----
def run_index_ops(args, local, gpu):
    """sd_op_top_k on (32 rows, 65 536 groups, k 2048) and sd_op_index_select on (32 rows, 16 384 groups of BF16 keys, 64 heads x 128, rope 64,
    k 2048), each timed with device events, checked against the oracle bit for bit, and timed on the reference's own library beside it
    when that library is present (host-timed around a synchronising read, as its calls queue on its own stream)."""
    from straydog_b200.backend import Backend
    from straydog_b200 import synthetic
    import oracle
    peak_hbm, _, peak_source = measured_peaks()
    rng = np.random.default_rng(SEED + 9)
    rows, groups, k = 32, 65536, 2048
    scores_np = rng.normal(0, 1, (rows, groups)).astype(np.float32)
    scores_np[:, ::97] = scores_np[:, 5::97]          # equal scores, so the tie rule takes part
    c = synthetic.index_case(rows, 16384, heads=64, dim=128, rope_dims=64, spread=0)
    halves = oracle.to_bf16(c["keys"])

    def measure(lib_gpu, device_events):
        scores, picked = lib_gpu.upload(scores_np), lib_gpu.buffer(rows * k * 4)
        bufs = {name: lib_gpu.upload(c[name]) for name in ("q", "weights", "visible", "positions", "frequencies")}
        keys = lib_gpu.upload(halves)
        index_scores, index_picked = lib_gpu.buffer(rows * c["groups"] * 4), lib_gpu.buffer(rows * k * 4)
        steps_top = lambda: lib_gpu.top_k(scores.pointer, rows, groups, k, picked.pointer)
        steps_select = lambda: lib_gpu.index_select(bufs["q"].pointer, keys.tagged_bf16(), bufs["weights"].pointer, bufs["visible"].pointer, rows,
                                                    c["groups"], c["heads"], c["dim"], c["scale"],
                                                    (c["rope_dims"], bufs["positions"].pointer, bufs["frequencies"].pointer),
                                                    index_scores.pointer, k, index_picked.pointer)
        times = {}
        for name, step, probe in (("top_k", steps_top, picked), ("index_select", steps_select, index_picked)):
            if device_events:
                for _ in range(5):
                    step()
                start, stop = lib_gpu.event(), lib_gpu.event()
                lib_gpu.record(start)
                for _ in range(200):
                    step()
                lib_gpu.record(stop)
                lib_gpu.synchronize()
                times[name] = Backend.elapsed_ms(start, stop) / 200
            else:
                times[name] = host_timed(lib_gpu, step, probe, 50)
        got = lib_gpu.read(picked, np.int32, (rows, k)), lib_gpu.read(index_scores, np.float32, (rows, c["groups"])), lib_gpu.read(index_picked, np.int32, (rows, k))
        for b in [scores, picked, keys, index_scores, index_picked] + list(bufs.values()):
            lib_gpu.release(b)
        return times, got
    times, (picked, index_scores, index_picked) = measure(gpu, True)
    if not np.array_equal(picked, oracle.top_k(scores_np, k)) or not np.array_equal(index_picked, oracle.top_k(index_scores, k)):
        raise SystemExit("index ops: the chosen indices differ from the oracle's")
    entry = {"workload": "sd_op_top_k (32 x 65536 scores, k 2048) and sd_op_index_select (32 rows, 16384 BF16 keys of 128, 64 heads, rope 64, k 2048)",
             "top_k_ms": times["top_k"], "index_select_ms": times["index_select"], "indices_equal_oracle": True,
             "top_k_roofline": {"bound": "hbm", "achieved": rows * groups * 4 / times["top_k"] / 1e6, "peak": peak_hbm, "unit": "GB/s",
                                "frac": rows * groups * 4 / times["top_k"] / 1e6 / peak_hbm,
                                "note": "algorithmic bytes = the scores once (8.4 MB: they fit L2, and the kernel reads them twice); a row is a cluster of 4 CTAs (128 SMs), a launch a chain of block and cluster barriers: latency-bound"},
             "peak_source": peak_source}
    if os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libstraydog_ref.so")):
        ref = reference_gpu_backend(1 << 30)
        ref_times, (ref_picked, ref_scores, ref_index) = measure(ref, False)
        ref.close()
        entry.update({"reference_top_k_ms": ref_times["top_k"], "reference_index_select_ms": ref_times["index_select"],
                      "equal_to_reference_library": bool(np.array_equal(picked, ref_picked) and np.array_equal(index_picked, ref_index) and
                                                         np.array_equal(index_scores.view(np.uint32), ref_scores.view(np.uint32)))})
    return entry


# ---- the Qwen seam: the indexer's block choice, then selection-list attention over the lists it wrote (a verification's rows) ----
def run_qsa_rows(args, local, gpu):
    """sdx_qsa_index_select (8 rows at positions near 32 768: 8192 blocks scored, 512 chosen, 2048 + tail positions listed) followed by
    sdx_qsa_attention_rows over those lists (16 query / 2 K/V heads, Q8_0 state of 32 768 positions), and the fused front of 8 rows
    (sdx_qsa_normalize_rows): each timed with device events, the attention checked against the oracle's scalar selection attention over
    the oracle's lists, the front against the oracle's restatement."""
    from straydog_b200.backend import Backend
    from straydog_b200 import synthetic
    import oracle
    peak_hbm, _, peak_source = measured_peaks()
    steps, context, selected = 8, 32768, 2052
    base = context - steps
    rng = np.random.default_rng(SEED + 11)
    c = synthetic.qsa_index_case(steps, base, context // 4, HEADS, KV_HEADS, selected)
    state_np = synthetic.q8_state(rng, context, KV_HEADS)
    q, blocks, packed, state = gpu.upload(c["queries"]), gpu.upload(c["blocks"]), gpu.upload(c["packed"]), gpu.upload(state_np)
    out = gpu.buffer(steps * HEADS * DIM * 4)
    index = lambda: gpu.qsa_index_select(q.pointer, 512, blocks.pointer, c["pool"], base, None, steps, selected, HEADS, KV_HEADS, packed.pointer)
    attend = lambda: gpu.qsa_attention_rows(state, context, base, None, steps, selected, HEADS, KV_HEADS, SCALE, packed.pointer, out.pointer)
    # (the rows' own keys and values are appended first, as the reference's span does before it attends)
    gpu._c(gpu.lib.sdx_kv_write(gpu.handle, state.pointer, context, KV_HEADS, base, steps, packed.at(steps * HEADS * DIM * 4), packed.at(steps * (HEADS + KV_HEADS) * DIM * 4)))
    times = {}
    for name, step in (("index_select_ms", index), ("attention_rows_ms", attend)):
        for _ in range(5):
            step()
        start, stop = gpu.event(), gpu.event()
        gpu.record(start)
        for _ in range(200):
            step()
        gpu.record(stop)
        gpu.synchronize()
        times[name] = Backend.elapsed_ms(start, stop) / 200
    got_lists, got = gpu.read(packed, np.float32, c["packed"].shape), gpu.read(out, np.float32, (steps, HEADS, DIM))
    want_lists = oracle.qsa_index_select(c["queries"], c["blocks"], base, steps, selected, c["row_floats"], c["packed"].copy())
    want = oracle.attention_sequence(state_np.copy(), context, HEADS, KV_HEADS, base, steps, selected, want_lists, scale=SCALE)
    ok, error = within_tolerance(got, want)
    if not np.array_equal(got_lists.view(np.uint32), want_lists.view(np.uint32)) or not ok or gpu.decode_status() != 0:
        raise SystemExit(f"qsa rows: lists or outputs differ from the oracle (max abs error {error})")
    listed = int(sum(want_lists[steps * c["row_floats"] + steps * selected + r] for r in range(steps)))
    nbytes = listed * 2 * KV_HEADS * ROW
    # the fused front of the same 8 rows (sdx_qsa_normalize_rows: norm, rotation, Q8_0 K/V write, index-key pooling), behind the checks
    # above because it writes the state; its rows sit at positions 2040..2047, where the host's and the device's powf / cosf / sinf
    # agree to 2e-4 (a last place of 1e7^(c/32) moves the angle by position * 6e-8)
    stride, pool = HEADS * 512 + KV_HEADS * 512 + 640, context // 4 + 1
    positions = np.arange(2040, 2040 + steps, dtype=np.uint32)
    proj_np = rng.normal(0, 1, (steps, stride)).astype(np.float32)
    norms_np = [rng.normal(1, 0.1, n).astype(np.float32) for n in (256, 256, 128, 128)]
    index_np = np.zeros((pool + 16) * 128, np.float32)
    proj, index_state, pos = gpu.upload(proj_np), gpu.upload(index_np), gpu.upload(positions)
    norms = [gpu.upload(n) for n in norms_np]
    front = lambda: gpu.qsa_normalize_rows(proj.pointer, stride, steps, HEADS, KV_HEADS, *[n.pointer for n in norms], pos.pointer, pos.pointer,
                                           packed.pointer, selected, state, context, index_state.pointer)
    front()
    front_packed = gpu.read(packed, np.float32, c["packed"].shape)[:steps * (HEADS + KV_HEADS) * DIM]
    start, stop = gpu.event(), gpu.event()
    for _ in range(5):
        front()
    gpu.record(start)
    for _ in range(200):
        front()
    gpu.record(stop)
    gpu.synchronize()
    times["normalize_rows_ms"] = Backend.elapsed_ms(start, stop) / 200
    want_packed, want_state = c["packed"].copy(), state_np.view(np.uint8).ravel().copy()
    oracle.qsa_normalize_rows(proj_np.copy(), HEADS, KV_HEADS, *norms_np, positions, positions, want_packed, want_state, context, index_np.copy())
    front_error = float(np.abs(front_packed - want_packed[:front_packed.size]).max())
    if front_error > 2e-4 or gpu.decode_status() != 0:
        raise SystemExit(f"qsa rows: the fused front differs from the oracle (max abs error {front_error})")
    for b in (q, blocks, packed, state, out, proj, index_state, pos, *norms):
        gpu.release(b)
    return {"workload": "Qwen's indexer (8 rows, 8192 blocks, 512 chosen) and selection-list attention of the 8 rows over the lists it wrote (32768-position Q8_0 state)",
            **times, "lists_equal_oracle": True, "max_abs_error_vs_oracle": error, "normalize_rows_max_abs_error_vs_oracle": front_error,
            "attention_rows_roofline": {"bound": "hbm", "achieved": nbytes / times["attention_rows_ms"] / 1e6, "peak": peak_hbm, "unit": "GB/s",
                                        "frac": nbytes / times["attention_rows_ms"] / 1e6 / peak_hbm,
                                        "note": f"algorithmic bytes = {listed} listed positions x 2 K/V heads x (K row + V row) x 272 B; a call of 8 rows is "
                                                "528 small CTAs of gathered 272-byte rows and two launches: latency, not bandwidth"},
            "peak_source": peak_source}


# ---- configurations 3 and 4: latent sparse attention, decode rows and verify spans ----
def latent_inputs(gpu, cfg, heads, context, local, device_rows=True):
    """Seeded inputs of configurations 3 / 4. The BF16 latent rows (2.4 GB / 0.6 GB) are drawn on the device by torch's seeded
    generator, N(0, 0.05) rounded to BF16, straight into the library's buffer; the oracle check reads back the rows it needs."""
    import torch
    from straydog_b200 import synthetic
    dim, selections = 576, 2048
    rows, window, calls = (32, 1, 1) if cfg == 3 else (8, 8, 16)
    total_rows = rows * context if cfg == 3 else calls * context
    rng = np.random.default_rng(SEED + cfg)
    comp = gpu.buffer(total_rows * dim * 2)
    view = torch.as_tensor(DeviceArray(comp.pointer, total_rows * dim, "<i2"), device=torch.device("cuda", local))
    generator = torch.Generator(device=torch.device("cuda", local))
    generator.manual_seed(SEED + cfg)
    slab = 1 << 18
    for at in range(0, total_rows, slab):
        n = min(slab, total_rows - at)
        draw = torch.randn(n * dim, generator=generator, device=view.device, dtype=torch.float32) * 0.05
        view[at * dim:(at + n) * dim] = draw.to(torch.bfloat16).view(torch.int16)
    torch.cuda.synchronize()
    _, q_np = synthetic.bf16_round(rng.normal(0, 1, (calls, rows, heads, dim)).astype(np.float32))
    raw_np = rng.normal(0, 0.05, (calls, max(rows, window), dim)).astype(np.float32)
    # config 3 touches 75.5 MB a step, which would stay in the 126 MB L2: successive steps rotate over `variants` index lists
    # (302 MB in all); config 4's 16 spans touch 302 MB a step as it is
    variants = 4 if cfg == 3 else 1
    selected = np.stack([np.sort(rng.choice(context, selections, replace=False)) for _ in range(variants * calls * rows)]).astype(np.int32)
    if cfg == 3:
        selected += (np.tile(np.arange(rows), variants) * context)[:, None].astype(np.int32)
    else:
        selected += (np.repeat(np.arange(calls), rows) * context)[:, None].astype(np.int32)
    selected = selected.reshape(variants * calls, rows, selections)
    return dict(comp=comp, view=view, q=q_np, raw=raw_np, selected=selected, rows=rows, window=window, calls=calls, dim=dim,
                selections=selections, total_rows=total_rows, variants=variants, positions=np.arange(rows, dtype=np.int32),
                scale=float(np.float32(1.0) / np.sqrt(np.float32(dim))))


def latent_error(inp, got, samples, heads_first=0):
    """Max abs error of sampled (call, row, head) outputs against the oracle (F64), reading the selected rows back from the device."""
    import oracle
    worst, ok_all = 0.0, True
    dim, selections = inp["dim"], inp["selections"]
    for call, variant, row, head in samples:
        index = inp["selected"][variant * inp["calls"] + call][row]
        import torch
        rows_host = inp["view"].view(-1, dim)[torch.as_tensor(index.astype(np.int64), device=inp["view"].device)].cpu().numpy().view(np.uint16)
        want = oracle.sparse_attention(inp["q"][call, row:row + 1, head:head + 1], inp["raw"][call], inp["raw"].shape[1], inp["positions"][row:row + 1],
                                       inp["window"], rows_host, np.arange(selections, dtype=np.int32)[None], selections,
                                       np.full(1, -1e30, np.float32), 1, 1, dim, inp["scale"], f64=True)
        ok, error = within_tolerance(got[call, row, head - heads_first], want[0, 0])
        worst, ok_all = max(worst, error), ok_all and ok
    return ok_all, worst


def run_latent_config(cfg, args, local, gpu=None, head_shards=None):
    from straydog_b200.backend import Backend
    peak_hbm, peak_tensor, peak_source = measured_peaks()
    ref = args.impl == "reference-gpu"
    shards = head_shards or max(1, args.head_shards)
    heads = 128 // shards
    context = args.context or (65536 if cfg == 3 else 32768)
    own = gpu is None
    gpu = reference_gpu_backend(16 << 30) if ref else (gpu or Backend(local, 16 << 30))
    inp = latent_inputs(gpu, cfg, heads, context, local)
    rows, window, calls, dim, selections, variants = inp["rows"], inp["window"], inp["calls"], inp["dim"], inp["selections"], inp["variants"]
    comp, total_rows, scale = inp["comp"], inp["total_rows"], inp["scale"]
    sinks = gpu.upload(np.full(heads, -1e30, np.float32))
    pb = gpu.upload(inp["positions"])
    turn = [0]
    if cfg == 4 and not ref and not args.per_call:
        # the 16 spans in one launch (sdx_sparse_attention_spans): their buffers laid end to end
        q_all, raw_all, sel_all = gpu.upload(inp["q"]), gpu.upload(inp["raw"]), gpu.upload(inp["selected"])
        pos_all = gpu.upload(np.tile(inp["positions"], calls))
        out_all = gpu.buffer(calls * rows * heads * dim * 4)
        buffers = [q_all, raw_all, sel_all, pos_all, out_all]

        def step():
            gpu.sparse_attention_spans(q_all.pointer, raw_all.pointer, inp["raw"].shape[1], pos_all.pointer, window, (comp.tagged_bf16(), total_rows),
                                       (sel_all.pointer, selections), sinks.pointer, calls, rows, heads, dim, scale, None, out_all.pointer)
        read = lambda: gpu.read(out_all, np.float32, (calls, rows, heads, dim))
        form = "one launch for the 16 spans"
    else:
        qb = [gpu.upload(inp["q"][c]) for c in range(calls)]
        rb = [gpu.upload(inp["raw"][c]) for c in range(calls)]
        sb = [gpu.upload(inp["selected"][c]) for c in range(variants * calls)]
        outs = [gpu.buffer(rows * heads * dim * 4) for _ in range(calls)]
        scratch = gpu.buffer(512 << 20) if ref else None
        buffers = qb + rb + sb + outs + ([scratch] if scratch else [])

        def step():
            turn[0] = (turn[0] + 1) % variants
            for c in range(calls):
                gpu.sparse_attention(qb[c].pointer, rb[c].pointer, inp["raw"].shape[1], pb.pointer, window, (comp.tagged_bf16(), total_rows),
                                     (sb[turn[0] * calls + c].pointer, selections), sinks.pointer, rows, heads, dim, scale, None, scratch, outs[c].pointer)
        read = lambda: np.stack([gpu.read(o, np.float32, (rows, heads, dim)) for o in outs])
        form = "one call per sequence" if cfg == 4 else "one call"
    entry = {"workload": ("config 3: latent sparse decode, 32 queries x top-2048 of 65536, 576-wide BF16 rows" if cfg == 3 else
                          "config 4: verify spans, 16 sequences x 8 draft rows, top-2048 of 32768, causal window in the span") + "; " + form,
             "impl": args.impl, "heads": heads, "head_shards": shards,
             "l2": "steps rotate over 4 index lists (302 MB of rows against the 126 MB L2)" if cfg == 3 else "302 MB of rows a step"}
    if ref:
        ms = host_timed(gpu, step, outs[-1], args.steps)
        entry["steps"] = args.steps
    else:
        ms, count, clocks = measured(gpu, step, local, steps=args.steps if args.config == cfg and args.steps_given else None)
        got = read()
        samples = [(0, turn[0], 0, 0), (0, turn[0], rows - 1, heads - 1), (calls - 1, turn[0], rows // 2, heads // 2)]
        ok, error = latent_error(inp, got, samples)
        if gpu.decode_status() != 0:
            raise SystemExit(f"config {cfg}: a kernel reported a status: the result is invalid")
        if not ok:
            raise SystemExit(f"config {cfg}: the timed output differs from the oracle (max abs error {error})")
        entry.update({"steps": count, "clocks": clocks, "max_abs_error_vs_oracle": error})
    keys_per_row = selections + (window if cfg == 3 else (window + 1) / 2)
    nbytes = calls * rows * selections * dim * 2
    flops = 4.0 * dim * heads * calls * rows * keys_per_row
    hbm = {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peak_hbm, "unit": "GB/s", "frac": nbytes / ms / 1e6 / peak_hbm}
    tensor = {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": peak_tensor, "unit": "TFLOP/s", "frac": flops / ms / 1e9 / peak_tensor}
    # 32 flop per byte at 16 heads, 256 at 128: the bound is the one whose floor is the longer
    entry.update({"ms": ms, "tokens_per_s": calls * rows / ms * 1e3, "roofline": hbm if nbytes / peak_hbm / 1e3 > flops / peak_tensor / 1e6 else tensor,
                  "roofline_hbm": hbm, "roofline_tensor": tensor, "peak_source": peak_source})
    for b in buffers + [sinks, pb, comp]:
        gpu.release(b)
    if own or ref:
        gpu.close()
    return entry


def run_head_sharded(args, rank, world, local, gpu):
    """Config 3 on N GPUs: the 128 heads are dealt over the ranks, every rank holds the latent cache (it is shared by all heads), and
    a rank's outputs [32][128 / N][576] reach every GPU's gathered buffer [N][32][128 / N][576]: by the kernel's own peer stores
    over NVLink (the product) and, beside it, by an NCCL all-gather on the library's stream right behind the kernel."""
    import torch
    import torch.distributed as dist
    from straydog_b200 import sharding
    all_heads = 128
    first, heads = sharding.head_range(all_heads, rank, world)
    context = args.context or 65536
    inp = latent_inputs(gpu, 3, all_heads, context, local)   # (the same seeded inputs on every rank)
    rows, window, dim, selections, variants, total_rows, scale = (inp[k] for k in ("rows", "window", "dim", "selections", "variants", "total_rows", "scale"))
    comp = inp["comp"]
    qb, rb = gpu.upload(np.ascontiguousarray(inp["q"][0][:, first:first + heads])), gpu.upload(inp["raw"][0])
    sb = [gpu.upload(inp["selected"][v]) for v in range(variants)]
    pb, kb = gpu.upload(inp["positions"]), gpu.upload(np.full(heads, -1e30, np.float32))
    shard = gpu.buffer(rows * heads * dim * 4)
    device = torch.device("cuda", local)
    stream = torch.cuda.ExternalStream(gpu.stream(), device=device)
    shard_t = torch.as_tensor(DeviceArray(shard.pointer, rows * heads * dim), device=device)
    full_t = torch.empty(world * rows * heads * dim, dtype=torch.float32, device=device)
    turn = [0]

    def attend():
        turn[0] = (turn[0] + 1) % variants
        gpu.sparse_attention(qb.pointer, rb.pointer, rows, pb.pointer, window, (comp.tagged_bf16(), total_rows), (sb[turn[0]].pointer, selections),
                             kb.pointer, rows, heads, dim, scale, None, None, shard.pointer)

    def with_nccl():
        attend()
        with torch.cuda.stream(stream):
            dist.all_gather_into_tensor(full_t, shard_t)

    def region(fn, steps):
        for _ in range(5):
            fn()
        gpu.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = gpu.event(), gpu.event()
        gpu.record(start)
        for _ in range(steps):
            fn()
        gpu.record(stop)
        gpu.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        return gpu.elapsed_ms(start, stop) / steps

    # the fused form: two gathered buffers taken in turn, so that a rank that is a step ahead never stores into a buffer its
    # peers' consumers may still read (sdx_sparse_attention_gather's rule)
    fulls = [gpu.buffer(world * rows * heads * dim * 4) for _ in range(2)]
    flags = gpu.buffer(world * 4)
    tokens = [None] * world
    dist.all_gather_object(tokens, ([gpu.ipc_export(f) for f in fulls], gpu.ipc_export(flags)))
    outs = [[fulls[b].pointer if r == rank else gpu.ipc_open(tokens[r][0][b], fulls[b].size) for r in range(world)] for b in range(2)]
    counters = [flags.pointer if r == rank else gpu.ipc_open(tokens[r][1], flags.size) for r in range(world)]
    calls = [0]

    def fused():
        turn[0] = (turn[0] + 1) % variants
        calls[0] += 1
        gpu.sparse_attention_gather(qb.pointer, rb.pointer, rows, pb.pointer, window, (comp.tagged_bf16(), total_rows),
                                    (sb[turn[0]].pointer, selections), kb.pointer, rows, heads, dim, scale, None, rank, outs[sharding.gathered_buffer_of(calls[0])], counters, calls[0])

    steps = 400
    sampler = ClockSampler(local)
    ms_attention, ms_nccl, ms_fused = region(attend, steps), region(with_nccl, steps), region(fused, steps)
    clocks = sampler.stop()
    clocks["note"] = "nvidia-smi every 100 ms on rank 0's GPU over the three timed regions"
    status = gpu.decode_status()
    (ms_attention, ms_nccl, ms_fused), (bad,) = sharding.whole_job([ms_attention, ms_nccl, ms_fused], [float(status != 0)], device="cuda")
    fused_result = gpu.read(fulls[sharding.gathered_buffer_of(calls[0])], np.float32, (world, rows, heads, dim)).transpose(1, 0, 2, 3).reshape(rows, world * heads, dim)
    fused_turn = turn[0]
    with_nccl()   # (the NCCL form once more, for the comparison below)
    nccl_turn = turn[0]
    gpu.synchronize()
    torch.cuda.synchronize()
    gathered = sharding.heads_from_gathered(full_t.view(world, rows, heads, dim)).cpu().numpy()
    entry = None
    if rank == 0:
        samples = lambda t: [(0, t, 0, 0), (0, t, 5, 77), (0, t, rows - 1, all_heads - 1), (0, t, 17, all_heads // world)]
        ok_f, worst_fused = latent_error(inp, fused_result[None], samples(fused_turn))
        ok_n, worst_nccl = latent_error(inp, gathered[None], samples(nccl_turn))
        peak_hbm, _, peak_source = measured_peaks()
        nbytes = rows * selections * dim * 2
        entry = {"workload": "config 3: latent sparse decode, 32 queries x top-2048 of 65536, 576-wide BF16 rows; the 128 heads dealt over the GPUs, "
                             "every GPU ends with all outputs", "ranks": world, "heads_per_gpu": heads, "steps": steps,
                 "ms_attention_only": ms_attention, "ms_fused": ms_fused, "ms_nccl_all_gather": ms_nccl,
                 "tokens_per_s_fused": rows / ms_fused * 1e3, "gathered_bytes_per_gpu": int(rows * heads * dim * 4 * (world - 1)),
                 "roofline_hbm_attention_only": {"bound": "hbm", "achieved": nbytes / ms_attention / 1e6, "peak": peak_hbm, "unit": "GB/s",
                                                 "frac": nbytes / ms_attention / 1e6 / peak_hbm},
                 "max_abs_error_vs_oracle_fused": worst_fused, "max_abs_error_vs_oracle_nccl": worst_nccl, "parity": bool(ok_f and ok_n),
                 "ranks_with_a_wait_that_gave_up": int(bad), "timing": "device events on the library's stream, max over ranks", "clocks": clocks,
                 "l2": "steps rotate over 4 index lists (302 MB of rows against the 126 MB L2)", "peak_source": peak_source}
    dist.barrier()
    for b in range(2):
        for r in range(world):
            if r != rank:
                gpu.ipc_close(outs[b][r])
    for r in range(world):
        if r != rank:
            gpu.ipc_close(counters[r])
    dist.barrier()
    for b in [qb, rb, pb, kb, shard, flags, comp] + sb + fulls:
        gpu.release(b)
    return entry


def run_strong(gpu, rank, world, states, contexts, lengths, q_np, barrier):
    """Config 1 as BASELINE words it: the ONE 64-sequence batch dealt over the ranks longest first (every rank holds the same seeded
    lengths, so a rank's share is a subset of the states it already has)."""
    from straydog_b200.sharding import whole_job
    from straydog_b200.synthetic import partition_longest_first
    mine = partition_longest_first(lengths, world)[rank]
    q = gpu.upload(np.ascontiguousarray(q_np[mine]))
    out = gpu.buffer(max(1, len(mine)) * HEADS * DIM * 4)
    my_lengths = [lengths[i] for i in mine]
    plan = gpu.qsa_plan([states[i] for i in mine], [contexts[i] for i in mine], my_lengths, HEADS, KV_HEADS)
    steps = 500
    for _ in range(20):
        gpu.qsa_plan_run(plan, SCALE, q.pointer, out.pointer)
    gpu.synchronize()
    barrier()
    start, stop = gpu.event(), gpu.event()
    gpu.record(start)
    for _ in range(steps):
        gpu.qsa_plan_run(plan, SCALE, q.pointer, out.pointer)
    gpu.record(stop)
    gpu.synchronize()
    barrier()
    ms = gpu.elapsed_ms(start, stop) / steps
    my_bytes = sum(my_lengths) * 2 * KV_HEADS * ROW
    (ms_max,), (total_bytes, total_sequences) = whole_job([ms], [float(my_bytes), float(len(mine))], device="cuda")
    (bytes_max,), _ = whole_job([float(my_bytes)], [0.0], device="cuda")
    gpu.qsa_plan_release(plan)
    gpu.release(q)
    gpu.release(out)
    return {"workload": "config 1, strong: one 64-sequence batch dealt over the ranks longest first by K/V bytes", "ranks": world, "steps": steps,
            "value": total_bytes / ms_max / 1e6, "unit": UNIT, "ms_per_step": ms_max, "tokens_per_s": total_sequences / ms_max * 1e3,
            "max_over_mean_bytes_per_rank": bytes_max / (total_bytes / world), "timing": "device events, max over ranks"}


def run_config1_reference_gpu(args):
    """The reference's own kernels on config 1's batch: sd_op_attention (gpu/token_mixing.hpp:652) over each sequence's dequantised F32
    K/V [context][kv_heads][256], one call a sequence (the reference ABI holds one sequence a call)."""
    import oracle
    lengths, seeds = batch_for(0, 1, "weak", args.sequences)
    gpu = reference_gpu_backend(sum(lengths) * KV_HEADS * DIM * 4 * 2 + (4 << 30))
    from straydog_b200.synthetic import queries_f16
    rng = np.random.default_rng(SEED + 7)
    q_np = queries_f16(rng, len(lengths), HEADS, DIM).astype(np.float32)
    calls = []
    for s, (length, seed) in enumerate(zip(lengths, seeds)):
        state = make_states([length], [seed])[0]
        planes = oracle.q8_decode_rows(state.reshape(-1, ROW)).reshape(2 * KV_HEADS, length, DIM)
        kb = gpu.upload(np.ascontiguousarray(planes[:KV_HEADS].transpose(1, 0, 2)))
        vb = gpu.upload(np.ascontiguousarray(planes[KV_HEADS:].transpose(1, 0, 2)))
        calls.append((kb, vb, gpu.upload(q_np[s]), gpu.upload(np.array([length - 1], np.int32)), gpu.buffer(HEADS * DIM * 4), length))
    scratch = gpu.buffer(HEADS * 64 * (DIM + 2) * 4)

    def step():
        for kb, vb, qb, pb, out, length in calls:
            gpu.attention(qb.pointer, kb.pointer, vb.pointer, length, pb.pointer, 1, HEADS, KV_HEADS, DIM, SCALE, None, scratch, out.pointer)
    ms = host_timed(gpu, step, calls[-1][4], args.steps)
    kv_bytes = sum(lengths) * 2 * KV_HEADS * ROW
    print(json.dumps({"config_id": 1, "impl": "reference-gpu", "workload": workload_config(lengths)["workload"] + "; the reference's sd_op_attention "
                      "over the dequantised F32 K/V, one call a sequence", "ms": ms, "kv_gbps_q8_equivalent": kv_bytes / ms / 1e6,
                      "f32_bytes_read_gbps": sum(lengths) * KV_HEADS * DIM * 4 * 2 / ms / 1e6, "tokens_per_s": len(lengths) / ms * 1e3, "steps": args.steps}), flush=True)
    gpu.close()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    parser.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4], help="1 is the benchmark line; another number prints that configuration's entry alone")
    parser.add_argument("--context", type=int, default=0, help="configs 3/4: override the per-query context (a smaller resident set for a profiler capture)")
    parser.add_argument("--head-shards", type=int, default=1, help="configs 3/4: heads per GPU = 128 / head_shards (the per-GPU work of head sharding)")
    parser.add_argument("--per-call", action="store_true", help="config 4: one sd_op_sparse_attention call per sequence instead of one sdx_sparse_attention_spans launch")
    parser.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    parser.add_argument("--cpu-seconds", type=float, default=12.0)
    parser.add_argument("--sequences", type=int, default=64, help="sequences per batch (64 is the benchmark; fewer for a profiler capture)")
    parser.add_argument("--profile", action="store_true", help="device-resident steps only, no load padding: the command an ncu capture wraps")
    parser.add_argument("--no-extras", action="store_true", help="the headline alone: no other configuration, no strong / head-sharded curve")
    parser.add_argument("--index-ops", action="store_true", help="the index producers' entry alone (sd_op_top_k, sd_op_index_select): the command an ncu capture wraps")
    parser.add_argument("--fixed-cuts", action="store_true", help="the decode work list cut by each sequence's own length (same bits in any batch)")
    args = parser.parse_args()
    args.steps_given = args.steps is not None
    if args.steps is None:
        args.steps = 50
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.impl == "reference-gpu":
        if rank == 0:
            if args.config == 1:
                run_config1_reference_gpu(args)
            else:
                entry = run_qsa_config(args.config, args, 0) if args.config in (0, 2) else run_latent_config(args.config, args, 0)
                print(json.dumps({"config_id": args.config, **entry}), flush=True)
        return
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU: the attention library has no CPU fallback")
    if args.index_ops:
        if rank == 0:
            from straydog_b200.backend import Backend
            torch.cuda.set_device(local)
            gpu = Backend(local, 2 << 30)
            print(json.dumps({"config_id": "index_ops", **run_index_ops(args, local, gpu)}), flush=True)
            gpu.close()
        return
    if args.config != 1:
        if rank == 0:
            torch.cuda.set_device(local)
            entry = run_qsa_config(args.config, args, local) if args.config in (0, 2) else run_latent_config(args.config, args, local)
            print(json.dumps({"config_id": args.config, **entry}), flush=True)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch.distributed as dist
    from straydog_b200.backend import Backend, lib, _check
    from straydog_b200.sharding import whole_job
    from straydog_b200.synthetic import queries_f16
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    barrier_token = torch.zeros(1, device="cuda")

    def barrier():
        if world > 1:
            dist.all_reduce(barrier_token)
        torch.cuda.synchronize()

    lengths, seeds = batch_for(rank, world, args.scaling, args.sequences)
    kv_bytes = sum(lengths) * 2 * KV_HEADS * ROW
    e2e_steps = args.steps + args.warmup
    slack = e2e_steps + 8   # room for the rows the end-to-end steps append
    gpu = Backend(local, kv_bytes + len(lengths) * slack * 2 * KV_HEADS * ROW + (24 << 30))
    if args.fixed_cuts:
        gpu.decode_cuts(True)
    states_np = make_states(lengths, seeds, slack)
    contexts = [l + slack for l in lengths]
    states = []
    for s in states_np:
        buffer = gpu.allocate(s.nbytes)
        gpu.write(buffer, s)
        states.append(buffer)
    n = len(lengths)
    rng = np.random.default_rng(SEED + 7 + rank)
    q_np = queries_f16(rng, n, HEADS, DIM)
    q = gpu.upload(q_np)
    out = gpu.buffer(n * HEADS * DIM * 4)
    plan = gpu.qsa_plan(states, contexts, lengths, HEADS, KV_HEADS)
    info = gpu.qsa_plan_info(plan)

    def step():
        gpu.qsa_plan_run(plan, SCALE, q.pointer, out.pointer)

    # ---- device-resident: K steps of the planned decode (two kernel launches each) ----
    if args.profile:
        for _ in range(args.warmup + args.steps):
            step()
        gpu.synchronize()
        print(json.dumps({"profile": True, "plan": info, "launches": gpu.launch_count()}))
        gpu.qsa_plan_release(plan)
        gpu.close()
        return
    sampler = ClockSampler(local)
    for _ in range(args.warmup):
        step()
    gpu.synchronize()

    def load_for(seconds, until_samples=None):
        """Untimed back-to-back steps: the clock samples bracket the timed region under the same load."""
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < seconds and (until_samples is None or sampler.count() < until_samples):
            for _ in range(20):
                step()
            gpu.synchronize()
    load_for(3.0, until_samples=2)
    start, stop = gpu.event(), gpu.event()
    barrier()
    launches_before = gpu.launch_count()
    gpu.record(start)
    for _ in range(args.steps):
        step()
    gpu.record(stop)
    gpu.synchronize()
    launches = gpu.launch_count() - launches_before
    barrier()
    device_ms = Backend.elapsed_ms(start, stop)
    # the streaming kernel alone, right behind the timed region under the same load: events recorded inside the library around that
    # kernel on its stream (an event between the two launches keeps the merge from being placed early, so these steps are not the
    # timed ones)
    marks = [(gpu.event(), gpu.event()) for _ in range(args.steps)]
    for before, after in marks:
        gpu.qsa_plan_run_marked(plan, SCALE, q.pointer, out.pointer, before, after)
    gpu.synchronize()
    kernel_ms = [Backend.elapsed_ms(b, a) for b, a in marks]
    # per-step times over 500 further steps (an event after every step)
    ticks = [gpu.event() for _ in range(501)]
    gpu.record(ticks[0])
    for tick in ticks[1:]:
        step()
        gpu.record(tick)
    gpu.synchronize()
    per_step = sorted(Backend.elapsed_ms(a, b) for a, b in zip(ticks[:-1], ticks[1:]))
    load_for(0.3)
    clocks = sampler.stop()
    clocks["note"] = ("nvidia-smi every 100 ms over the untimed back-to-back steps just before the timed region, the region itself, the kernel-only "
                      "steps and the 500 per-step timings behind it")
    if gpu.decode_status() != 0:
        raise SystemExit("a bounded wait inside the decode kernel gave up: the result is invalid")
    got_all = gpu.read(out, np.float32, (n, HEADS, DIM))

    # ---- end to end: host buffers in, host buffers out, a new position every step (as a decode loop appends) ----
    q_host = torch.from_numpy(q_np.view(np.int16).copy()).pin_memory()
    k_host = torch.from_numpy(rng.normal(0, 1, (n, KV_HEADS, DIM)).astype(np.float32)).pin_memory()
    v_host = torch.from_numpy(rng.normal(0, 1, (n, KV_HEADS, DIM)).astype(np.float32)).pin_memory()
    out_host = torch.empty((n, HEADS, DIM), dtype=torch.float32).pin_memory()
    ptrs = (C.c_void_p * n)(*[s.pointer for s in states])
    ctx = (C.c_uint64 * n)(*contexts)
    position = [0]
    # (the positions of every step, laid out before the clock starts: an engine keeps its arrays, it does not rebuild them in Python)
    bases_of_step = [(C.c_uint64 * n)(*[l + p for l in lengths]) for p in range(args.warmup + args.steps)]
    batch_entry = lib().sdx_attention_batch
    q_ptr, k_ptr, v_ptr, out_ptr = q_host.data_ptr(), k_host.data_ptr(), v_host.data_ptr(), out_host.data_ptr()

    def e2e_step():
        bs = bases_of_step[position[0]]
        position[0] += 1
        _check(batch_entry(gpu.handle, ptrs, ctx, bs, n, HEADS, KV_HEADS, SCALE, q_ptr, k_ptr, v_ptr, out_ptr))
    for _ in range(args.warmup):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    e2e_bytes = float(kv_bytes + n * 2 * KV_HEADS * ROW * (args.warmup + (args.steps + 1) / 2))   # a step's mean (the contexts grow by one a step)

    # ---- max over ranks, sums over ranks ----
    (device_ms_max, e2e_ms_max, kernel_ms_mean), (total_bytes, total_sequences, total_e2e_bytes) = whole_job(
        [device_ms, e2e_s * 1e3, statistics.mean(kernel_ms)], [float(kv_bytes), float(n), e2e_bytes], device="cuda")

    line = None
    if rank == 0:
        import oracle
        peak, _, peak_source = measured_peaks()
        value = total_bytes * args.steps / (device_ms_max / 1e3) / 1e9
        achieved = kv_bytes / (statistics.mean(kernel_ms) / 1e3) / 1e9
        # the CPU baseline is timed at N = 1 only (a multi-rank run shares the host's cores with the other ranks)
        cpu_gbps, cpu_used, cpu_bytes, cpu_spent, cpu_threads = cpu_sample(lengths, seeds, args.cpu_seconds) if world == 1 else (None, 0, 0, 0.0, 0)
        # parity of the timed output against the oracle, every sequence of this rank's batch: a wrong kernel cannot post a number
        oracle.set_threads(os.cpu_count() or 1)
        want_all = np.stack([oracle.gqa_decode_q8(states_np[s], contexts[s], lengths[s], HEADS, KV_HEADS, q_np[s], SCALE, f64=True) for s in range(n)])
        ok, error = within_tolerance(got_all, want_all)
        if not ok:
            raise SystemExit(f"the timed output differs from the oracle beyond the tolerance (max abs error {error})")
        pick = lambda f: per_step[min(len(per_step) - 1, int(f * len(per_step)))]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": device_ms_max / args.steps, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16 x int8 products, f32 accumulate", "data": "synthetic (seeded)",
            "config": workload_config(lengths),
            "tokens_per_s": total_sequences * args.steps / (device_ms_max / 1e3),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         # DRAM bytes a launch: the ncu capture of a 16-sequence case read and wrote 1.022 x its algorithmic bytes
                         # (the extra is the split partials); traffic grows with the K/V bytes, so it is scaled to this launch
                         "traffic": kv_bytes * 1.022, "traffic_source": "ncu dram__bytes of a 16-sequence launch (226.2 MB for 220.9 MB), scaled by K/V bytes",
                         "peak_source": peak_source, "kernel": "qsa_decode_kernel", "kernel_ms": statistics.mean(kernel_ms),
                         "kernel_ms_source": f"{args.steps} steps with events around the kernel, directly behind the timed region",
                         "frac_of_nominal_8tbs": achieved / 8000.0},
            "cpu_baseline": ({"value": cpu_gbps, "unit": UNIT, "cores": cpu_threads, "kind": "port",
                              "sample": f"first {cpu_used} of {n} sequences ({cpu_bytes} K/V bytes, {cpu_spent:.1f} s)"} if world == 1 else None),
            "e2e": {"value": total_e2e_bytes * args.steps / (e2e_ms_max / 1e3) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": int(q_host.nbytes + k_host.nbytes + v_host.nbytes), "d2h_bytes_per_step": int(out_host.nbytes),
                    "ms_per_step": e2e_ms_max / args.steps, "tokens_per_s": total_sequences * args.steps / (e2e_ms_max / 1e3),
                    "note": "sdx_attention_batch from pinned host buffers; every step appends a row at a new position; the entry keeps its work list from step to step (new tiles join a sequence's last piece, a new list every 8 tiles of growth)"},
            "gpu_launches": int(launches), "clocks": clocks, "plan": info, "cuts": "fixed" if args.fixed_cuts else "moving",
            "max_abs_error_vs_oracle": error, "sequences_checked": n,
            "step_ms_percentiles": {"p10": pick(0.10), "p50": pick(0.50), "p90": pick(0.90), "steps": len(per_step),
                                    "note": "an event after every step (which costs each step a little)"},
        }
    extras = not args.no_extras and args.sequences == 64
    if extras and world > 1:
        strong = run_strong(gpu, rank, world, states, contexts, lengths, q_np, barrier)
        if rank == 0:
            line["config1_strong"] = strong
    gpu.qsa_plan_release(plan)
    for b in states + [q, out]:
        gpu.release(b)
    if extras:
        if world > 1:
            sharded = run_head_sharded(args, rank, world, local, gpu)
            if rank == 0:
                line["config3_head_sharded"] = sharded
        if rank == 0:
            # the other configurations on rank 0's GPU while the other ranks wait at the barrier below
            shards = 8
            line["configs"] = {
                "0": run_qsa_config(0, args, local, gpu),
                "2": run_qsa_config(2, args, local, gpu),
                "3": run_latent_config(3, args, local, gpu, head_shards=shards),
                "3_128_heads": run_latent_config(3, args, local, gpu, head_shards=1),
                "4": run_latent_config(4, args, local, gpu, head_shards=shards),
                "4_128_heads": run_latent_config(4, args, local, gpu, head_shards=1),
                "index_ops": run_index_ops(args, local, gpu),
                "qsa_rows": run_qsa_rows(args, local, gpu),
            }
    if rank == 0:
        print(json.dumps(line), flush=True)
    barrier()
    gpu.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
