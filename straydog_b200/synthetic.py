"""Seeded synthetic inputs of the benchmark configurations, shared by the tests, the smoke test and bench.py.

Q8_0 K/V rows hold int8 values uniform in [-127, 127] and one FP16 scale per 32-value block drawn as
|N(0, 0.02)|; queries are FP16 N(0, 1); latent rows are BF16 N(0, 0.05). The xorshift generators
restate the ones the reference's GPU tests seed their inputs with
(crates/straydog-engine/tests/attention_gpu.rs:10-20, ds_state_bf16_gpu.rs:13-24), so that those
tests' exact inputs can be rebuilt.
"""
import numpy as np

ROW_Q8 = 272
M64 = (1 << 64) - 1


def q8_state(rng, context, kv_heads, filled=None):
    """uint8 [2*kv_heads, context, 272]: rows 0..filled-1 random, the rest zero."""
    filled = context if filled is None else filled
    state = np.zeros((2 * kv_heads, context, ROW_Q8), np.uint8)
    values = rng.integers(-127, 128, size=(2 * kv_heads, filled, 256), dtype=np.int8)
    scales = np.abs(rng.normal(0.0, 0.02, size=(2 * kv_heads, filled, 8))).astype(np.float16)
    state[:, :filled, :256] = values.view(np.uint8)
    state[:, :filled, 256:] = scales.view(np.uint8).reshape(2 * kv_heads, filled, 16)
    return state


def queries_f16(rng, *shape):
    return rng.normal(0.0, 1.0, size=shape).astype(np.float16)


def bf16_round(x):
    """float32 array -> (uint16 BF16 bits, float32 widened), round to nearest even."""
    bits = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    halves = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    return halves, (halves.astype(np.uint32) << 16).view(np.float32)


def unique_sorted_indices(rng, rows, count, limit):
    out = np.empty((rows, count), np.int32)
    for r in range(rows):
        out[r] = np.sort(rng.choice(limit, size=count, replace=False)).astype(np.int32)
    return out


class XorShift:
    """The reference tests' xorshift64 (13, 7, 17)."""

    def __init__(self, seed):
        self.s = seed & M64

    def next(self):
        s = self.s
        s ^= (s << 13) & M64
        s ^= s >> 7
        s ^= (s << 17) & M64
        self.s = s
        return s

    def floats_unit(self, count):
        """attention_gpu.rs: (state >> 40) / 2^23 - 1, in [-1, 1)."""
        return np.array([np.float32(self.next() >> 40) / np.float32(1 << 23) - np.float32(1.0) for _ in range(count)], np.float32)

    def floats_scaled(self, count, scale):
        """ds_state_bf16_gpu.rs: ((next % 2e6) / 1e6 - 1) * scale."""
        return np.array([(np.float32(self.next() % 2_000_000) / np.float32(1_000_000.0) - np.float32(1.0)) * np.float32(scale)
                         for _ in range(count)], np.float32)


def close(actual, expected, atol=2e-3, rtol=1e-2):
    """The benchmark's tolerance: every output within max-abs 2e-3 or max-rel 1e-2 of the oracle. Returns (ok, max abs error)."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    error = np.abs(actual - expected)
    ok = (error <= atol) | (error <= rtol * np.abs(expected))
    return bool(np.all(ok) and np.all(np.isfinite(actual))), float(error.max())


def ragged_lengths(seed, sequences=64, low=1024, high=32768):
    """Context lengths of the ragged decode batch: uniform in [low, high], seeded."""
    return [int(x) for x in np.random.default_rng(seed).integers(low, high + 1, sequences)]


def partition_longest_first(lengths, parts):
    """Greedy longest-first bin packing of sequences over `parts` ranks; returns a list of index lists."""
    bins = [[] for _ in range(parts)]
    loads = [0] * parts
    for index in sorted(range(len(lengths)), key=lambda i: -lengths[i]):
        target = loads.index(min(loads))
        bins[target].append(index)
        loads[target] += lengths[index]
    return [sorted(b) for b in bins]


# ---- inputs of the reference's own model-free GPU tests, rebuilt from their seeds ----
def attention_sequence_input(rng, steps, selected, base, context, kind, heads=24, kv_heads=2):
    """The packed F32 input of sd_attention_sequence: q | k | v | positions as floats | counts as floats."""
    q = rng.normal(0, 1, (steps, heads, 256)).astype(np.float32)
    k = rng.normal(0, 1, (steps, kv_heads, 256)).astype(np.float32)
    v = rng.normal(0, 1, (steps, kv_heads, 256)).astype(np.float32)
    idx = np.zeros((steps, selected), np.float32)
    counts = np.zeros(steps, np.float32)
    for s in range(steps):
        limit = base + s
        if kind == "dense":
            n = min(selected, limit + 1)
            idx[s, :n] = np.arange(limit + 1 - n, limit + 1)
        else:   # sparse: unsorted, with dead slots (negative, future, past the context)
            n = selected
            idx[s] = rng.integers(0, limit + 1, selected)
            idx[s, ::7] = -1
            idx[s, 3::11] = limit + 1 + rng.integers(0, 5)
            idx[s, 5::13] = context + 3
            idx[s, 0] = limit     # its own position: written by this call
        counts[s] = n
    return np.concatenate([q.ravel(), k.ravel(), v.ravel(), idx.ravel(), counts]).astype(np.float32)


def op_attention_case(rows, heads, kv_heads, dim, context, zero_queries=False):
    """crates/straydog-engine/tests/attention_gpu.rs:89-104: the inputs of check(shape, zero_queries)."""
    random = XorShift(0x9E3779B97F4A7C15 ^ rows ^ (dim << 16))
    q = random.floats_unit(rows * heads * dim)
    if zero_queries:
        q[:] = 0
    keys = random.floats_unit(context * kv_heads * dim)
    values = random.floats_unit(context * kv_heads * dim)
    special = [0, 1, 15, 16, context - 1, context + 7]
    positions = np.array([special[r] if r < len(special) else (r * 17 + 3) % context for r in range(rows)], np.int32)
    gate = np.array([[-12.0, -1.0, 0.0, 1.0, 12.0][i % 5] for i in range(q.size)], np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(dim)))
    return dict(q=q, keys=keys, values=values, positions=positions, gate=gate, scale=scale)


def sparse_attention_case(rows, heads):
    """crates/straydog-engine/tests/ds_state_bf16_gpu.rs:66-80: the inputs of attention(rows, heads, _)."""
    dim, window, raw_rows, compressed_rows, selections, rope_dims = 512, 128, 256, 300, 512, 64
    random = XorShift(0x9E3779B9 ^ (rows * 131 + heads))
    q = random.floats_scaled(rows * heads * dim, 1.0)
    raw = random.floats_scaled(raw_rows * dim, 1.0)
    halves, widened = bf16_round(random.floats_scaled(compressed_rows * dim, 1.0))
    sinks = random.floats_scaled(heads, 2.0)
    freq = np.array([np.float32(10000.0) ** np.float32(-(2.0 * i) / rope_dims) for i in range(rope_dims // 2)], np.float32)
    positions = np.array([1000 + r for r in range(rows)], np.int32)
    selected = np.array([-1 if at % 37 == 5 else int(random.next() % compressed_rows) for at in range(rows * selections)], np.int32)
    return dict(q=q, raw=raw, halves=halves, widened=widened, sinks=sinks, freq=freq, positions=positions, selected=selected,
                dim=dim, window=window, raw_rows=raw_rows, compressed_rows=compressed_rows, selections=selections, rope_dims=rope_dims,
                rows=rows, heads=heads, scale=float(np.float32(1.0) / np.sqrt(np.float32(dim))))


def latent_decode_case(seed, rows, heads, dim, context, selections):
    """The benchmark's DeepSeek-style decode at any size: BF16 latent rows N(0, 0.05) per query's own cache, unique sorted
    top-k indices, BF16-exact queries N(0, 1), window 1 (the query's own row as F32), sinks -inf, no rope."""
    rng = np.random.default_rng(seed)
    halves, widened = bf16_round(rng.normal(0, 0.05, (rows * context, dim)).astype(np.float32))
    _, q = bf16_round(rng.normal(0, 1, (rows, heads, dim)).astype(np.float32))
    raw = widened.reshape(rows, context, dim)[:, -1].copy()
    selected = np.stack([np.sort(rng.choice(context, selections, replace=False)) + r * context for r in range(rows)]).astype(np.int32)
    return dict(q=q, raw=raw, halves=halves, sinks=np.full(heads, -np.inf, np.float32), freq=np.zeros(1, np.float32),
                positions=np.arange(rows, dtype=np.int32), selected=selected, dim=dim, window=1, raw_rows=rows,
                compressed_rows=rows * context, selections=selections, rope_dims=0, rows=rows, heads=heads,
                scale=float(np.float32(1.0) / np.sqrt(np.float32(dim))))


def dspark_case():
    """crates/straydog-engine/tests/dspark_attention_gpu.rs:56-63: the inputs of its main test (xorshift64 floats in [-scale, scale))."""
    random = XorShift(0x9E3779B97F4A7C15)

    def floats(count, scale):
        return np.array([(np.float32(random.next() >> 40) / np.float32(1 << 24) - np.float32(0.5)) * np.float32(2.0) * np.float32(scale)
                         for _ in range(count)], np.float32)
    q, ring, block, sinks = floats(5 * 64 * 512, 0.3), floats(128 * 512, 0.4), floats(5 * 512, 0.6), floats(64, 2.0)
    sinks[0::16] = 30.0
    sinks[1::16] = -30.0
    return dict(q=q.reshape(5, 64, 512), ring=ring.reshape(128, 512), block=block.reshape(5, 512), sinks=sinks)


INDEX_CASES = [(1, 3000), (4, 2000), (1, 300)]          # crates/straydog-engine/tests/fused_gpu.rs:399
TWO_LEVEL_CASES = [(1, 6000, 256, 8), (3, 5001, 1024, 8)]   # (rows, groups, blocks, block): the second keeps every block (626 < 1024)


def index_case(rows, groups, heads=32, dim=128, rope_dims=64, spread=3, seed=0):
    """crates/straydog-engine/tests/fused_gpu.rs:391-412 in shape and value ranges (q in [-2, 2), keys and weights in [-1, 1), rope
    frequencies 1.6e5 ^ (-2 i / rope), visible = groups - spread * row, positions 20000 + 7 * row, scale 1 / (sqrt(dim) sqrt(heads))),
    seeded here."""
    rng = np.random.default_rng([rows, groups, heads, dim, seed])
    frequencies = np.array([np.float32(1.6e5) ** (np.float32(-2.0 * i) / np.float32(rope_dims)) for i in range(rope_dims // 2)], np.float32)
    return dict(q=rng.uniform(-2, 2, (rows, heads, dim)).astype(np.float32), keys=rng.uniform(-1, 1, (groups, dim)).astype(np.float32),
                weights=rng.uniform(-1, 1, (rows, heads)).astype(np.float32), visible=np.array([groups - spread * r for r in range(rows)], np.int32),
                positions=np.array([20000 + 7 * r for r in range(rows)], np.int32), frequencies=frequencies, rows=rows, groups=groups, heads=heads,
                dim=dim, rope_dims=rope_dims, scale=float(np.float32(1.0) / (np.sqrt(np.float32(dim)) * np.sqrt(np.float32(heads)))))


# (weight kind, columns, heads, groups, bytes the input is pushed off 16-byte alignment): F32, F16 and BF16 matrices whose rows a warp sums in
# 16-byte units, a width that is no whole number of units and an input off alignment (both take the element path)
INDEX_PROJ_CASES = [(30, 4096, 64, 4096, 0), (30, 2560, 32, 1000, 0), (0, 2560, 32, 4096, 0), (1, 4096, 64, 1000, 0), (30, 2052, 32, 600, 0),
                    (0, 514, 32, 600, 0), (1, 1024, 32, 600, 4)]


def index_proj_case(kind, cols, heads, groups, seed=0):
    """sd_op_index_select_proj's inputs: index_case of one row plus the projection W [heads][cols] (kind 0: F32; 1: F16 bits; 30: BF16 bits, both
    as uint16) and its input x [cols]; the head weights are what the call computes."""
    c = index_case(1, groups, heads=heads, seed=seed + 100)
    rng = np.random.default_rng([kind, cols, heads, groups, seed])
    w = rng.uniform(-1, 1, (heads, cols)).astype(np.float32)
    if kind == 1:
        w = w.astype(np.float16).view(np.uint16)
    elif kind == 30:
        w = bf16_round(w)[0]
    c.update(proj=np.ascontiguousarray(w), proj_kind=kind, proj_cols=cols, x=rng.uniform(-1, 1, cols).astype(np.float32))
    return c


# (context, position, steps, seed): a prompt's first chunk (every position listed); a decode step that completes a block with 751 blocks to
# choose from; a chunk of five tokens across a block's end with the choice running; a decode step in the middle of a block; a decode step that
# lists every position (375 blocks): the dense decode of 1501 positions; a prompt chunk of 60 tokens after 100 cached (every position listed: the
# dense causal prompt attention)
QSA_SEQUENCE_CASES = [(256, 0, 7, 1), (4096, 3003, 1, 2), (4096, 3001, 5, 3), (8192, 5001, 1, 4), (2048, 1500, 1, 5), (1024, 100, 60, 6)]
QSA_HIDDEN, QSA_HEADS, QSA_KV_HEADS = 2560, 24, 2
# a projection's row r reads input column (r * a + b) % 2560 (weight 1, the rest of the row 0): the reference's own layer call
# (sd_qsa_sequence) then projects exactly, whatever order its GEMV sums in, and everything behind the projections is its kernels' arithmetic
QSA_SELECTORS = dict(qgate=(12288, 7, 3), key=(512, 11, 5), value=(512, 13, 17), iq=(512, 17, 29), ik=(128, 19, 31))


def qsa_selection_matrix(name):
    rows, a, b = QSA_SELECTORS[name]
    w = np.zeros((rows, QSA_HIDDEN), np.float32)
    w[np.arange(rows), (np.arange(rows) * a + b) % QSA_HIDDEN] = 1.0
    return w


def qsa_output_matrix():
    """[2560][6144]: output i = attended value i (the first ten heads' 256 columns each)."""
    w = np.zeros((QSA_HIDDEN, QSA_HEADS * 256), np.float32)
    w[np.arange(QSA_HIDDEN), np.arange(QSA_HIDDEN)] = 1.0
    return w


def qsa_sequence_case(context, position, steps, seed):
    """The inputs of one sd_qsa_sequence call over selection matrices: the layer input x [steps][2560], the four norm vectors, the K/V state
    and the indexer state as the positions before `position` left them (seeded), and the five projections the selection matrices give."""
    rng = np.random.default_rng([context, position, steps, seed])
    pool = context // 4 + 1
    c = dict(context=context, position=position, steps=steps, pool=pool, x=rng.normal(0, 1, (steps, QSA_HIDDEN)).astype(np.float32))
    c["norms"] = [rng.normal(1, 0.1, n).astype(np.float32) for n in (256, 256, 128, 128)]
    c["state"] = q8_state(rng, context, QSA_KV_HEADS, filled=position)
    index_state = np.zeros((pool + 16) * 128, np.float32)
    index_state[:pool * 128].reshape(128, pool)[:, :position // 4] = rng.normal(0, 1, (128, position // 4)).astype(np.float32)
    index_state[pool * 128:] = rng.normal(0, 1, 16 * 128).astype(np.float32)
    c["index_state"] = index_state
    for name, (rows, a, b) in QSA_SELECTORS.items():
        c[name] = np.ascontiguousarray(c["x"][:, (np.arange(rows) * a + b) % QSA_HIDDEN])
    return c


def compress_case(groups=37, ratio=4, dim=128, seed=5):
    rng = np.random.default_rng(seed)
    return dict(kv=rng.uniform(-1, 1, (groups * ratio, dim)).astype(np.float32), gate=rng.uniform(-4, 4, (groups * ratio, dim)).astype(np.float32),
                groups=groups, ratio=ratio, dim=dim)


def tie_scores(random, rows, groups):
    """crates/straydog-engine/tests/fused_gpu.rs:366-377: quarter steps in [-2, 2], -0 beside +0, -inf and +inf."""
    out = np.empty(rows * groups, np.float32)
    for i in range(rows * groups):
        draw = random.next()
        if groups == 600 and draw % 8 != 0:
            out[i] = -np.inf
            continue
        m = draw % 97
        if m <= 6:
            out[i] = -np.inf
        elif m == 7:
            out[i] = np.inf
        elif m == 8:
            out[i] = -0.0
        else:
            out[i] = np.float32((draw >> 8) % 17) * np.float32(0.25) - np.float32(2.0) + (np.float32(0.125) if i % 1000 == 999 else np.float32(0.0))
    return out.reshape(rows, groups)


def qsa_index_case(steps, base, pool, heads=16, kv_heads=2, selected=2052, seed=0, integers=False):
    """Inputs of Qwen's indexer: `steps` rows of four 128-wide index queries, the pooled index keys [128][pool], and packed rows
    (gpu/core.hpp:392) whose list and count parts are to be written. integers: small whole numbers, so that every sum is exact in any
    order and equal scores are common (the tie rule shows)."""
    rng = np.random.default_rng([steps, base, pool, seed])
    if integers:
        queries, blocks = rng.integers(-3, 4, (steps, 512)).astype(np.float32), rng.integers(-2, 3, (128, pool)).astype(np.float32)
    else:
        queries, blocks = rng.normal(0, 1, (steps, 512)).astype(np.float32), rng.normal(0, 1, (128, pool)).astype(np.float32)
    row_floats = heads * 256 + kv_heads * 512
    packed = rng.normal(0, 1, steps * (row_floats + selected + 1)).astype(np.float32)
    return dict(queries=queries, blocks=blocks, packed=packed, row_floats=row_floats, steps=steps, base=base, pool=pool, selected=selected,
                heads=heads, kv_heads=kv_heads)
