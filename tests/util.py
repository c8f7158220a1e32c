"""Seeded input generators shared by the tests, the smoke test and the benchmark.

Shapes and value distributions follow the five benchmark configurations: Q8_0 K/V rows hold int8
values uniform in [-127, 127] and one FP16 scale per 32-value block drawn as |N(0, 0.02)|; queries are
FP16 N(0, 1); latent rows are BF16 N(0, 0.05). The xorshift generators restate the ones the
reference's GPU tests seed their inputs with (crates/straydog-engine/tests/attention_gpu.rs:10-20,
ds_state_bf16_gpu.rs:13-24), so those tests' exact inputs can be rebuilt.
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
    """The benchmark's tolerance: every output within max-abs 2e-3 or max-rel 1e-2 of the oracle."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    error = np.abs(actual - expected)
    ok = (error <= atol) | (error <= rtol * np.abs(expected))
    return bool(np.all(ok) and np.all(np.isfinite(actual))), float(error.max())
