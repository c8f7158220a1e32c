"""ctypes binding of the CPU oracle (oracle.cpp). TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs import this
package; the product (straydog_b200) never does.
"""
import ctypes as C

import numpy as np

from . import build as _build

_lib = C.CDLL(_build.build())

_u64, _f32, _i32 = C.c_uint64, C.c_float, C.c_int
_p = C.c_void_p


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_p)


def _sig(name, args, res=None):
    f = getattr(_lib, name)
    f.argtypes, f.restype = args, res
    return f


_sig("orc_f32_to_f16", [_f32], C.c_uint16)
_sig("orc_f16_to_f32", [C.c_uint16], _f32)
_sig("orc_q8_encode_rows", [_p, _u64, _p])
_sig("orc_q8_decode_rows", [_p, _u64, _p])
_sig("orc_kv_write", [_p, _u64, _u64, _u64, _u64, _p, _p])
_sig("orc_attention_sequence", [_p, _u64, _u64, _u64, _u64, _u64, _u64, _p, _f32, _p])
_sig("orc_gqa_decode_q8", [_p, _u64, _u64, _u64, _u64, _p, _f32, _i32, _p])
_sig("orc_gqa_prompt_q8", [_p, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _p, _f32, _i32, _p])
_sig("orc_op_attention", [_p, _p, _p, _u64, _p, _u64, _u64, _u64, _u64, _f32, _p, _p, _p, _p])
_sig("orc_sparse_attention", [_p, _p, _u64, _p, _u64, _p, _i32, _p, _u64, _p, _u64, _u64, _u64, _f32, _u64, _p, _i32, _p])
_sig("orc_dspark_attention", [_p, _p, _p, _p, _u64, _u64, _u64, _u64, _i32, _p])
_sig("orc_rope", [_p, _u64, _u64, _u64, _u64, _p, _p, _i32])
_sig("orc_compress", [_p, _p, _u64, _u64, _u64, _p])
_sig("orc_index_scores", [_p, _p, _i32, _p, _p, _u64, _u64, _u64, _u64, _f32, _p, _u64, _u64, _p])
_sig("orc_index_block_tops", [_p, _p, _u64, _u64, _u64, _p])
_sig("orc_qsa_index_select", [_p, _u64, _p, _u64, _u64, _p, _u64, _u64, _u64, _p])
_sig("orc_qsa_normalize_rows", [_p, _u64, _u64, _u64, _u64, _p, _p, _p, _p, _p, _p, _p, _p, _u64, _p])
_sig("orc_qsa_normalize_chunk", [_p, _p, _p, _p, _p, _u64, _u64, _u64, _u64, _p, _p, _p, _p, _p, _p, _u64, _p, _p, _u64])
_sig("orc_index_proj", [_p, _i32, _u64, _u64, _p, _i32, _p])
_sig("orc_top_k", [_p, _u64, _u64, _u64, _p])
_sig("orc_to_bf16", [_p, _u64, _p])
_sig("orc_threads", [], _i32)
_sig("orc_set_threads", [_i32])

ROW_Q8 = 272
DIM = 256


def threads() -> int:
    return int(_lib.orc_threads())


def set_threads(n: int) -> None:
    _lib.orc_set_threads(int(n))


def f32_to_f16(x: float) -> int:
    return int(_lib.orc_f32_to_f16(x))


def f16_to_f32(h: int) -> float:
    return float(_lib.orc_f16_to_f32(h))


def q8_encode_rows(values: np.ndarray) -> np.ndarray:
    """[rows, 256] F32 -> [rows, 272] uint8 (Q8_0 rows)."""
    values = np.ascontiguousarray(values, np.float32).reshape(-1, DIM)
    out = np.empty((values.shape[0], ROW_Q8), np.uint8)
    _lib.orc_q8_encode_rows(_ptr(values), values.shape[0], _ptr(out))
    return out


def q8_decode_rows(packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, np.uint8).reshape(-1, ROW_Q8)
    out = np.empty((packed.shape[0], DIM), np.float32)
    _lib.orc_q8_decode_rows(_ptr(packed), packed.shape[0], _ptr(out))
    return out


def kv_write(state: np.ndarray, context: int, kv_heads: int, base: int, keys: np.ndarray, values: np.ndarray) -> None:
    """state: uint8 [2*kv_heads, context, 272], written in place. keys/values [steps, kv_heads, 256]."""
    keys = np.ascontiguousarray(keys, np.float32)
    values = np.ascontiguousarray(values, np.float32)
    assert state.dtype == np.uint8 and state.flags.c_contiguous and state.size == 2 * kv_heads * context * ROW_Q8
    _lib.orc_kv_write(_ptr(state), context, kv_heads, base, keys.shape[0], _ptr(keys), _ptr(values))


def attention_sequence(state, context, heads, kv_heads, base, steps, selected, packed_input, scale=0.0625):
    packed_input = np.ascontiguousarray(packed_input, np.float32)
    assert packed_input.size == steps * (heads * DIM + 2 * kv_heads * DIM + selected + 1)
    out = np.empty((steps, heads, DIM), np.float32)
    _lib.orc_attention_sequence(_ptr(state), context, heads, kv_heads, base, steps, selected, _ptr(packed_input), scale, _ptr(out))
    return out


def gqa_decode_q8(state, context, length, heads, kv_heads, q_f16, scale, f64=False):
    """q_f16: [heads, 256] float16."""
    q = np.ascontiguousarray(q_f16, np.float16)
    out = np.empty((heads, DIM), np.float32)
    _lib.orc_gqa_decode_q8(_ptr(state), context, length, heads, kv_heads, _ptr(q), scale, int(f64), _ptr(out))
    return out


def gqa_prompt_q8(state, context, first, heads, kv_heads, q_f16, scale, rows=None, f64=False):
    """q_f16: [rows, heads, 256] float16; rows: iterable of row numbers to compute (default all). Others stay NaN."""
    q = np.ascontiguousarray(q_f16, np.float16)
    n = q.shape[0]
    out = np.full((n, heads, DIM), np.nan, np.float32)
    if rows is None:
        _lib.orc_gqa_prompt_q8(_ptr(state), context, first, n, 0, n, 1, heads, kv_heads, _ptr(q), scale, int(f64), _ptr(out))
    else:
        for r in rows:
            _lib.orc_gqa_prompt_q8(_ptr(state), context, first, n, r, r + 1, 1, heads, kv_heads, _ptr(q), scale, int(f64), _ptr(out))
    return out


def op_attention(q, keys, values, context, positions, rows, heads, kv_heads, dim, scale, gate=None, want64=False):
    q = np.ascontiguousarray(q, np.float32)
    keys = np.ascontiguousarray(keys, np.float32)
    values = np.ascontiguousarray(values, np.float32)
    positions = np.ascontiguousarray(positions, np.int32)
    gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
    out = np.empty((rows, heads, dim), np.float32)
    out64 = np.empty((rows, heads, dim), np.float64) if want64 else None
    bound = np.empty((rows, heads, dim), np.float64) if want64 else None
    _lib.orc_op_attention(_ptr(q), _ptr(keys), _ptr(values), context, _ptr(positions), rows, heads, kv_heads, dim, scale,
                          _ptr(gate), _ptr(out), _ptr(out64), _ptr(bound))
    return (out, out64, bound) if want64 else out


def sparse_attention(q, raw, raw_rows, positions, window, compressed, selected, selections, sinks, rows, heads, dim, scale,
                     rope_dims=0, frequencies=None, f64=False):
    """compressed: float32 [n, dim] or uint16 (BF16 bits) [n, dim]."""
    q = np.ascontiguousarray(q, np.float32)
    raw = np.ascontiguousarray(raw, np.float32)
    positions = np.ascontiguousarray(positions, np.int32)
    sinks = np.ascontiguousarray(sinks, np.float32)
    bf16 = compressed is not None and compressed.dtype == np.uint16
    if compressed is not None:
        compressed = np.ascontiguousarray(compressed)
    selected = None if selected is None else np.ascontiguousarray(selected, np.int32)
    frequencies = None if frequencies is None else np.ascontiguousarray(frequencies, np.float32)
    out = np.empty((rows, heads, dim), np.float32)
    _lib.orc_sparse_attention(_ptr(q), _ptr(raw), raw_rows, _ptr(positions), window, _ptr(compressed), int(bf16), _ptr(selected),
                              selections, _ptr(sinks), rows, heads, dim, scale, rope_dims, _ptr(frequencies), int(f64), _ptr(out))
    return out


def dspark_attention(q, ring, block, sinks, heads, slots, anchor, history, f64=False):
    """q [slots, heads, 512], ring [128, 512], block [>= slots, 512], sinks [>= heads] F32 -> out [slots, heads, 512]."""
    q, ring, block, sinks = (np.ascontiguousarray(x, np.float32) for x in (q, ring, block, sinks))
    out = np.empty((slots, heads, 512), np.float32)
    _lib.orc_dspark_attention(_ptr(q), _ptr(ring), _ptr(block), _ptr(sinks), heads, slots, anchor, history, int(f64), _ptr(out))
    return out


def rope(x, positions, frequencies, inverse=False):
    """x [rows, vectors, width] F32 (a rotated copy is returned), rope over the last 2 * len(frequencies) columns."""
    x = np.array(x, np.float32, order="C")
    rows, vectors, width = x.shape
    positions, frequencies = np.ascontiguousarray(positions, np.int32), np.ascontiguousarray(frequencies, np.float32)
    _lib.orc_rope(_ptr(x), rows, vectors, width, 2 * frequencies.size, _ptr(positions), _ptr(frequencies), int(inverse))
    return x


def compress(kv, gate, ratio):
    """kv, gate [groups * ratio, dim] F32 -> [groups, dim]."""
    kv = np.ascontiguousarray(kv, np.float32)
    gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
    groups, dim = kv.shape[0] // ratio, kv.shape[1]
    out = np.empty((groups, dim), np.float32)
    _lib.orc_compress(_ptr(kv), _ptr(gate), groups, ratio, dim, _ptr(out))
    return out


def index_scores(q, keys, weights, visible, scale, candidates=None, block=1):
    """q [rows, heads, dim] F32, keys [groups, dim] F32 or BF16 halves (uint16), weights [rows, heads], visible [rows] ->
    scores [rows, groups], or [rows, blocks * block] in candidate order with candidates [rows, blocks]."""
    q, weights, visible = np.ascontiguousarray(q, np.float32), np.ascontiguousarray(weights, np.float32), np.ascontiguousarray(visible, np.int32)
    bf16 = keys.dtype == np.uint16
    keys = np.ascontiguousarray(keys, np.uint16 if bf16 else np.float32)
    rows, heads, dim = q.shape
    groups = keys.shape[0]
    blocks = 0
    if candidates is not None:
        candidates = np.ascontiguousarray(candidates, np.int32)
        blocks = candidates.shape[1]
    out = np.empty((rows, blocks * block if blocks else groups), np.float32)
    _lib.orc_index_scores(_ptr(q), _ptr(keys), int(bf16), _ptr(weights), _ptr(visible), rows, groups, heads, dim, scale, _ptr(candidates), blocks, block, _ptr(out))
    return out


def index_candidates(scores, visible, blocks, block):
    """scores [rows, groups] -> candidates [rows, blocks]: the top blocks by their highest score, in index order, -1 past the last."""
    scores, visible = np.ascontiguousarray(scores, np.float32), np.ascontiguousarray(visible, np.int32)
    rows, groups = scores.shape
    tops = np.empty((rows, (groups + block - 1) // block), np.float32)
    _lib.orc_index_block_tops(_ptr(scores), _ptr(visible), rows, groups, block, _ptr(tops))
    return top_k(tops, blocks)


def index_select(q, keys, weights, visible, scale, positions, frequencies, k, candidates=None, block=1):
    """gpu/ops.hpp:1978-2300 by its contract (crates/straydog-engine/tests/fused_gpu.rs:391-431): rope, scores, top k -> (scores, indices);
    with candidates the indices are the groups' (gpu/ops.hpp:1967-1975)."""
    rotated = rope(q, positions, frequencies) if len(frequencies) else np.ascontiguousarray(q, np.float32)
    scores = index_scores(rotated, keys, weights, visible, scale, candidates, block)
    picked = top_k(scores, k)
    if candidates is not None:
        c = np.take_along_axis(np.asarray(candidates, np.int64), np.maximum(picked, 0) // block, axis=1)
        picked = np.where(picked < 0, -1, c * block + np.maximum(picked, 0) % block).astype(np.int32)
    return scores, picked


def qsa_index_select(queries, blocks, base, steps, selected, row_floats, packed, positions=None):
    """queries [steps, 512] F32, blocks [128, pool] F32; writes the lists and counts into `packed` (float32, in place) and returns it."""
    queries, blocks = np.ascontiguousarray(queries, np.float32), np.ascontiguousarray(blocks, np.float32)
    positions = None if positions is None else np.ascontiguousarray(positions, np.uint32)
    assert packed.dtype == np.float32 and packed.flags.c_contiguous and packed.size == steps * (row_floats + selected + 1)
    _lib.orc_qsa_index_select(_ptr(queries), queries.shape[1], _ptr(blocks), blocks.shape[1], base, _ptr(positions), steps, selected, row_floats, _ptr(packed))
    return packed


def qsa_normalize_rows(projections, heads, kv_heads, qnorm, knorm, iqnorm, pool_norm, positions, ropes, packed, state, context, index_state):
    """projections [rows, stride] F32 (the index queries are normalised in place); packed (float32), state (uint8 Q8_0 planes) and
    index_state ([128 * pool + 16 * 128] float32: pooled blocks, then the history ring) are written in place."""
    assert projections.dtype == np.float32 and projections.flags.c_contiguous and packed.dtype == np.float32 and packed.flags.c_contiguous
    assert state.dtype == np.uint8 and state.flags.c_contiguous and index_state.dtype == np.float32 and index_state.flags.c_contiguous
    assert index_state.size == (context // 4 + 1 + 16) * 128 and state.size == context * 2 * kv_heads * ROW_Q8
    rows, stride = projections.shape
    norms = [np.ascontiguousarray(n, np.float32) for n in (qnorm, knorm, iqnorm, pool_norm)]
    positions, ropes = np.ascontiguousarray(positions, np.uint32), np.ascontiguousarray(ropes, np.uint32)
    _lib.orc_qsa_normalize_rows(_ptr(projections), stride, rows, heads, kv_heads, *[_ptr(n) for n in norms], _ptr(positions), _ptr(ropes),
                                _ptr(packed), _ptr(state), context, _ptr(index_state))


def qsa_normalize_chunk(qgate, key, value, iq, ik, position, heads, kv_heads, qnorm, knorm, iqnorm, pool_norm, packed, state, context, index_state,
                        rope_rows=None, rope_first=0):
    """A prompt chunk's front: qgate [count, heads, 512], key / value [count, kv_heads, 256], iq [count, 4, 128] (normalised in place),
    ik [count, 128]; packed, state and index_state are written in place. rope_rows [n, 3] uint32 from position rope_first: the rope
    table of a sequence with images."""
    arrays = [qgate, key, value, iq, ik, packed, index_state]
    assert all(x.dtype == np.float32 and x.flags.c_contiguous for x in arrays) and state.dtype == np.uint8 and state.flags.c_contiguous
    count = ik.shape[0]
    assert qgate.size == count * heads * 512 and key.size == value.size == count * kv_heads * 256 and iq.size == count * 512
    assert index_state.size == (context // 4 + 1 + 16) * 128 and state.size == context * 2 * kv_heads * ROW_Q8
    norms = [np.ascontiguousarray(n, np.float32) for n in (qnorm, knorm, iqnorm, pool_norm)]
    table = np.ascontiguousarray(rope_rows, np.uint32) if rope_rows is not None else None
    _lib.orc_qsa_normalize_chunk(_ptr(qgate), _ptr(key), _ptr(value), _ptr(iq), _ptr(ik), count, position, heads, kv_heads, *[_ptr(n) for n in norms],
                                 _ptr(packed), _ptr(state), context, _ptr(index_state), _ptr(table) if table is not None else None, rope_first)


def index_proj(w, kind, x, units=True):
    """The head weights sd_op_index_select_proj projects: w [heads, cols] (kind 0: float32; 1 / 30: uint16 F16 / BF16 bits), x [cols] F32.
    units: the 16-byte unit path (aligned operands, a width of whole units), else the element path."""
    w, x = np.ascontiguousarray(w), np.ascontiguousarray(x, np.float32)
    assert w.dtype == (np.float32 if kind == 0 else np.uint16)
    out = np.empty(w.shape[0], np.float32)
    _lib.orc_index_proj(_ptr(w), kind, w.shape[0], w.shape[1], _ptr(x), int(units), _ptr(out))
    return out


def top_k(scores, k):
    scores = np.ascontiguousarray(scores, np.float32)
    rows, groups = scores.shape
    out = np.empty((rows, k), np.int32)
    _lib.orc_top_k(_ptr(scores), rows, groups, k, _ptr(out))
    return out


def to_bf16(x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    _lib.orc_to_bf16(_ptr(x), x.size, _ptr(out))
    return out


def bf16_to_f32(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)
