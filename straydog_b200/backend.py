"""Host-side mirror of the reference engine's GPU wrapper for the attention path.

The reference's Rust `Backend` (crates/straydog-engine/src/gpu.rs) and `Ops` (src/ops.rs:878-886,
1158-1171, 1241-1244) wrap the sd_* C ABI; this module wraps the same entry points of
libstraydog_gpu_b200.so with the same method names and argument meaning, so that parity tests read
like the reference's own (tests/attention_gpu.rs, ds_state_bf16_gpu.rs, fused_gpu.rs). A failed call
raises StraydogError carrying sd_error()'s text, as the Rust wrappers return Err(last_error()).
"""
import ctypes as C

import numpy as np

from . import _lib

_L = None


def lib():
    global _L
    if _L is None:
        _L = _lib.load()
    return _L


class StraydogError(RuntimeError):
    pass


def _fail(library=None):
    raise StraydogError((library or lib()).sd_error().decode("utf-8", "replace"))


def _check(result, library=None):
    if result is None or (isinstance(result, int) and result < 0):
        _fail(library)
    return result


def _host(a):
    return a.ctypes.data_as(C.c_void_p)


class Buffer:
    """A device allocation of the backend (zeroed at creation). base() is its device address."""

    def __init__(self, backend, pointer, size):
        self.backend, self.pointer, self.size = backend, pointer, size

    def base(self):
        return self.pointer

    def at(self, byte_offset):
        return self.pointer + byte_offset

    def tagged_bf16(self):
        """The pointer with the reference's BF16 tag in bit 0 (gpu/ops.hpp:1208-1210)."""
        return self.pointer | 1


class Backend:
    def __init__(self, ordinal=0, budget=1 << 30, library=None):
        """library: a ctypes handle of another build of the same sd_* ABI (tests/golden drives the
        reference's own library through this wrapper); default: libstraydog_gpu_b200.so."""
        self.lib = library or lib()
        self.handle = self.lib.sd_create(ordinal, budget)
        if not self.handle:
            _fail(self.lib)
        self.ordinal = ordinal

    def _c(self, result):
        return _check(result, self.lib)

    def close(self):
        if self.handle:
            self.lib.sd_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- memory ----
    def buffer(self, size):
        pointer = self.lib.sd_buffer(self.handle, size)
        if not pointer:
            _fail(self.lib)
        return Buffer(self, pointer, size)

    def upload(self, array):
        array = np.ascontiguousarray(array)
        buffer = self.buffer(max(array.nbytes, 4))
        self.write_buffer(buffer, 0, array)
        return buffer

    def allocate(self, size):
        pointer = self.lib.sd_allocate(self.handle, size)
        if not pointer:
            _fail(self.lib)
        return Buffer(self, pointer, size)

    def write_buffer(self, buffer, offset, array):
        array = np.ascontiguousarray(array)
        self._c(self.lib.sd_buffer_write(self.handle, buffer.pointer, offset, _host(array), array.nbytes))

    def read_buffer(self, buffer, offset, out):
        assert out.flags.c_contiguous
        self._c(self.lib.sd_buffer_read(self.handle, buffer.pointer, offset, _host(out), out.nbytes))
        return out

    def read(self, buffer, dtype, shape, offset=0):
        return self.read_buffer(buffer, offset, np.empty(shape, dtype))

    def write(self, buffer, array):
        array = np.ascontiguousarray(array)
        self._c(self.lib.sd_write(self.handle, buffer.pointer, _host(array), array.nbytes))

    def download(self, buffer, out):
        self._c(self.lib.sd_download(self.handle, buffer.pointer, _host(out), out.nbytes))
        return out

    def zero(self, buffer):
        self._c(self.lib.sd_zero(self.handle, buffer.pointer))

    def release(self, buffer):
        self._c(self.lib.sd_release(self.handle, buffer.pointer))
        buffer.pointer = None

    def memory(self):
        used, budget = C.c_uint64(), C.c_uint64()
        self._c(self.lib.sd_memory(self.handle, C.byref(used), C.byref(budget)))
        return used.value, budget.value

    def synchronize(self):
        self._c(self.lib.sdx_synchronize(self.handle))

    def stream(self):
        return self.lib.sdx_stream(self.handle)

    def event(self):
        e = self.lib.sdx_event_create()
        if not e:
            _fail(self.lib)
        return e

    def record(self, event):
        self._c(self.lib.sdx_event_record(self.handle, event))

    @staticmethod
    def elapsed_ms(before, after):
        ms = C.c_float()
        _check(lib().sdx_event_elapsed_ms(before, after, C.byref(ms)))
        return ms.value

    def launch_count(self):
        return int(self.lib.sdx_launch_count(self.handle))

    # ---- K/V ----
    def kv_format(self, row):
        self._c(self.lib.sd_kv_format(self.handle, row))

    def kv_stage(self, buffer, rows):
        self._c(self.lib.sd_kv_stage(self.handle, buffer.pointer, rows))

    def kv_write(self, state, context, kv_heads, base, steps, keys, values):
        self._c(self.lib.sdx_kv_write(self.handle, state.pointer, context, kv_heads, base, steps, keys.pointer, values.pointer))

    def kv_decode_rows(self, rows_pointer, count, out):
        self._c(self.lib.sdx_kv_decode_rows(self.handle, rows_pointer, count, out.pointer))

    # ---- Qwen-style attention ----
    def attention_sequence(self, state, context, base, steps, selected, packed_input):
        """sd_attention_sequence: host floats in, host floats out ([steps, 24, 256])."""
        packed_input = np.ascontiguousarray(packed_input, np.float32)
        out = np.empty(steps * 24 * 256, np.float32)
        self._c(self.lib.sd_attention_sequence(self.handle, state.pointer, context, base, steps, selected, _host(packed_input),
                                           packed_input.size, _host(out), out.size))
        return out.reshape(steps, 24, 256)

    def attention(self, q, keys, values, context, positions, rows, heads, kv_heads, dim, scale, gate, scratch, out):
        """sd_op_attention over device pointers (ints); gate and scratch may be None."""
        self._c(self.lib.sd_op_attention(self.handle, q, keys, values, context, positions, rows, heads, kv_heads, dim, scale, gate,
                                     scratch.pointer if scratch else None, scratch.size if scratch else 0, out))

    def qsa_decode(self, states, contexts, lengths, heads, kv_heads, scale, q, out):
        n = len(states)
        ptrs = (C.c_void_p * n)(*[s.pointer if isinstance(s, Buffer) else s for s in states])
        ctx = (C.c_uint64 * n)(*contexts)
        lens = (C.c_uint64 * n)(*lengths)
        self._c(self.lib.sdx_qsa_decode(self.handle, ptrs, ctx, lens, n, heads, kv_heads, scale, q, out))

    def qsa_decode_static(self, states, contexts, lengths, heads, kv_heads, scale, q, out):
        """sdx_qsa_decode_static: the same decode with its scratch inside the library's device image (no allocation)."""
        n = len(states)
        ptrs = (C.c_void_p * n)(*[s.pointer if isinstance(s, Buffer) else s for s in states])
        ctx = (C.c_uint64 * n)(*contexts)
        lens = (C.c_uint64 * n)(*lengths)
        self._c(self.lib.sdx_qsa_decode_static(self.handle, ptrs, ctx, lens, n, heads, kv_heads, scale, q, out))

    def decode_cuts(self, fixed):
        """sdx_decode_cuts: fixed cuts (a sequence's bits do not depend on its batch) or the default moving cuts."""
        self._c(self.lib.sdx_decode_cuts(self.handle, int(bool(fixed))))

    def qsa_plan(self, states, contexts, lengths, heads, kv_heads):
        n = len(states)
        ptrs = (C.c_void_p * n)(*[s.pointer if isinstance(s, Buffer) else s for s in states])
        ctx = (C.c_uint64 * n)(*contexts)
        lens = (C.c_uint64 * n)(*lengths)
        plan = self.lib.sdx_qsa_plan(self.handle, ptrs, ctx, lens, n, heads, kv_heads)
        if not plan:
            _fail(self.lib)
        return plan

    def qsa_plan_run(self, plan, scale, q, out):
        self._c(self.lib.sdx_qsa_plan_run(self.handle, plan, scale, q, out))

    def qsa_plan_run_marked(self, plan, scale, q, out, before, after):
        self._c(self.lib.sdx_qsa_plan_run_marked(self.handle, plan, scale, q, out, before, after))

    def qsa_plan_info(self, plan):
        vals = [C.c_uint64() for _ in range(4)]
        self._c(self.lib.sdx_qsa_plan_info(plan, *[C.byref(v) for v in vals]))
        return dict(zip(("kv_bytes", "pieces", "ctas", "virtual_warps"), [v.value for v in vals]))

    def qsa_plan_release(self, plan):
        self._c(self.lib.sdx_qsa_plan_release(self.handle, plan))

    def qsa_prompt(self, state, context, first, rows, heads, kv_heads, scale, q, out):
        self._c(self.lib.sdx_qsa_prompt(self.handle, state.pointer if isinstance(state, Buffer) else state, context, first, rows, heads,
                                        kv_heads, scale, q, out))

    def qsa_attention_rows(self, state, context, base, positions, steps, selected, heads, kv_heads, scale, packed, out, mirror=None,
                           gates=None):
        """sdx_qsa_attention_rows: the reference's qsa_attention / qsa_attention_rows over device pointers. positions: device pointer
        or None; mirror: (pointer, rows) or None; gates: (pointer, row stride in floats) or None."""
        m_ptr, m_rows = mirror if mirror else (None, 0)
        g_ptr, g_stride = gates if gates else (None, 0)
        self._c(self.lib.sdx_qsa_attention_rows(self.handle, state.pointer if isinstance(state, Buffer) else state, context, base, positions,
                                                steps, selected, heads, kv_heads, scale, packed, m_ptr, m_rows, g_ptr, g_stride, out))

    def host_state(self, size):
        """sd_host_state: a zeroed state in page-locked host memory the GPU reads in place (outside the VRAM budget)."""
        pointer = self.lib.sd_host_state(self.handle, size)
        if not pointer:
            _fail(self.lib)
        return Buffer(self, pointer, size)

    def qsa_attention_gathered(self, state, context, base, positions, steps, selected, heads, kv_heads, scale, packed, out, gates=None):
        """sdx_qsa_attention_gathered: sdx_qsa_attention_rows over a host-resident state through the registered K/V stage; returns the
        number of row groups the call made."""
        g_ptr, g_stride = gates if gates else (None, 0)
        passes = C.c_uint64(0)
        self._c(self.lib.sdx_qsa_attention_gathered(self.handle, state.pointer if isinstance(state, Buffer) else state, context, base, positions,
                                                    steps, selected, heads, kv_heads, scale, packed, g_ptr, g_stride, out, C.byref(passes)))
        return passes.value

    def qsa_index_select(self, queries, query_stride, blocks, pool, base, positions, steps, selected, heads, kv_heads, packed):
        """sdx_qsa_index_select: Qwen's block scores and exact top-512 block choice, written into the packed rows (device pointers)."""
        self._c(self.lib.sdx_qsa_index_select(self.handle, queries, query_stride, blocks, pool, base, positions, steps, selected, heads, kv_heads, packed))

    def qsa_normalize_rows(self, projections, stride, rows, heads, kv_heads, qnorm, knorm, iqnorm, pool_norm, positions, ropes, packed,
                           selected, state, context, index_state, mirror=None, mirror_rows=0):
        """sdx_qsa_normalize_rows: normalisation and rotation of the rows' queries, keys and index queries, their K/V rows written,
        their index keys pooled (device pointers)."""
        state = state.pointer if isinstance(state, Buffer) else state
        self._c(self.lib.sdx_qsa_normalize_rows(self.handle, projections, stride, rows, heads, kv_heads, qnorm, knorm, iqnorm, pool_norm,
                                                positions, ropes, packed, selected, state, context, mirror, mirror_rows, index_state))

    def qsa_normalize_chunk(self, qgate, key, value, iq, ik, count, position, heads, kv_heads, qnorm, knorm, iqnorm, pool_norm, packed, selected,
                            state, context, index_state, mirror=None, mirror_rows=0):
        """sdx_qsa_normalize_chunk: the same front for a prompt chunk of `count` tokens from `position` (device pointers)."""
        state = state.pointer if isinstance(state, Buffer) else state
        self._c(self.lib.sdx_qsa_normalize_chunk(self.handle, qgate, key, value, iq, ik, count, position, heads, kv_heads, qnorm, knorm, iqnorm,
                                                 pool_norm, packed, selected, state, context, mirror, mirror_rows, index_state))

    def rope_rows(self, first, axes):
        """sd_rope_rows: the rope table of a sequence with images, axes [count, 3] uint32 from position `first`; None or empty clears it."""
        if axes is None or len(axes) == 0:
            self._c(self.lib.sd_rope_rows(self.handle, 0, 0, None))
            return
        axes = np.ascontiguousarray(axes, np.uint32)
        assert axes.ndim == 2 and axes.shape[1] == 3
        self._c(self.lib.sd_rope_rows(self.handle, first, axes.shape[0], axes.ctypes.data_as(C.c_void_p)))

    def kv_grow(self, kv_heads, from_context, to_context, valid, state, index_state, row=272):
        """sdx_kv_grow: the state and the index state (Buffers) grown to `to_context` positions; returns the two new Buffers. The library
        has released the old state (and the old index state unless it was large enough: then the same Buffer comes back)."""
        s, i = C.c_void_p(state.pointer), C.c_void_p(index_state.pointer)
        self._c(self.lib.sdx_kv_grow(self.handle, kv_heads, from_context, to_context, valid, C.byref(s), C.byref(i)))
        grown = Buffer(self, s.value, to_context * 2 * kv_heads * row)
        index = index_state
        if i.value != index_state.pointer:
            index, index_state.pointer = Buffer(self, i.value, ((to_context // 4 + 1) * 128 + 2048) * 4), None
        state.pointer = None
        return grown, index

    def decode_status(self):
        return self._c(self.lib.sdx_decode_status(self.handle))

    def attention_batch(self, states, contexts, bases, heads, kv_heads, scale, q_host, k_host, v_host, out_host):
        n = len(states)
        ptrs = (C.c_void_p * n)(*[s.pointer if isinstance(s, Buffer) else s for s in states])
        ctx = (C.c_uint64 * n)(*contexts)
        bs = (C.c_uint64 * n)(*bases)
        self._c(self.lib.sdx_attention_batch(self.handle, ptrs, ctx, bs, n, heads, kv_heads, scale, _host(q_host), _host(k_host),
                                         _host(v_host), _host(out_host)))
        return out_host

    # ---- DeepSeek-style latent attention ----
    def attention_turns_reserve(self, rows, rope_dims):
        self._c(self.lib.sd_attention_turns_reserve(self.handle, rows, rope_dims))

    def attention_turns_arm(self, rows):
        self._c(self.lib.sd_attention_turns_arm(self.handle, rows))

    def sparse_attention(self, q, raw, raw_rows, positions, window, compressed, selected, sinks, rows, heads, dim, scale, rope,
                         scratch, out):
        """compressed: (pointer, rows) or None; selected: (pointer, selections) or None; rope: (rope_dims, frequencies pointer) or None."""
        c_ptr, c_rows = compressed if compressed else (None, 0)
        s_ptr, selections = selected if selected else (None, 0)
        rope_dims, freq = rope if rope else (0, None)
        self._c(self.lib.sd_op_sparse_attention(self.handle, q, raw, raw_rows, positions, window, c_ptr, c_rows, s_ptr, selections, sinks,
                                            rows, heads, dim, scale, rope_dims, freq, scratch.pointer if scratch else None,
                                            scratch.size if scratch else 0, out))

    def sparse_attention_spans(self, q, raw, raw_rows, positions, window, compressed, selected, sinks, spans, span_rows, heads, dim, scale,
                               rope, out):
        """`spans` calls of sparse_attention with rows = span_rows in one launch (an addition; every span its own window ring)."""
        c_ptr, c_rows = compressed if compressed else (None, 0)
        s_ptr, selections = selected if selected else (None, 0)
        rope_dims, freq = rope if rope else (0, None)
        self._c(self.lib.sdx_sparse_attention_spans(self.handle, q, raw, raw_rows, positions, window, c_ptr, c_rows, s_ptr, selections, sinks,
                                                spans, span_rows, heads, dim, scale, rope_dims, freq, out))

    def ipc_export(self, buffer):
        """64 bytes another rank's process hands to ipc_open to map `buffer` (an allocation of this handle)."""
        token = C.create_string_buffer(64)
        self._c(self.lib.sdx_ipc_export(self.handle, buffer.pointer, token))
        return token.raw

    def ipc_open(self, token, size):
        pointer = self.lib.sdx_ipc_open(self.handle, token, size)
        if not pointer:
            _fail(self.lib)
        return pointer

    def ipc_close(self, pointer):
        self._c(self.lib.sdx_ipc_close(self.handle, pointer))

    def sparse_attention_gather(self, q, raw, raw_rows, positions, window, compressed, selected, sinks, rows, heads, dim, scale, rope,
                                rank, outs, flags, step):
        """sparse_attention of this rank's heads with its outputs stored into slot `rank` of every rank's gathered buffer
        (outs, flags: one device pointer per rank, the others' mapped by ipc_open)."""
        c_ptr, c_rows = compressed if compressed else (None, 0)
        s_ptr, selections = selected if selected else (None, 0)
        rope_dims, freq = rope if rope else (0, None)
        world = len(outs)
        out_table, flag_table = (C.c_void_p * world)(*outs), (C.c_void_p * world)(*flags)
        self._c(self.lib.sdx_sparse_attention_gather(self.handle, q, raw, raw_rows, positions, window, c_ptr, c_rows, s_ptr, selections, sinks,
                                                 rows, heads, dim, scale, rope_dims, freq, world, rank, out_table, flag_table, step))

    def dspark_attention(self, q, ring, block, sinks, heads, slots, anchor, anchor_at, history, out):
        """sd_op_dspark_attention over device pointers (crates/straydog-engine/src/ops.rs:232-237); anchor_at: device pointer or None."""
        self._c(self.lib.sd_op_dspark_attention(self.handle, q, ring.pointer if isinstance(ring, Buffer) else ring, block,
                                                sinks.pointer if isinstance(sinks, Buffer) else sinks, heads, slots, anchor, anchor_at, history, out))

    # ---- the indexer (crates/straydog-engine/src/ops.rs:1173-1222); device pointers (ints) throughout ----
    def rope(self, x, rows, vectors, width, rope_dims, positions, frequencies, inverse=False):
        self._c(self.lib.sd_op_rope(self.handle, x, rows, vectors, width, rope_dims, positions, frequencies, int(inverse)))

    def compress(self, kv, gate, groups, ratio, dim, out):
        self._c(self.lib.sd_op_compress(self.handle, kv, gate, groups, ratio, dim, out))

    def index_scores(self, q, keys, weights, visible, rows, groups, heads, dim, scale, scores):
        self._c(self.lib.sd_op_index_scores(self.handle, q, keys, weights, visible, rows, groups, heads, dim, scale, scores))

    def index_candidates(self, scores, visible, rows, groups, blocks, block, out, scratch):
        self._c(self.lib.sd_op_index_candidates(self.handle, scores, visible, rows, groups, blocks, block, out, scratch.pointer, scratch.size))

    def index_select(self, q, keys, weights, visible, rows, groups, heads, dim, scale, rope, scores, k, out, candidates=None):
        """rope: (rope_dims, positions pointer, frequencies pointer); candidates: (pointer, blocks, block) or None."""
        rope_dims, positions, frequencies = rope
        c_ptr, blocks, block = candidates if candidates else (None, 0, 0)
        self._c(self.lib.sd_op_index_select(self.handle, q, keys, weights, visible, rows, groups, heads, dim, scale, rope_dims, positions,
                                            frequencies, scores, k, out, c_ptr, blocks, block))

    def index_select_proj(self, proj_weights, proj_kind, proj_cols, x, q, keys, weights, visible, groups, heads, dim, scale, rope, scores, k, out,
                          candidates=None):
        """sd_op_index_select_proj: one row; weights = W . x first (W of kind 0 F32, 1 F16, 30 BF16). rope and candidates as index_select."""
        rope_dims, positions, frequencies = rope
        c_ptr, blocks, block = candidates if candidates else (None, 0, 0)
        self._c(self.lib.sd_op_index_select_proj(self.handle, proj_weights, proj_kind, proj_cols, x, q, keys, weights, visible, groups, heads, dim,
                                                 scale, rope_dims, positions, frequencies, scores, k, out, c_ptr, blocks, block))

    def top_k(self, scores, rows, groups, k, out):
        self._c(self.lib.sd_op_top_k(self.handle, scores, rows, groups, k, out))

    def to_bf16(self, x, count, out):
        self._c(self.lib.sd_op_to_bf16(self.handle, x, count, out))


def device_count():
    return _check(lib().sd_device_count())
