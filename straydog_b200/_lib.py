"""Loads libstraydog_gpu_b200.so and declares its C ABI (include/straydog_gpu_b200.h) for ctypes.

There is no fallback: when the library is missing, the import fails with the command that builds it.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstraydog_gpu_b200.so")

u64, u32, i32, f32, p = C.c_uint64, C.c_uint32, C.c_int, C.c_float, C.c_void_p
pp = C.POINTER(C.c_void_p)
pu64 = C.POINTER(C.c_uint64)

# name -> (argument types, result type); mirrors include/straydog_gpu_b200.h declaration by declaration
SIGNATURES = {
    "sd_error": ([], C.c_char_p),
    "sd_device_count": ([], i32),
    "sd_create": ([i32, u64], p),
    "sd_destroy": ([p], None),
    "sd_memory": ([p, pu64, pu64], i32),
    "sd_upload": ([p, p, u64], p),
    "sd_allocate": ([p, u64], p),
    "sd_write": ([p, p, p, u64], i32),
    "sd_release": ([p, p], i32),
    "sd_allocation_bytes": ([p, p, pu64], i32),
    "sd_zero": ([p, p], i32),
    "sd_download": ([p, p, p, u64], i32),
    "sd_buffer": ([p, u64], p),
    "sd_buffer_write": ([p, p, u64, p, u64], i32),
    "sd_buffer_read": ([p, p, u64, p, u64], i32),
    "sd_kv_format": ([p, u32], i32),
    "sd_kv_stage": ([p, p, u64], i32),
    "sd_attention_sequence": ([p, p, u64, u64, u64, u64, p, u64, p, u64], i32),
    "sd_op_attention": ([p, p, p, p, u64, p, u64, u64, u64, u64, f32, p, p, u64, p], i32),
    "sd_attention_turns_reserve": ([p, u64, u64], i32),
    "sd_attention_turns_arm": ([p, u64], i32),
    "sd_op_sparse_attention": ([p, p, p, u64, p, u64, p, u64, p, u64, p, u64, u64, u64, f32, u64, p, p, u64, p], i32),
    "sdx_sparse_attention_gather": ([p, p, p, u64, p, u64, p, u64, p, u64, p, u64, u64, u64, f32, u64, p, u64, u64, p, p, i32], i32),
    "sdx_ipc_export": ([p, p, p], i32),
    "sdx_ipc_open": ([p, p, u64], p),
    "sdx_ipc_close": ([p, p], i32),
    "sdx_sparse_attention_spans": ([p, p, p, u64, p, u64, p, u64, p, u64, p, u64, u64, u64, u64, f32, u64, p, p], i32),
    "sd_op_dspark_attention": ([p, p, p, p, p, u64, u64, u32, p, u64, p], i32),
    "sd_host_state": ([p, u64], p),
    "sd_host_state_supported": ([p], i32),
    "sdx_qsa_attention_gathered": ([p, p, u64, u64, p, u64, u64, u64, u64, f32, p, p, u64, p, p], i32),
    "sdx_qsa_index_select": ([p, p, u64, p, u64, u64, p, u64, u64, u64, u64, p], i32),
    "sdx_kv_grow": ([p, u64, u64, u64, u64, p, p], i32),
    "sdx_qsa_normalize_rows": ([p, p, u64, u64, u64, u64, p, p, p, p, p, p, p, u64, p, u64, p, u64, p], i32),
    "sdx_qsa_normalize_chunk": ([p, p, p, p, p, p, u64, u64, u64, u64, p, p, p, p, p, u64, p, u64, p, u64, p], i32),
    "sd_rope_rows": ([p, u64, u64, p], i32),
    "sd_op_rope": ([p, p, u64, u64, u64, u64, p, p, i32], i32),
    "sd_op_compress": ([p, p, p, u64, u64, u64, p], i32),
    "sd_op_index_scores": ([p, p, p, p, p, u64, u64, u64, u64, f32, p], i32),
    "sd_op_index_candidates": ([p, p, p, u64, u64, u64, u64, p, p, u64], i32),
    "sd_op_index_select": ([p, p, p, p, p, u64, u64, u64, u64, f32, u64, p, p, p, u64, p, p, u64, u64], i32),
    "sd_op_index_select_proj": ([p, p, i32, u64, p, p, p, p, p, u64, u64, u64, f32, u64, p, p, p, u64, p, p, u64, u64], i32),
    "sd_op_top_k": ([p, p, u64, u64, u64, p], i32),
    "sd_op_to_bf16": ([p, p, u64, p], i32),
    "sdx_adopt": ([i32, p], p),
    "sdx_synchronize": ([p], i32),
    "sdx_stream": ([p], p),
    "sdx_launch_count": ([p], u64),
    "sdx_event_create": ([], p),
    "sdx_event_record": ([p, p], i32),
    "sdx_event_elapsed_ms": ([p, p, C.POINTER(C.c_float)], i32),
    "sdx_event_destroy": ([p], None),
    "sdx_kv_write": ([p, p, u64, u64, u64, u64, p, p], i32),
    "sdx_kv_decode_rows": ([p, p, u64, p], i32),
    "sdx_qsa_decode": ([p, pp, pu64, pu64, u64, u64, u64, f32, p, p], i32),
    "sdx_qsa_decode_static": ([p, pp, pu64, pu64, u64, u64, u64, f32, p, p], i32),
    "sdx_qsa_plan": ([p, pp, pu64, pu64, u64, u64, u64], p),
    "sdx_qsa_plan_run": ([p, p, f32, p, p], i32),
    "sdx_qsa_plan_run_marked": ([p, p, f32, p, p, p, p], i32),
    "sdx_qsa_plan_info": ([p, pu64, pu64, pu64, pu64], i32),
    "sdx_qsa_plan_release": ([p, p], i32),
    "sdx_decode_cuts": ([p, i32], i32),
    "sdx_qsa_cuts": ([pu64, u64, u64, u64, i32, u64, C.POINTER(C.c_uint32), u64, pu64], i32),
    "sdx_decode_status": ([p], i32),
    "sdx_trace_read": ([p, C.POINTER(C.c_int64), u64], i32),
    "sdx_qsa_prompt": ([p, p, u64, u64, u64, u64, u64, f32, p, p], i32),
    "sdx_qsa_attention_rows": ([p, p, u64, u64, p, u64, u64, u64, u64, f32, p, p, u64, p, u64, p], i32),
    "sdx_attention_batch": ([p, pp, pu64, pu64, u64, u64, u64, f32, p, p, p, p], i32),
}


def load(path: str = LIB_PATH, reference_abi_only: bool = False) -> C.CDLL:
    """reference_abi_only: declare the sd_* entries alone (another build of the reference ABI has no sdx_* additions)."""
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m straydog_b200.build` (needs nvcc; there is no CPU fallback)")
    lib = C.CDLL(path)
    for name, (args, res) in SIGNATURES.items():
        if reference_abi_only and name.startswith("sdx_"):
            continue
        f = getattr(lib, name)   # AttributeError if the library does not export what the header declares
        f.argtypes, f.restype = args, res
    return lib
