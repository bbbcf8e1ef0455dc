"""ctypes binding of libvn_b200.so (the C ABI declared in include/vn_b200.h).

The library is the only compute path of this package: if it cannot be
loaded, or no CUDA device answers, the error is raised to the caller --
there is no CPU fallback.  (The reference's own native module follows the
opposite convention, "import fails -> silently fall back":
verse_torch/tensor.py:31-34.)
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvn_b200.so")

VN_OK, VN_ERR_INVALID, VN_ERR_OOM, VN_ERR_OVERFLOW, VN_ERR_TIMEOUT, VN_ERR_CUDA, VN_ERR_NCCL, \
    VN_ERR_INDEX, VN_ERR_UNSUPPORTED = range(9)


class VnError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[vn_b200 status {code}] {msg}")
        self.code = code


# status code -> exception type of the reference API for the same failure
_EXC = {
    VN_ERR_INVALID: ValueError,        # speculative.py:188-196 rank / batch mismatch
    VN_ERR_OOM: MemoryError,
    VN_ERR_OVERFLOW: RuntimeError,     # kv_cache_parallel.py:152-159
    VN_ERR_TIMEOUT: RuntimeError,      # a bounded wait inside a kernel ran out
    VN_ERR_INDEX: IndexError,          # kv_cache_parallel.py:136-139
    VN_ERR_UNSUPPORTED: NotImplementedError,
}

_p = C.c_void_p
_i32, _i64, _u32, _u64, _f32, _sz = C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float, C.c_size_t

# name -> argtypes; every function returns int32 unless listed in _RESTYPE
PROTOTYPES = {
    "vn_version": [],
    "vn_ctx_create": [_i32, C.POINTER(_p)],
    "vn_ctx_destroy": [_p],
    "vn_last_error": [_p],
    "vn_sync": [_p],
    "vn_launch_count": [_p, C.POINTER(_u64)],
    "vn_stream": [_p, C.POINTER(_p)],
    "vn_alloc": [_p, _sz, C.POINTER(_p)],
    "vn_free": [_p, _p],
    "vn_memset": [_p, _p, _i32, _sz],
    "vn_h2d": [_p, _p, _p, _sz],
    "vn_d2h": [_p, _p, _p, _sz],
    "vn_d2d": [_p, _p, _p, _sz],
    "vn_copy_2d": [_p, _p, _sz, _p, _sz, _sz, _sz],
    "vn_host_alloc": [_p, _sz, C.POINTER(_p)],
    "vn_host_free": [_p, _p],
    "vn_h2d_async": [_p, _p, _p, _sz],
    "vn_d2h_async": [_p, _p, _p, _sz],
    "vn_mem_info": [_p, C.POINTER(_sz), C.POINTER(_sz)],
    "vn_event_create": [_p, C.POINTER(_p)],
    "vn_event_destroy": [_p, _p],
    "vn_event_record": [_p, _p],
    "vn_event_elapsed_ms": [_p, _p, _p, C.POINTER(_f32)],
    "vn_flush_l2": [_p],
    "vn_profile": [_p, _i32],
    "vn_profile_report": [_p, C.c_char_p, _sz],
    "vn_matmul": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32],
    "vn_linear": [_p, _p, _p, _p, _p, _i64, _i64, _i64],
    "vn_softmax": [_p, _p, _p, _i64, _i64, _i64],
    "vn_layernorm": [_p, _p, _p, _p, _p, _i64, _i64, _f32],
    "vn_rmsnorm": [_p, _p, _p, _p, _i64, _i64, _f32],
    "vn_rope": [_p, _p, _p, _p, _p, _i64, _i64, _i64],
    "vn_attention": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64],
    "vn_accept": [_p, _p, _p, _p, _p, _p, _u64, _u32, _f32, _i32, _i32, _i32, _i32, _i32, _p, _p],
    "vn_accept_strided": [_p, _p, _i64, _i64, _p, _i64, _i64, _p, _p, _p, _u64, _u32, _f32, _i32, _i32,
                          _i32, _i32, _i32, _p, _p],
    "vn_accept_noalloc": [_p, _p, _p, _p, _p, _p, _u64, _u32, _f32, _i32, _i32, _i32, _i32, _p, _p],
    "vn_philox_uniform": [_p, _u64, _u32, _i32, _i32, _i32, _p],
    "vn_sample": [_p, _p, _i64, _i32, _i32, _f32, _i32, _p, _u64, _u32, _u32, _u32, _p],
    "vn_top_m": [_p, _p, _i64, _i32, _i32, _i32, _p, _i64],
    "vn_tree_accept_greedy": [_p, _p, _p, _p, _i32, _i32, _i32, _p, _p, _p, _p],
    "vn_tree_accept_sample": [_p, _p, _p, _p, _i32, _i32, _i32, _p, _p, _u64, _u32, _p, _p, _p, _p],
    "vn_draft_propose": [_p, _p, _p, _i32, _i32, _f32, _i32, _u64, _u32, _p, _p, _p],
    "vn_sample_lists": [_p, _p, _i64, _i32, _i32, _f32, _i32, _p, _u64, _u32, _u32, _u32, _p, _p],
    "vn_topk_row_bytes": [],
    "vn_verify_accept": [_p, _p, _p, _i32, _i32, _i32, _p, _i64, _i64, _p, _i64, _i64, _p, _p, _p, _u64, _u32, _f32,
                         _i32, _i32, _p, _p, _p],
    "vn_comm_unique_id": [_p],
    "vn_comm_create": [_p, _p, _i32, _i32, C.POINTER(_p)],
    "vn_comm_destroy": [_p],
    "vn_comm_info": [_p, C.POINTER(_i32), C.POINTER(_i32)],
    "vn_all_gather": [_p, _p, _p, _sz],
    "vn_shard_accept": [_p, _p, _p, _p, _p, _i32, _i32, _f32, _u64, _u64, _u32, _i32, _i32, _i32, _i32, _p, _p],
    "vn_spec_gather": [_p, _p, _p, _i32, _i32, _i32, _p, _p],
    "vn_spec_advance": [_p, _p, _i32, _i32, _p, _p, _i32, _p, _p],
    "vn_set_offset_source": [_p, _p],
    "vn_graph_begin": [_p],
    "vn_graph_end": [_p, C.POINTER(_p)],
    "vn_graph_launch": [_p, _p],
    "vn_graph_destroy": [_p, _p],
    "vn_model_create": [_p, C.c_char_p, C.POINTER(_p)],
    "vn_model_destroy": [_p],
    "vn_model_load_tensor": [_p, C.c_char_p, _p, _i32, C.POINTER(_i64)],
    "vn_model_finalize": [_p],
    "vn_model_quantize": [_p, C.c_char_p],
    "vn_quantize": [_p, _p, _i64, _i32, C.c_char_p, _p, _p],
    "vn_model_load_quant_tensor": [_p, C.c_char_p, C.c_char_p, _p, _p, _i64, _i64],
    "vn_model_read_quant": [_p, C.c_char_p, _p, _sz, _p, _sz],
    "vn_row_stats": [_p, _p, _i64, _i32, _i32, _f32, _p, _p, _p, _p],
    "vn_row_residual": [_p, _p, _i64, _p, _i64, _i32, _i32, _f32, _p, _p, _p, _p, _p, _p, _p],
    "vn_row_pick": [_p, _p, _i64, _p, _i64, _i32, _i32, _f32, _p, _p, _p, _p, _p, _p, _p, _p],
    "vn_model_param_bytes": [_p, C.POINTER(_u64)],
    "vn_model_head": [_p, _p, _i32, _i32, _i32, _p, _i64],
    "vn_model_set_recurrent": [_p, _i32],
    "vn_model_set_fused_stack": [_p, _i32],
    "vn_model_set_wait_limit": [_p, _u64],
    "vn_model_probe_wait": [_p, C.POINTER(_i64)],
    "vn_model_status": [_p, C.POINTER(_i32), C.POINTER(_i32)],
    "vn_kv_create": [_p, _i32, _i32, C.POINTER(_p)],
    "vn_kv_destroy": [_p],
    "vn_kv_view": [_p, _i32, _i32, C.POINTER(_p)],
    "vn_kv_reset_seq": [_p, _i32],
    "vn_kv_lengths": [_p, _p],
    "vn_kv_set_lengths": [_p, _p],
    "vn_kv_commit": [_p, _i32, _p, _i32, _p, _i32],
    "vn_kv_read": [_p, _i32, _i32, _i32, _p, _i32],
    "vn_model_forward": [_p, _p, _p, _i32, _i32, _p, _p, _p, _i32, _i32],
}
_RESTYPE = {"vn_last_error": C.c_char_p, "vn_topk_row_bytes": C.c_size_t}

_lib = None


def load():
    """Load the shared library once; raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m versenext_b200.csrc.build` "
            "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = argtypes
        fn.restype = _RESTYPE.get(name, _i32)
    _lib = lib
    return lib


def check(ctx_handle, status):
    if status == VN_OK:
        return
    msg = load().vn_last_error(ctx_handle)
    msg = msg.decode("utf-8", "replace") if msg else ""
    exc = _EXC.get(status)
    if exc is None:
        raise VnError(status, msg)
    raise exc(f"[vn_b200 status {status}] {msg}")
