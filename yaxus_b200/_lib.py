"""ctypes bindings of libyaxus_cuda.so and libyaxus_host.so.

The CUDA library is the product; there is no fallback.  If it is missing, loading fails with
an error that says how to build it.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
# YAXUS_CUDA_LIB names another build of the same library (the diagnostic build with time stamps).
CUDA_LIB = os.environ.get("YAXUS_CUDA_LIB") or os.path.join(HERE, "libyaxus_cuda.so")
HOST_LIB = os.path.join(HERE, "libyaxus_host.so")

YX_OK, YX_ERR_INVALID, YX_ERR_CUDA, YX_ERR_OOM, YX_ERR_STATE, YX_ERR_DEVICE, YX_ERR_NCCL, YX_ERR_UNSUPPORTED = range(8)
F32, F16, BF16 = 0, 1, 2
PAGE = 128
HEAD_DIM = 128
STATIC_SPLITS, STATIC_MAX_ROW_HEADS = 8, 1024   # yx_attend_static's built-in scratch
PROBE_ITEM_WORDS = 41


class Rope(ctypes.Structure):
    _fields_ = [("inv_freq", c_float * (HEAD_DIM // 2)), ("concentration", c_float)]


class Layer(ctypes.Structure):
    _fields_ = [("window", c_int32), ("rope", Rope)]


class Tuning(ctypes.Structure):
    _fields_ = [("force_path", c_int32), ("ctas_per_sm", c_int32), ("share_prefix", c_int32),
                ("tile_min_rows", c_int32), ("cost32", c_int32), ("cost64", c_int32), ("stages", c_int32), ("share_rows", c_int32), ("item_cost", c_int32), ("fused_merge", c_int32), ("tile_single", c_int32), ("min_piece", c_int32), ("overlap_calls", c_int32)]


class PlanInfo(ctypes.Structure):
    _fields_ = [("path", c_int32), ("n_ctas", c_int32), ("n_items", c_int32), ("n_parts", c_int32),
                ("tiles", c_int64), ("unique_kv_bytes", c_int64), ("logical_kv_bytes", c_int64),
                ("launches", c_int32), ("shared_groups", c_int32)]


_U32P = POINTER(c_uint32)
_F32P = POINTER(c_float)

# name -> (restype, argtypes); exactly the functions include/yaxus_cuda.h declares.
SIGNATURES = {
    "yx_ctx_create": (c_int, [c_int, c_void_p, POINTER(c_void_p)]),
    "yx_ctx_destroy": (None, [c_void_p]),
    "yx_status": (c_int, [c_void_p]),
    "yx_last_error": (c_char_p, [c_void_p]),
    "yx_clear_error": (None, [c_void_p]),
    "yx_sync": (c_int, [c_void_p]),
    "yx_stream": (c_void_p, [c_void_p]),
    "yx_set_tuning": (c_int, [c_void_p, POINTER(Tuning)]),
    "yx_last_plan": (c_int, [c_void_p, POINTER(PlanInfo)]),
    "yx_launch_count": (c_int64, [c_void_p]),
    "yx_profile_begin": (c_int, [c_void_p]),
    "yx_profile_end": (c_int, [c_void_p, POINTER(c_float), POINTER(c_float), POINTER(c_int)]),
    "yx_tensor_alloc": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "yx_tensor_free": (c_int, [c_void_p, c_void_p]),
    "yx_upload": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "yx_download": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int]),
    "yx_host_alloc": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "yx_host_free": (c_int, [c_void_p, c_void_p]),
    "yx_kv_create": (c_int, [c_void_p, c_int, POINTER(Layer), c_uint32, c_int, c_int, c_int, c_uint32, POINTER(c_void_p)]),
    "yx_kv_destroy": (None, [c_void_p, c_void_p]),
    "yx_kv_copy_page": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32]),
    "yx_kv_read_pages": (c_int, [c_void_p, c_void_p, c_int, c_uint32, c_uint32, c_void_p, c_void_p]),
    "yx_kv_write_pages": (c_int, [c_void_p, c_void_p, c_int, c_uint32, c_uint32, c_void_p, c_void_p]),
    "yx_begin_pass": (c_int, [c_void_p, c_uint32, _U32P, _U32P, _U32P, _U32P, c_uint32]),
    "yx_attention": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "yx_kv_append": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int]),
    "yx_attend": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_void_p, c_int]),
    "yx_embed": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, _U32P, c_uint32, c_void_p]),
    "yx_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_float, c_float, c_void_p]),
    "yx_add_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_float, c_uint32, c_uint32, c_void_p]),
    "yx_matmul": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_void_p]),
    "yx_matmul_glu": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_void_p]),
    "yx_swiglu": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, c_void_p]),
    "yx_add_assign": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "yx_select_rows": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, _U32P, c_uint32, c_void_p]),
    "yx_argmax_rows": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, _U32P]),
    "yx_attend_static": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_void_p, c_int]),
    "yx_attend_partial": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_uint64, c_uint64,
                                  c_void_p, c_void_p, c_void_p]),
    "yx_lse_combine": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_int]),
    "yx_comm_unique_id": (c_int, [c_void_p]),
    "yx_comm_create": (c_int, [c_void_p, c_int, c_int, c_void_p]),
    "yx_comm_destroy": (c_int, [c_void_p]),
    "yx_attend_allgather": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_uint64, c_uint64,
                                    c_void_p, c_int]),
}

# The library's own test and measurement hooks (csrc/yx_hooks.h); not part of the C ABI.
HOOK_SIGNATURES = {
    "yx_plan_probe": (c_int, [c_uint32, _U32P, _U32P, _U32P, c_uint32, c_int, c_int, c_int64, c_uint64, c_uint64,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(PlanInfo), _U32P, c_uint32]),
    "yx_hook_plan_steps": (c_int, [c_uint32, _U32P, _U32P, _U32P, c_uint32, c_int, c_int, c_int64, c_int, c_int, c_int, POINTER(c_int)]),
    "yx_hook_forget_plan_shape": (c_int, [c_void_p]),
    "yx_hook_skip_merge": (c_int, [c_void_p, c_int]),
    "yx_hook_expire_wait": (c_int, [c_void_p, c_uint64]),
    "yx_hook_set_trace": (c_int, [c_void_p, c_void_p]),
    "yx_hook_host_times": (c_int, [c_void_p, POINTER(ctypes.c_double), c_int]),
}

HOST_SIGNATURES = {
    "yxh_last_error": (c_char_p, []),
    "yxh_kvcache_new": (c_void_p, [c_uint64, c_uint64]),
    "yxh_kvcache_free": (None, [c_void_p]),
    "yxh_set_prefix_reuse": (None, [c_void_p, c_int]),
    "yxh_new_seq": (c_int64, [c_void_p]),
    "yxh_free_seq": (None, [c_void_p, c_uint64]),
    "yxh_finish": (None, [c_void_p, c_uint64]),
    "yxh_seq_len": (c_int64, [c_void_p, c_uint64]),
    "yxh_free_pages": (c_int64, [c_void_p]),
    "yxh_total_pages": (c_int64, [c_void_p]),
    "yxh_page_refs": (c_int64, [c_void_p, c_uint32]),
    "yxh_seq_pages": (c_int64, [c_void_p, c_uint64, _U32P, c_uint64]),
    "yxh_seq_tokens": (c_int64, [c_void_p, c_uint64, _U32P, c_uint64]),
    "yxh_begin": (c_int64, [c_void_p, _U32P, c_uint64, POINTER(c_uint64)]),
    "yxh_fork": (c_int64, [c_void_p, c_uint64, c_uint64]),
    "yxh_truncate": (c_int64, [c_void_p, c_uint64, c_uint64]),
    "yxh_append": (c_int64, [c_void_p, c_uint64, POINTER(c_uint64), POINTER(c_uint64), _U32P]),
    "yxh_meta_pages": (c_int64, [c_void_p]),
    "yxh_meta_get": (None, [c_void_p, _U32P, _U32P, _U32P, _U32P, _U32P, _U32P]),
    "yxh_meta_items": (c_int64, [c_void_p]),
    "yxh_copies_pending": (c_int64, [c_void_p]),
    "yxh_copies_take": (c_int64, [c_void_p, _U32P, _U32P, c_uint64]),
}

_cuda = None
_host = None


def _bind(lib, sigs):
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    return lib


def cuda_lib():
    """The C-ABI library.  Raises if it has not been built: there is no other compute path."""
    global _cuda
    if _cuda is None:
        if not os.path.exists(CUDA_LIB):
            raise RuntimeError(
                f"{CUDA_LIB} is missing: build it with `python -m yaxus_b200.build` "
                "(needs nvcc; targets sm_100a). yaxus_b200 has no CPU or PyTorch fallback.")
        _cuda = _bind(_bind(ctypes.CDLL(CUDA_LIB), SIGNATURES), HOOK_SIGNATURES)
    return _cuda


def host_lib():
    global _host
    if _host is None:
        if not os.path.exists(HOST_LIB):
            raise RuntimeError(f"{HOST_LIB} is missing: build it with `python -m yaxus_b200.build`")
        _host = _bind(ctypes.CDLL(HOST_LIB), HOST_SIGNATURES)
    return _host
