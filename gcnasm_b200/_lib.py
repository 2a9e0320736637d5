"""ctypes binding of ``libb200gemm.so`` (the C ABI in ``include/b200gemm.h``).

The library must have been built (``python -m gcnasm_b200.build``); there is no fallback of any
kind -- if the shared object is missing or fails to load, importing the operators raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# B200GEMM_LIB overrides the in-tree library path (e.g. an instrumented build)
LIB_PATH = os.environ.get("B200GEMM_LIB") or os.path.join(_PKG, "libb200gemm.so")

# enums (include/b200gemm.h)
SCALE_NONE, SCALE_TENSOR, SCALE_BLOCK, SCALE_MX = 0, 1, 2, 3
B_NK_ROWMAJOR, B_FLAT_16x16 = 0, 1
OUT_F32, OUT_BF16 = 0, 1
(TILE_AUTO, TILE_128x128, TILE_128x256, TILE_DECODE, TILE_PAIR_256x256, TILE_128x64, TILE_PAIR_256x128,
 TILE_PAIR_256x224, TILE_PAIR_256x192) = range(9)
GEMM_INPUTS_READY, GEMM_BATCH_READY = 1, 2
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_NO_DEVICE, ERR_TOO_LARGE = 0, -1, -2, -3, -4, -5, -6
ERR_IO, ERR_CORRUPT = -7, -8

# every symbol include/b200gemm.h declares
EXPORTS = (
    "b200_gemm_a8w8", "b200_gemm_check", "b200_gemm_a8w8_simple", "b200_gemm_a8w8_host", "b200_gemm_a8w8_decode_static",
    "b200_shuffle_b", "b200_unshuffle_b", "b200_gemm_a16w16", "b200_gemm_a16w16_check", "b200_shuffle_b_bf16",
    "b200_unshuffle_b_bf16",
    "b200_cast_e4m3", "b200_quantize_tensor", "b200_quantize_tensor_workspace", "b200_quantize_1x128",
    "b200_quantize_128x128", "b200_quantize_mx32", "b200_mx_sf_relayout", "b200_mx_sf_bytes",
    "b200_quantize_act_bf16_1x128", "b200_quantize_act_bf16_mx32", "b200_membw_read", "b200_membw_copy",
    "b200_weight_file_write", "b200_weight_file_stat", "b200_weight_file_read",
    "b200_fill_uniform", "b200_fill_normal",
    "b200_flag_write", "b200_flag_wait", "b200_stream_copy", "b200_ipc_alloc", "b200_ipc_open", "b200_ipc_close", "b200_ipc_free",
    "b200_slab_bytes", "b200_slab_upload", "b200_last_status", "b200_peek_status", "b200_selftest_bounded_wait", "b200_last_cuda_error", "b200_strerror", "b200_sm_count", "b200_release",
    "b200_version", "b200_launch_count", "b200_last_tail_split",
)


class GemmArgs(C.Structure):
    """``b200_gemm_args``: superset of the reference's ``opus_gemm_kargs`` / ``opus_fmm_kargs``."""

    _fields_ = [
        ("ptr_a", C.c_void_p), ("ptr_b", C.c_void_p), ("ptr_c", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("batch", C.c_int64),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_c", C.c_int64),
        ("stride_a_batch", C.c_int64), ("stride_b_batch", C.c_int64), ("stride_c_batch", C.c_int64),
        ("ptr_sfa", C.c_void_p), ("ptr_sfb", C.c_void_p),
        ("stride_sfa", C.c_int64), ("stride_sfb", C.c_int64),
        ("stride_sfa_batch", C.c_int64), ("stride_sfb_batch", C.c_int64),
        ("ptr_scale_a", C.c_void_p), ("ptr_scale_b", C.c_void_p),
        ("scale_mode", C.c_int32), ("b_layout", C.c_int32), ("out_dtype", C.c_int32), ("tile_hint", C.c_int32),
        ("flags", C.c_int32), ("batch_epoch", C.c_int32),
        ("ptr_batch_ready", C.c_void_p),
    ]


class B200Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().b200_strerror(code).decode()
        extra = ""
        if code == ERR_CUDA:
            extra = f" (cuda error {lib().b200_last_cuda_error()})"
        super().__init__(f"{where}: {msg}{extra} [{code}]")


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m gcnasm_b200.build` (needs nvcc). "
            "There is no CPU or library fallback for these operators.")
    L = C.CDLL(LIB_PATH)
    vp, i32, i64, sz, u64, u32, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_uint64, C.c_uint32, C.c_float
    P = C.POINTER(GemmArgs)
    sig = {
        "b200_gemm_a8w8": (i32, [P, vp]),
        "b200_gemm_check": (i32, [P, C.POINTER(i32)]),
        "b200_gemm_a8w8_simple": (i32, [P, vp]),
        "b200_gemm_a8w8_host": (i32, [P, vp]),
        "b200_gemm_a8w8_decode_static": (i32, [P, vp]),
        "b200_gemm_a16w16": (i32, [P, vp]),
        "b200_gemm_a16w16_check": (i32, [P, C.POINTER(C.c_int32)]),
        "b200_shuffle_b_bf16": (i32, [vp, vp, i64, i64, i32, vp]),
        "b200_unshuffle_b_bf16": (i32, [vp, vp, i64, i64, i32, vp]),
        "b200_shuffle_b": (i32, [vp, vp, i64, i64, i32, vp]),
        "b200_unshuffle_b": (i32, [vp, vp, i64, i64, i32, vp]),
        "b200_cast_e4m3": (i32, [vp, vp, i64, vp]),
        "b200_quantize_tensor": (i32, [vp, vp, vp, i64, vp, vp]),
        "b200_quantize_tensor_workspace": (sz, []),
        "b200_quantize_1x128": (i32, [vp, vp, vp, i64, i64, vp]),
        "b200_quantize_128x128": (i32, [vp, vp, vp, i64, i64, vp]),
        "b200_quantize_mx32": (i32, [vp, vp, vp, i64, i64, vp]),
        "b200_quantize_act_bf16_1x128": (i32, [vp, i64, vp, i64, vp, i64, i64, i64, vp]),
        "b200_quantize_act_bf16_mx32": (i32, [vp, i64, vp, i64, vp, i64, i64, vp]),
        "b200_weight_file_write": (i32, [C.c_char_p, i32, i32, i64, i64, vp, vp]),
        "b200_weight_file_stat": (i32, [C.c_char_p, vp]),
        "b200_weight_file_read": (i32, [C.c_char_p, vp, sz, vp, sz]),
        "b200_membw_read": (i32, [vp, sz, vp, vp]),
        "b200_membw_copy": (i32, [vp, vp, sz, vp]),
        "b200_mx_sf_relayout": (i32, [vp, vp, i64, i64, vp]),
        "b200_mx_sf_bytes": (sz, [i64, i64]),
        "b200_fill_uniform": (None, [vp, sz, u64, u32, f32, f32]),
        "b200_fill_normal": (None, [vp, sz, u64, u32]),
        "b200_flag_write": (i32, [vp, i32, vp]),
        "b200_flag_wait": (i32, [vp, i32, vp]),
        "b200_stream_copy": (i32, [vp, vp, sz, vp]),
        "b200_ipc_alloc": (i32, [sz, C.POINTER(vp), vp]),
        "b200_ipc_open": (i32, [vp, C.POINTER(vp)]),
        "b200_ipc_close": (i32, [vp]),
        "b200_ipc_free": (i32, [vp]),
        "b200_slab_bytes": (sz, [i64, i64]),
        "b200_slab_upload": (i32, [vp, vp, vp, i64, i64, i64, i64, vp]),
        "b200_last_status": (i32, []),
        "b200_peek_status": (i32, []),
        "b200_selftest_bounded_wait": (i32, [i64, i32, vp]),
        "b200_last_cuda_error": (i32, []),
        "b200_strerror": (C.c_char_p, [i32]),
        "b200_sm_count": (i32, []),
        "b200_release": (i32, []),
        "b200_version": (C.c_char_p, []),
        "b200_launch_count": (u64, []),
        "b200_last_tail_split": (i32, [vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def check(code: int, where: str) -> None:
    if code != 0:
        raise B200Error(code, where)
