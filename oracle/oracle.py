"""ctypes/numpy front-end of the CPU oracle (``liboracle.so``).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark import this
module; the product package never does.  Every function maps 1:1 onto a C function in
``oracle.c``, which carries the reference citations.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with gcc (a few seconds)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        vp, i32, i64, f32, u64, u32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint64, C.c_uint32, C.c_size_t
        L.orc_e4m3_to_f32.restype = f32
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e4m3.restype = C.c_uint8
        L.orc_f32_to_e4m3.argtypes = [f32]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [f32]
        L.orc_e8m0_to_f32.restype = f32
        L.orc_e8m0_to_f32.argtypes = [C.c_uint8]
        L.orc_fill_uniform.argtypes = [vp, sz, u64, u32, f32, f32]
        L.orc_fill_normal.argtypes = [vp, sz, u64, u32]
        L.orc_cast_e4m3.argtypes = [vp, sz, vp]
        L.orc_quant_tensor.argtypes = [vp, sz, vp, vp]
        L.orc_quant_1x128.argtypes = [vp, i32, i32, vp, vp]
        L.orc_quant_128x128.argtypes = [vp, i32, i32, vp, vp]
        L.orc_quant_mx32.argtypes = [vp, i32, i32, vp, vp]
        L.orc_gemm_ref_nt.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, f32, f32, i32]
        L.orc_gemm_ref_blockscale.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i64, i32, i32, i32, i32]
        L.orc_gemm_ref_blockscale_rows.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i64, i32]
        L.orc_gemm_ref_kn.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32]
        L.orc_gemm_ref_mx.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i32]
        L.orc_gemm_ref_nt_bf16.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32]
        L.orc_gemm_ref_kn_bf16.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32]
        for name in ("orc_shuffle_b_bf16", "orc_unshuffle_b_bf16"):
            getattr(L, name).argtypes = [vp, vp, i32, i32]
            getattr(L, name).restype = i32
        for name in ("orc_shuffle_b", "orc_unshuffle_b", "orc_shuffle_b_nk"):
            getattr(L, name).argtypes = [vp, vp, i32, i32]
            getattr(L, name).restype = i32
        L.orc_valid_vector.argtypes = [vp, vp, i64, f32, i32]
        L.orc_valid_vector.restype = i32
        L.orc_max_err.argtypes = [vp, vp, i64, vp, vp]
        L.orc_num_threads.restype = i32
        _lib = L
    return _lib


def _p(a: np.ndarray) -> C.c_void_p:
    assert a.flags["C_CONTIGUOUS"], "oracle wants C-contiguous arrays"
    return C.c_void_p(a.ctypes.data)


# ---- generators -----------------------------------------------------------------------
def fill_uniform(shape, seed: int, tensor_id: int, lo: float, hi: float) -> np.ndarray:
    out = np.empty(shape, np.float32)
    lib().orc_fill_uniform(_p(out), out.size, seed, tensor_id, lo, hi)
    return out


def fill_normal(shape, seed: int, tensor_id: int) -> np.ndarray:
    out = np.empty(shape, np.float32)
    lib().orc_fill_normal(_p(out), out.size, seed, tensor_id)
    return out


# ---- codecs ---------------------------------------------------------------------------
def e4m3_decode_table() -> np.ndarray:
    L = lib()
    return np.array([L.orc_e4m3_to_f32(i) for i in range(256)], np.float32)


def cast_e4m3(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    lib().orc_cast_e4m3(_p(x), x.size, _p(q))
    return q


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


# ---- quantisers -----------------------------------------------------------------------
def quant_tensor(x: np.ndarray):
    x = np.ascontiguousarray(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    s = np.zeros(1, np.float32)
    lib().orc_quant_tensor(_p(x), x.size, _p(q), _p(s))
    return q, s


def quant_1x128(x: np.ndarray):
    """x [M,K] -> q [M,K] uint8, sfa [K/128, M] float32 (the reference's transposed layout)."""
    x = np.ascontiguousarray(x, np.float32)
    M, K = x.shape
    assert K % 128 == 0
    q = np.empty((M, K), np.uint8)
    sfa = np.empty((K // 128, M), np.float32)
    lib().orc_quant_1x128(_p(x), M, K, _p(q), _p(sfa))
    return q, sfa


def quant_128x128(x: np.ndarray):
    """x [N,K] -> q [N,K] uint8, sfb [N/128, K/128] float32."""
    x = np.ascontiguousarray(x, np.float32)
    N, K = x.shape
    assert N % 128 == 0 and K % 128 == 0
    q = np.empty((N, K), np.uint8)
    sfb = np.empty((N // 128, K // 128), np.float32)
    lib().orc_quant_128x128(_p(x), N, K, _p(q), _p(sfb))
    return q, sfb


def quant_mx32(x: np.ndarray):
    """x [R,K] -> q [R,K] uint8, sf [R, K/32] uint8 (E8M0)."""
    x = np.ascontiguousarray(x, np.float32)
    R, K = x.shape
    assert K % 32 == 0
    q = np.empty((R, K), np.uint8)
    sf = np.empty((R, K // 32), np.uint8)
    lib().orc_quant_mx32(_p(x), R, K, _p(q), _p(sf))
    return q, sf


# ---- GEMM references ------------------------------------------------------------------
def _out(m, n, out_bf16):
    return np.empty((m, n), np.uint16 if out_bf16 else np.float32)


def gemm_ref_nt(a, b, scale_a=1.0, scale_b=1.0, out_bf16=False):
    m, k = a.shape
    n = b.shape[0]
    c = _out(m, n, out_bf16)
    lib().orc_gemm_ref_nt(_p(a), _p(b), _p(c), m, n, k, k, k, n, float(scale_a), float(scale_b), int(out_bf16))
    return c


def gemm_ref_blockscale(a, b, sfa, sfb, out_bf16=False, rows=None):
    m, k = a.shape
    n = b.shape[0]
    assert sfa.shape == (k // 128, m) and sfb.shape == (n // 128, k // 128)
    if rows is None:
        c = _out(m, n, out_bf16)
        lib().orc_gemm_ref_blockscale(_p(a), _p(b), _p(sfa), _p(sfb), _p(c), m, n, k, k, k, n, m, k // 128,
                                      1, 128, 128, int(out_bf16))
        return c
    m0, m1 = rows
    c = _out(m, n, out_bf16)
    lib().orc_gemm_ref_blockscale_rows(_p(a), _p(b), _p(sfa), _p(sfb), _p(c), m0, m1, n, k, k, k, n, m, k // 128,
                                       int(out_bf16))
    return c[m0:m1]


def gemm_ref_kn(a, b_kn, out_bf16=False):
    m, k = a.shape
    n = b_kn.shape[1]
    c = _out(m, n, out_bf16)
    lib().orc_gemm_ref_kn(_p(a), _p(b_kn), _p(c), m, n, k, k, n, n, int(out_bf16))
    return c


def gemm_ref_mx(a, b, sfa, sfb, out_bf16=False):
    m, k = a.shape
    n = b.shape[0]
    c = _out(m, n, out_bf16)
    lib().orc_gemm_ref_mx(_p(a), _p(b), _p(sfa), _p(sfb), _p(c), m, n, k, k, k, n, int(out_bf16))
    return c


# ---- layout ---------------------------------------------------------------------------
def shuffle_b(b_kn: np.ndarray) -> np.ndarray:
    K, N = b_kn.shape
    out = np.empty(N * K, np.uint8)
    if lib().orc_shuffle_b(_p(b_kn), _p(out), N, K) != 0:
        raise ValueError("shuffle_b needs N % 16 == 0 and K % 16 == 0")
    return out


def unshuffle_b(flat: np.ndarray, N: int, K: int) -> np.ndarray:
    out = np.empty((K, N), np.uint8)
    if lib().orc_unshuffle_b(_p(flat), _p(out), N, K) != 0:
        raise ValueError("unshuffle_b needs N % 16 == 0 and K % 16 == 0")
    return out


def shuffle_b_nk(b_nk: np.ndarray) -> np.ndarray:
    N, K = b_nk.shape
    out = np.empty(N * K, np.uint8)
    if lib().orc_shuffle_b_nk(_p(b_nk), _p(out), N, K) != 0:
        raise ValueError("shuffle_b needs N % 16 == 0 and K % 16 == 0")
    return out


# ---- a16w16 siblings (bf16 bit patterns as uint16) ----------------------------------------------
def gemm_ref_nt_bf16(a_bits, b_bits, out_bf16=True):
    m, k = a_bits.shape
    n = b_bits.shape[0]
    c = _out(m, n, out_bf16)
    lib().orc_gemm_ref_nt_bf16(_p(a_bits), _p(b_bits), _p(c), m, n, k, k, k, n, int(out_bf16))
    return c


def gemm_ref_kn_bf16(a_bits, b_kn_bits, out_bf16=True):
    m, k = a_bits.shape
    n = b_kn_bits.shape[1]
    c = _out(m, n, out_bf16)
    lib().orc_gemm_ref_kn_bf16(_p(a_bits), _p(b_kn_bits), _p(c), m, n, k, k, n, n, int(out_bf16))
    return c


def shuffle_b_bf16(b_kn_bits: np.ndarray) -> np.ndarray:
    K, N = b_kn_bits.shape
    out = np.empty(N * K, np.uint16)
    if lib().orc_shuffle_b_bf16(_p(b_kn_bits), _p(out), N, K) != 0:
        raise ValueError("bf16 shuffle_b needs N % 16 == 0 and K % 8 == 0")
    return out


def unshuffle_b_bf16(flat: np.ndarray, N: int, K: int) -> np.ndarray:
    out = np.empty((K, N), np.uint16)
    if lib().orc_unshuffle_b_bf16(_p(flat), _p(out), N, K) != 0:
        raise ValueError("bf16 unshuffle_b needs N % 16 == 0 and K % 8 == 0")
    return out


# ---- checker --------------------------------------------------------------------------
def valid_vector(ref, res, threshold, verbose=False) -> bool:
    ref = np.ascontiguousarray(ref, np.float32)
    res = np.ascontiguousarray(res, np.float32)
    return bool(lib().orc_valid_vector(_p(ref), _p(res), ref.size, threshold, int(verbose)))


def max_err(ref, res):
    ref = np.ascontiguousarray(ref, np.float32)
    res = np.ascontiguousarray(res, np.float32)
    e = np.zeros(1, np.float32)
    r = np.zeros(1, np.float32)
    lib().orc_max_err(_p(ref), _p(res), ref.size, _p(e), _p(r))
    return float(e[0]), float(r[0])


def num_threads() -> int:
    return lib().orc_num_threads()
