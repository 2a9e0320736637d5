"""ctypes/numpy front end of ``oracle/_ref``: the reference's own host checkers compiled by ``ref_build.py``.

TEST INFRASTRUCTURE ONLY.  ``strict`` is the build with IEEE evaluation order, ``fast`` the one with the
``-ffast-math`` of the reference's Makefiles.  Operands are the same numpy arrays the restated oracle takes:
e4m3 bytes as uint8, bf16 bit patterns as uint16.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import ref_build

_libs = {}


def available() -> bool:
    return ref_build.available()


def build(reference_root=None):
    """Builds oracle/_ref when a reference checkout is at hand; returns whether the libraries exist afterwards."""
    ref_build.build(reference_root)
    return available()


def lib(flavour: str = "strict") -> C.CDLL:
    if flavour not in _libs:
        path = os.path.join(ref_build.OUT, "libref_%s.so" % flavour)
        if not os.path.exists(path):
            raise FileNotFoundError(path + " (python oracle/ref_build.py <reference checkout> builds it)")
        L = C.CDLL(path)
        vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
        L.ref_cast_e4m3.restype, L.ref_cast_e4m3.argtypes = C.c_uint8, [f32]
        L.ref_e4m3_to_f32.restype, L.ref_e4m3_to_f32.argtypes = f32, [C.c_uint8]
        L.ref_gemm_nt.argtypes = [vp, vp, vp] + [i32] * 6
        L.ref_gemm_blockscale.argtypes = [vp, vp, vp, vp, vp] + [i32] * 11
        L.ref_gemm_kn.argtypes = [vp, vp, vp] + [i32] * 6
        L.ref_shuffle_b.argtypes = [vp, vp, i32, i32]
        L.ref_gemm_nt_bf16.argtypes = [vp, vp, vp] + [i32] * 6
        L.ref_gemm_kn_bf16.argtypes = [vp, vp, vp] + [i32] * 6
        L.ref_shuffle_b_bf16.argtypes = [vp, vp, i32, i32]
        for name in ("ref_valid_vector", "ref_valid_vector_bs"):
            getattr(L, name).argtypes = [vp, vp, i32, f32]
            getattr(L, name).restype = i32
        L.ref_fast_math.restype = i32
        assert L.ref_fast_math() == (1 if flavour == "fast" else 0)
        _libs[flavour] = L
    return _libs[flavour]


def _p(a: np.ndarray) -> C.c_void_p:
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def cast_e4m3(x: np.ndarray) -> np.ndarray:
    L = lib()
    return np.array([L.ref_cast_e4m3(float(v)) for v in np.asarray(x, np.float32).ravel()], np.uint8).reshape(np.shape(x))


def e4m3_decode_table() -> np.ndarray:
    L = lib()
    return np.array([L.ref_e4m3_to_f32(i) for i in range(256)], np.float32)


def gemm_ref_nt(a, b, flavour="strict"):
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), np.float32)
    lib(flavour).ref_gemm_nt(_p(a), _p(b), _p(c), m, n, k, k, k, n)
    return c


def gemm_ref_blockscale(a, b, sfa, sfb, flavour="strict", group=(1, 128, 128)):
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), np.float32)
    lib(flavour).ref_gemm_blockscale(_p(a), _p(b), _p(sfa), _p(sfb), _p(c), m, n, k, k, k, n, sfa.shape[1], sfb.shape[1], *group)
    return c


def gemm_ref_kn(a, b_kn, flavour="strict"):
    m, k = a.shape
    n = b_kn.shape[1]
    c = np.empty((m, n), np.float32)
    lib(flavour).ref_gemm_kn(_p(a), _p(b_kn), _p(c), m, n, k, k, n, n)
    return c


def shuffle_b(b_kn):
    K, N = b_kn.shape
    out = np.empty(N * K, np.uint8)
    lib().ref_shuffle_b(_p(b_kn), _p(out), N, K)
    return out


def gemm_ref_nt_bf16(a_bits, b_bits, flavour="strict"):
    m, k = a_bits.shape
    n = b_bits.shape[0]
    c = np.empty((m, n), np.uint16)
    lib(flavour).ref_gemm_nt_bf16(_p(a_bits), _p(b_bits), _p(c), m, n, k, k, k, n)
    return c


def gemm_ref_kn_bf16(a_bits, b_kn_bits, flavour="strict"):
    m, k = a_bits.shape
    n = b_kn_bits.shape[1]
    c = np.empty((m, n), np.uint16)
    lib(flavour).ref_gemm_kn_bf16(_p(a_bits), _p(b_kn_bits), _p(c), m, n, k, k, n, n)
    return c


def shuffle_b_bf16(b_kn_bits):
    K, N = b_kn_bits.shape
    out = np.empty(N * K, np.uint16)
    lib().ref_shuffle_b_bf16(_p(b_kn_bits), _p(out), N, K)
    return out


def valid_vector(ref, res, threshold, which="a8w8") -> bool:
    ref = np.ascontiguousarray(ref, np.float32)
    res = np.ascontiguousarray(res, np.float32)
    fn = lib().ref_valid_vector if which == "a8w8" else lib().ref_valid_vector_bs
    return bool(fn(_p(ref), _p(res), ref.size, threshold))
