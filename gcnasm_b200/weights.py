"""Weight files: a pre-quantised, optionally pre-shuffled B operand with its scales on disk.

The reference re-shuffles the weights on the host at every start (``opus_fmm/flatmm_a8w8_gfx950.cc:736-742``) and
has no file format.  This is the host-side front end of ``b200_weight_file_*`` (C, in ``libb200gemm.so``); no GPU is
involved.  Layout: 128-byte header, N*K operand bytes, padding to 64, scale bytes; FNV-1a/64 checksum.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

from . import _lib as L
from ._lib import check, lib


class WeightDesc(C.Structure):
    """``b200_weight_desc``"""

    _fields_ = [
        ("magic", C.c_char * 8), ("version", C.c_int32), ("b_layout", C.c_int32), ("scale_mode", C.c_int32),
        ("reserved0", C.c_int32), ("n", C.c_int64), ("k", C.c_int64), ("data_bytes", C.c_int64),
        ("scale_bytes", C.c_int64), ("checksum", C.c_uint64), ("reserved", C.c_uint8 * 64),
    ]


@dataclass
class WeightInfo:
    n: int
    k: int
    b_layout: int
    scale_mode: int
    data_bytes: int
    scale_bytes: int
    checksum: int


def save(path: str, data: np.ndarray, scales: Optional[np.ndarray], n: int, k: int, *, b_layout: int = L.B_NK_ROWMAJOR,
         scale_mode: int = L.SCALE_NONE) -> None:
    """``data``: N*K e4m3 bytes in ``b_layout``; ``scales``: the scale bytes of ``scale_mode`` (fp32 ``[N/128, K/128]``
    for block scales, MX atoms, one fp32 for per-tensor) or None."""
    data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    if data.size != n * k:
        raise ValueError("data must hold N*K bytes")
    sp = None
    if scales is not None:
        scales = np.ascontiguousarray(scales)
        sp = scales.ctypes.data
    check(lib().b200_weight_file_write(path.encode(), b_layout, scale_mode, n, k, data.ctypes.data, sp),
          "b200_weight_file_write")


def stat(path: str) -> WeightInfo:
    d = WeightDesc()
    check(lib().b200_weight_file_stat(path.encode(), C.byref(d)), "b200_weight_file_stat")
    return WeightInfo(d.n, d.k, d.b_layout, d.scale_mode, d.data_bytes, d.scale_bytes, d.checksum)


def load(path: str) -> Tuple[WeightInfo, np.ndarray, Optional[np.ndarray]]:
    """Returns (info, operand bytes as uint8 [N*K], scales).  Block scales come back as fp32 ``[N/128, K/128]``,
    per-tensor as fp32 ``[1]``, MX atoms as uint8; the checksum is verified."""
    info = stat(path)
    data = np.empty(info.data_bytes, np.uint8)
    raw = np.empty(info.scale_bytes, np.uint8) if info.scale_bytes else None
    check(lib().b200_weight_file_read(path.encode(), data.ctypes.data, data.nbytes, raw.ctypes.data if raw is not None else None,
                                      raw.nbytes if raw is not None else 0), "b200_weight_file_read")
    scales = raw
    if raw is not None and info.scale_mode == L.SCALE_BLOCK:
        scales = raw.view(np.float32).reshape(info.n // 128, info.k // 128)
    elif raw is not None and info.scale_mode == L.SCALE_TENSOR:
        scales = raw.view(np.float32)
    return info, data, scales
