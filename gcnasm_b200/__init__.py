"""B200-native (sm_100a) A8W8 FP8 GEMM family behind the reference's operator surface.

Importing the package does not load the native library; the first operator call does, and raises if
``libb200gemm.so`` has not been built -- there is no CPU or third-party-library fallback.
"""
from . import _lib  # noqa: F401
from ._lib import (B200Error, B_FLAT_16x16, B_NK_ROWMAJOR, OUT_BF16, OUT_F32, SCALE_BLOCK, SCALE_MX, SCALE_NONE,  # noqa: F401
                   SCALE_TENSOR, TILE_128x128, TILE_128x256, TILE_AUTO, TILE_DECODE)

__all__ = ["api", "build"]
