"""Host-side operators over the C ABI.  PyTorch supplies device memory and streams only.

Names and argument meaning follow the reference programs: ``gemm_a8w8`` (opus_gemm/gemm_a8w8_8wave.cc),
``gemm_a8w8_blockscale`` (opus_gemm/block_scale_gemm) and ``flatmm_a8w8`` + ``shuffle_b``
(opus_fmm/flatmm_a8w8_gfx950.cc).  A is ``[batch, M, K]`` (or ``[M, K]``), B is ``[batch, N, K]`` -- the NT
layout ``C = A . B^T`` -- operands are OCP E4M3 bytes (``torch.uint8`` or ``torch.float8_e4m3fn``).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
from typing import Optional

from . import _lib as L
from ._lib import GemmArgs, check, lib

_FP8 = (torch.uint8, torch.float8_e4m3fn)


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _same_device(*tensors) -> torch.device:
    """Every CUDA operand of a call must live on ONE device, and that device must be the current one: the C side
    picks its per-device state and the launch device with cudaGetDevice(), and the stream comes from
    ``torch.cuda.current_stream()``.  A tensor of another GPU would put a foreign address into a tensor map and
    fault on the device instead of raising here."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("operands must be CUDA tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"operands live on different devices: {dev} and {t.device}")
    if dev is not None and dev.index != torch.cuda.current_device():
        raise ValueError(f"operands live on {dev} but the current device is cuda:{torch.cuda.current_device()}; "
                         "wrap the call in `with torch.cuda.device(tensor.device):`")
    return dev


def _as_u8(t: torch.Tensor, what: str) -> torch.Tensor:
    if t.dtype not in _FP8:
        raise TypeError(f"{what} must hold E4M3 bytes (uint8 or float8_e4m3fn), got {t.dtype}")
    if not t.is_cuda:
        raise ValueError(f"{what} must be a CUDA tensor")
    return t.view(torch.uint8)


def _out_code(dtype) -> int:
    if dtype == torch.bfloat16:
        return L.OUT_BF16
    if dtype == torch.float32:
        return L.OUT_F32
    raise TypeError("output dtype must be torch.bfloat16 or torch.float32")


def _gemm(a, b, *, n=None, sfa=None, sfb=None, scale_a=None, scale_b=None, scale_mode=L.SCALE_NONE,
          b_layout=L.B_NK_ROWMAJOR, out=None, out_dtype=torch.bfloat16, tile=L.TILE_AUTO, simple=False, inputs_ready=False,
          batch_ready=None, batch_epoch=0):
    a = _as_u8(a, "A")
    b = _as_u8(b, "B")
    _same_device(a, b, sfa, sfb, scale_a, scale_b, out, batch_ready)
    squeeze = a.dim() == 2
    if squeeze:
        a = a.unsqueeze(0)
    batch, m, k = a.shape
    if a.stride(2) != 1:
        raise ValueError("A must be K-contiguous")
    # a 2-D B (or scale tensor) given with a batched A is ONE operand shared by every batch (batch stride 0)
    b_shared = batch > 1 and b_layout == L.B_NK_ROWMAJOR and b.dim() == 2
    if b_layout == L.B_NK_ROWMAJOR:
        if b.dim() == 2:
            b = b.unsqueeze(0)
        if (not b_shared and b.shape[0] != batch) or b.shape[2] != k or b.stride(2) != 1:
            raise ValueError("B must be [batch, N, K] (or [N, K], shared by all batches), K-contiguous, matching A")
        n = b.shape[1]
        stride_b, stride_b_batch = b.stride(1), (0 if b_shared else b.stride(0))
    else:
        if n is None:
            raise ValueError("flat B needs n=")
        if not b.is_contiguous() or b.numel() != batch * n * k:
            raise ValueError("flat B must be a contiguous image of batch*N*K bytes")
        stride_b, stride_b_batch = n, n * k       # the reference sets stride_b = N (flatmm_a8w8_gfx950.cc:765)
    if out is None:
        out = torch.empty((batch, m, n), dtype=out_dtype, device=a.device)
    else:
        if out.dim() == 2:
            out = out.unsqueeze(0)
        if out.shape != (batch, m, n) or out.stride(2) != 1:
            raise ValueError("out must be [batch, M, N], N-contiguous")
    args = GemmArgs()
    args.ptr_a, args.ptr_b, args.ptr_c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.n, args.k, args.batch = m, n, k, batch
    args.stride_a, args.stride_b, args.stride_c = a.stride(1), stride_b, out.stride(1)
    args.stride_a_batch, args.stride_b_batch, args.stride_c_batch = a.stride(0), stride_b_batch, out.stride(0)
    keep = [a, b, out]
    if scale_mode == L.SCALE_BLOCK:
        if sfa.dim() == 2:
            sfa = sfa.unsqueeze(0)
        if sfb.dim() == 2:
            sfb = sfb.unsqueeze(0)
        if sfa.dtype != torch.float32 or sfb.dtype != torch.float32:
            raise TypeError("block scales are float32")
        if sfa.shape != (batch, k // 128, m) or sfb.shape != (1 if b_shared else batch, n // 128, k // 128):
            raise ValueError("SFA must be [batch, K/128, M] and SFB [batch, N/128, K/128] ([N/128, K/128] with a shared B)")
        if sfa.stride(2) != 1 or sfb.stride(2) != 1:
            raise ValueError("scale tensors must be contiguous in their last dimension")
        args.ptr_sfa, args.ptr_sfb = sfa.data_ptr(), sfb.data_ptr()
        args.stride_sfa, args.stride_sfb = sfa.stride(1), sfb.stride(1)
        args.stride_sfa_batch, args.stride_sfb_batch = sfa.stride(0), (0 if b_shared else sfb.stride(0))
        keep += [sfa, sfb]
    elif scale_mode == L.SCALE_MX:
        need_a, need_b = lib().b200_mx_sf_bytes(m, k), lib().b200_mx_sf_bytes(n, k)
        sfa = sfa.view(torch.uint8).reshape(batch, -1)
        sfb = sfb.view(torch.uint8).reshape(batch, -1)
        if sfa.shape[1] != need_a or sfb.shape[1] != need_b or not sfa.is_contiguous() or not sfb.is_contiguous():
            raise ValueError("MX scales must be the relayouted atom images (see mx_sf_relayout)")
        args.ptr_sfa, args.ptr_sfb = sfa.data_ptr(), sfb.data_ptr()
        args.stride_sfa_batch, args.stride_sfb_batch = need_a, need_b
        keep += [sfa, sfb]
    elif scale_mode == L.SCALE_TENSOR:
        for name, s in (("ptr_scale_a", scale_a), ("ptr_scale_b", scale_b)):
            if s is not None:
                if s.dtype != torch.float32 or not s.is_cuda or s.numel() != 1:
                    raise TypeError("per-tensor scales are 1-element float32 CUDA tensors")
                setattr(args, name, s.data_ptr())
                keep.append(s)
    args.scale_mode, args.b_layout = scale_mode, b_layout
    args.out_dtype, args.tile_hint = _out_code(out.dtype), tile
    args.flags = L.GEMM_INPUTS_READY if inputs_ready else 0
    if batch_ready is not None:
        if batch_ready.dtype != torch.int32 or batch_ready.numel() < batch or not batch_ready.is_contiguous():
            raise ValueError("batch_ready must be a contiguous int32 CUDA tensor with one word per batch")
        args.flags |= L.GEMM_BATCH_READY
        args.ptr_batch_ready, args.batch_epoch = batch_ready.data_ptr(), int(batch_epoch)
        keep.append(batch_ready)
    fn = lib().b200_gemm_a8w8_simple if simple else lib().b200_gemm_a8w8
    check(fn(C.byref(args), _stream()), "b200_gemm_a8w8_simple" if simple else "b200_gemm_a8w8")
    return out[0] if squeeze else out


# ---- operators ---------------------------------------------------------------------------------
def gemm_a8w8(a, b, scale_a=None, scale_b=None, *, out=None, out_dtype=torch.bfloat16, tile=L.TILE_AUTO, simple=False,
              inputs_ready=False):
    """``C = (A . B^T) [* scale_a * scale_b]``.  Without scales this is the reference's gemm_a8w8_8wave.
    ``inputs_ready``: see ``B200_GEMM_INPUTS_READY`` in the header (operands not written by work still in flight)."""
    mode = L.SCALE_TENSOR if (scale_a is not None or scale_b is not None) else L.SCALE_NONE
    return _gemm(a, b, scale_a=scale_a, scale_b=scale_b, scale_mode=mode, out=out, out_dtype=out_dtype, tile=tile,
                 simple=simple, inputs_ready=inputs_ready)


def gemm_a8w8_blockscale(a, b, sfa, sfb, *, out=None, out_dtype=torch.bfloat16, tile=L.TILE_AUTO, simple=False,
                         b_flat_n=None, inputs_ready=False, batch_ready=None, batch_epoch=0):
    """Block-scale GEMM: SFA fp32 ``[K/128, M]`` (1x128 groups, M contiguous), SFB fp32 ``[N/128, K/128]``.

    With a batched A ``[batch, M, K]`` a 2-D ``b`` / ``sfb`` is shared by every batch.  ``batch_ready`` (int32, one
    word per batch) makes the kernel wait for ``batch_ready[b] >= batch_epoch`` before it reads anything of batch b's
    A or SFA (``B200_GEMM_BATCH_READY``: slabs that are still being delivered while the kernel runs)."""
    if b_flat_n is not None:
        return _gemm(a, b, n=b_flat_n, sfa=sfa, sfb=sfb, scale_mode=L.SCALE_BLOCK, b_layout=L.B_FLAT_16x16, out=out,
                     out_dtype=out_dtype, tile=tile, simple=simple, inputs_ready=inputs_ready)
    return _gemm(a, b, sfa=sfa, sfb=sfb, scale_mode=L.SCALE_BLOCK, out=out, out_dtype=out_dtype, tile=tile, simple=simple,
                 inputs_ready=inputs_ready, batch_ready=batch_ready, batch_epoch=batch_epoch)


def flag_write(flags: torch.Tensor, index: int, value: int) -> None:
    """Stream-ordered write of ``value`` into ``flags[index]`` (int32) on the current stream: it happens when everything
    queued on that stream before it has completed.  No kernel is launched (``b200_flag_write``)."""
    if flags.dtype != torch.int32 or not flags.is_contiguous():
        raise ValueError("flags must be a contiguous int32 CUDA tensor")
    _same_device(flags)
    if not (0 <= index < flags.numel()):
        raise IndexError("flag index out of range")
    check(lib().b200_flag_write(flags.data_ptr() + 4 * index, int(value), _stream()), "b200_flag_write")


def gemm_a8w8_mx(a, b, sfa_atoms, sfb_atoms, *, out=None, out_dtype=torch.bfloat16, tile=L.TILE_AUTO, simple=False):
    """MXFP8 GEMM: E8M0 scales per 1x32 block, given in the relayouted atom order."""
    return _gemm(a, b, sfa=sfa_atoms, sfb=sfb_atoms, scale_mode=L.SCALE_MX, out=out, out_dtype=out_dtype, tile=tile,
                 simple=simple)


def flatmm_a8w8(a, b_flat, n, scale_a=None, scale_b=None, *, out=None, out_dtype=torch.bfloat16, tile=L.TILE_AUTO,
                simple=False):
    """GEMM on a pre-shuffled B (output of :func:`shuffle_b`), the reference's flatmm_a8w8."""
    mode = L.SCALE_TENSOR if (scale_a is not None or scale_b is not None) else L.SCALE_NONE
    return _gemm(a, b_flat, n=n, scale_a=scale_a, scale_b=scale_b, scale_mode=mode, b_layout=L.B_FLAT_16x16, out=out,
                 out_dtype=out_dtype, tile=tile, simple=simple)


def shuffle_b(b: torch.Tensor, src: str = "kn") -> torch.Tensor:
    """Pre-shuffle a weight matrix into the flat layout ``[N/16][K/16][16][16]``.

    ``src='kn'``: ``b`` is ``[K, N]`` (what the reference's shuffle_b takes); ``src='nk'``: ``b`` is ``[N, K]``.
    """
    b = _as_u8(b, "B")
    _same_device(b)
    if not b.is_contiguous() or b.dim() != 2:
        raise ValueError("B must be a contiguous 2-D tensor")
    k, n = (b.shape if src == "kn" else (b.shape[1], b.shape[0]))
    out = torch.empty(n * k, dtype=torch.uint8, device=b.device)
    check(lib().b200_shuffle_b(b.data_ptr(), out.data_ptr(), n, k, 1 if src == "kn" else 0, _stream()), "b200_shuffle_b")
    return out


def unshuffle_b(flat: torch.Tensor, n: int, k: int, dst: str = "kn") -> torch.Tensor:
    flat = _as_u8(flat, "flat B")
    _same_device(flat)
    if not flat.is_contiguous() or flat.numel() != n * k:
        raise ValueError("flat B must be a contiguous image of N*K bytes")
    out = torch.empty((k, n) if dst == "kn" else (n, k), dtype=torch.uint8, device=flat.device)
    check(lib().b200_unshuffle_b(flat.data_ptr(), out.data_ptr(), n, k, 1 if dst == "kn" else 0, _stream()),
          "b200_unshuffle_b")
    return out


# ---- quantisers ----------------------------------------------------------------------------------
def _f32(x: torch.Tensor) -> torch.Tensor:
    if x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
        raise TypeError("quantiser input must be a contiguous float32 CUDA tensor")
    _same_device(x)
    return x


def cast_e4m3(x):
    x = _f32(x)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    check(lib().b200_cast_e4m3(x.data_ptr(), q.data_ptr(), x.numel(), _stream()), "b200_cast_e4m3")
    return q


def quantize_tensor(x):
    x = _f32(x)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    ws = torch.empty(lib().b200_quantize_tensor_workspace(), dtype=torch.uint8, device=x.device)
    check(lib().b200_quantize_tensor(x.data_ptr(), q.data_ptr(), scale.data_ptr(), x.numel(), ws.data_ptr(), _stream()),
          "b200_quantize_tensor")
    return q, scale


def quantize_1x128(x):
    x = _f32(x)
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    sfa = torch.empty((k // 128, m), dtype=torch.float32, device=x.device)
    check(lib().b200_quantize_1x128(x.data_ptr(), q.data_ptr(), sfa.data_ptr(), m, k, _stream()), "b200_quantize_1x128")
    return q, sfa


def quantize_128x128(x):
    x = _f32(x)
    n, k = x.shape
    q = torch.empty((n, k), dtype=torch.uint8, device=x.device)
    sfb = torch.empty((n // 128, k // 128), dtype=torch.float32, device=x.device)
    check(lib().b200_quantize_128x128(x.data_ptr(), q.data_ptr(), sfb.data_ptr(), n, k, _stream()), "b200_quantize_128x128")
    return q, sfb


def mx_sf_relayout(sf: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    sf = sf.view(torch.uint8)
    if not sf.is_contiguous() or sf.numel() != rows * (k // 32):
        raise ValueError("sf must be a contiguous [rows, K/32] byte tensor")
    out = torch.empty(lib().b200_mx_sf_bytes(rows, k), dtype=torch.uint8, device=sf.device)
    check(lib().b200_mx_sf_relayout(sf.data_ptr(), out.data_ptr(), rows, k, _stream()), "b200_mx_sf_relayout")
    return out


def quantize_mx32(x):
    """Returns (q [R,K] uint8, sf [R,K/32] E8M0 bytes, sf_atoms for the GEMM)."""
    x = _f32(x)
    r, k = x.shape
    q = torch.empty((r, k), dtype=torch.uint8, device=x.device)
    sf = torch.empty((r, k // 32), dtype=torch.uint8, device=x.device)
    check(lib().b200_quantize_mx32(x.data_ptr(), q.data_ptr(), sf.data_ptr(), r, k, _stream()), "b200_quantize_mx32")
    atoms = mx_sf_relayout(sf, r, k) if k % 128 == 0 else None
    return q, sf, atoms


def quantize_act_bf16_1x128(x, q=None, sfa=None):
    """Fused activation quantiser: bf16 [M,K] (rows may be strided) -> (q [M,K] uint8, sfa [K/128, M] fp32) in one
    pass.  `q` / `sfa` may be preallocated views (e.g. slices of a broadcast buffer); q rows may be strided."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a 2-D bf16 tensor with unit column stride")
    _same_device(x, q, sfa)
    m, k = x.shape
    if q is None:
        q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    if sfa is None:
        sfa = torch.empty((k // 128, m), dtype=torch.float32, device=x.device)
    if q.shape != (m, k) or q.dtype != torch.uint8 or q.stride(1) != 1:
        raise ValueError("q must be a [M,K] uint8 tensor with unit column stride")
    if sfa.shape != (k // 128, m) or sfa.dtype != torch.float32 or sfa.stride(1) != 1:
        raise ValueError("sfa must be a [K/128, M] fp32 tensor with unit column stride")
    check(lib().b200_quantize_act_bf16_1x128(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), sfa.data_ptr(),
                                             sfa.stride(0) if k > 128 else m, m, k, _stream()), "b200_quantize_act_bf16_1x128")
    return q, sfa


def quantize_act_bf16_mx32(x):
    """Fused MX activation quantiser: bf16 [R,K] -> (q [R,K] uint8, scale atoms for the MX GEMM) in one pass."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a 2-D bf16 tensor with unit column stride")
    _same_device(x)
    r, k = x.shape
    q = torch.empty((r, k), dtype=torch.uint8, device=x.device)
    atoms = torch.empty(lib().b200_mx_sf_bytes(r, k), dtype=torch.uint8, device=x.device)
    check(lib().b200_quantize_act_bf16_mx32(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), atoms.data_ptr(), r, k,
                                            _stream()), "b200_quantize_act_bf16_mx32")
    return q, atoms


# ---- a16w16 siblings (bf16 operands) ----------------------------------------------------------------
def gemm_a16w16(a, b, scale_a=None, scale_b=None, *, n=None, flat=False, out=None, out_dtype=torch.bfloat16,
                tile=L.TILE_AUTO):
    """``C = A @ B^T`` on bf16 operands, fp32 accumulate (``opus_gemm/gemm_a16w16_8wave.cc``).  ``a`` is
    ``[M, K]`` or ``[batch, M, K]`` bf16; ``b`` is ``[N, K]`` / ``[batch, N, K]`` bf16, or with ``flat=True`` the
    image made by :func:`shuffle_b_bf16` (then ``n=`` is required)."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("A and B must be torch.bfloat16")
    _same_device(a, b, scale_a, scale_b, out)
    squeeze = a.dim() == 2
    if squeeze:
        a = a.unsqueeze(0)
    batch, m, k = a.shape
    if a.stride(2) != 1:
        raise ValueError("A must be K-contiguous")
    if not flat:
        if b.dim() == 2:
            b = b.unsqueeze(0)
        if b.shape[0] != batch or b.shape[2] != k or b.stride(2) != 1:
            raise ValueError("B must be [batch, N, K], K-contiguous, matching A")
        n = b.shape[1]
        stride_b, stride_b_batch = b.stride(1), b.stride(0)
    else:
        if n is None:
            raise ValueError("flat B needs n=")
        if not b.is_contiguous() or b.numel() != batch * n * k:
            raise ValueError("flat B must be a contiguous image of batch*N*K values")
        stride_b, stride_b_batch = n, n * k
    if out is None:
        out = torch.empty((batch, m, n), dtype=out_dtype, device=a.device)
    else:
        if out.dim() == 2:
            out = out.unsqueeze(0)
        if out.shape != (batch, m, n) or out.stride(2) != 1:
            raise ValueError("out must be [batch, M, N], N-contiguous")
    args = GemmArgs()
    args.ptr_a, args.ptr_b, args.ptr_c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.n, args.k, args.batch = m, n, k, batch
    args.stride_a, args.stride_b, args.stride_c = a.stride(1), stride_b, out.stride(1)
    args.stride_a_batch, args.stride_b_batch, args.stride_c_batch = a.stride(0), stride_b_batch, out.stride(0)
    keep = [a, b, out]
    mode = L.SCALE_NONE
    if scale_a is not None or scale_b is not None:
        mode = L.SCALE_TENSOR
        for name, sc in (("ptr_scale_a", scale_a), ("ptr_scale_b", scale_b)):
            if sc is not None:
                if sc.dtype != torch.float32 or not sc.is_cuda or sc.numel() != 1:
                    raise TypeError("per-tensor scales are 1-element float32 CUDA tensors")
                setattr(args, name, sc.data_ptr())
                keep.append(sc)
    args.scale_mode, args.b_layout = mode, (L.B_FLAT_16x16 if flat else L.B_NK_ROWMAJOR)
    args.out_dtype, args.tile_hint = _out_code(out.dtype), tile
    check(lib().b200_gemm_a16w16(C.byref(args), _stream()), "b200_gemm_a16w16")
    return out[0] if squeeze else out


def shuffle_b_bf16(b: torch.Tensor, src: str = "kn") -> torch.Tensor:
    """bf16 weights ``[K, N]`` (``src='kn'``, what the reference's shuffle_b takes) or ``[N, K]`` -> flat
    ``[N/16][K/8][16][8]`` (``opus_fmm/flatmm_a16w16_gfx950.cc:623-666``)."""
    if b.dtype != torch.bfloat16 or not b.is_contiguous() or b.dim() != 2:
        raise ValueError("B must be a contiguous 2-D bf16 tensor")
    _same_device(b)
    k, n = (b.shape if src == "kn" else (b.shape[1], b.shape[0]))
    out = torch.empty(n * k, dtype=torch.bfloat16, device=b.device)
    check(lib().b200_shuffle_b_bf16(b.data_ptr(), out.data_ptr(), n, k, 1 if src == "kn" else 0, _stream()),
          "b200_shuffle_b_bf16")
    return out


def unshuffle_b_bf16(flat: torch.Tensor, n: int, k: int, dst: str = "kn") -> torch.Tensor:
    if flat.dtype != torch.bfloat16 or not flat.is_contiguous() or flat.numel() != n * k:
        raise ValueError("flat B must be a contiguous bf16 image of N*K values")
    _same_device(flat)
    out = torch.empty((k, n) if dst == "kn" else (n, k), dtype=torch.bfloat16, device=flat.device)
    check(lib().b200_unshuffle_b_bf16(flat.data_ptr(), out.data_ptr(), n, k, 1 if dst == "kn" else 0, _stream()),
          "b200_unshuffle_b_bf16")
    return out


# ---- HBM bandwidth probe ----------------------------------------------------------------------------
def membw_read(buf: torch.Tensor, word_sum: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Streams `buf` once (read only); returns a 1-element int32 tensor holding the sum of its 32-bit words
    mod 2^32 (added to `word_sum` when given)."""
    _same_device(buf, word_sum)
    if word_sum is None:
        word_sum = torch.zeros(1, dtype=torch.int32, device=buf.device)
    check(lib().b200_membw_read(buf.data_ptr(), buf.numel() * buf.element_size(), word_sum.data_ptr(), _stream()),
          "b200_membw_read")
    return word_sum


def membw_copy(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """Streams `src` into `dst` (read + write)."""
    _same_device(src, dst)
    nbytes = src.numel() * src.element_size()
    if dst.numel() * dst.element_size() != nbytes:
        raise ValueError("src and dst differ in size")
    check(lib().b200_membw_copy(src.data_ptr(), dst.data_ptr(), nbytes, _stream()), "b200_membw_copy")
    return dst


# ---- seeded inputs (host) ---------------------------------------------------------------------------
def fill_uniform(shape, seed: int, tensor_id: int, lo: float, hi: float) -> np.ndarray:
    out = np.empty(shape, np.float32)
    lib().b200_fill_uniform(out.ctypes.data, out.size, seed, tensor_id, lo, hi)
    return out


def fill_normal(shape, seed: int, tensor_id: int) -> np.ndarray:
    out = np.empty(shape, np.float32)
    lib().b200_fill_normal(out.ctypes.data, out.size, seed, tensor_id)
    return out


# ---- host-buffer entry (the reference main()'s copy-in / launch / copy-out) -----------------------------
def gemm_a8w8_host(a: np.ndarray, b: np.ndarray, c: np.ndarray, *, sfa=None, sfb=None, scale_a=None, scale_b=None,
                   scale_mode=L.SCALE_NONE, b_layout=L.B_NK_ROWMAJOR, n=None, tile=L.TILE_AUTO, stream=None):
    """Operands and result are HOST arrays (numpy, or pinned torch tensors via ``.numpy()``)."""
    m, k = a.shape[-2], a.shape[-1]
    batch = a.shape[0] if a.ndim == 3 else 1
    if b_layout == L.B_NK_ROWMAJOR:
        n = b.shape[-2]
    args = GemmArgs()
    args.ptr_a, args.ptr_b, args.ptr_c = a.ctypes.data, b.ctypes.data, c.ctypes.data
    args.m, args.n, args.k, args.batch = m, n, k, batch
    args.stride_a, args.stride_b, args.stride_c = k, (k if b_layout == L.B_NK_ROWMAJOR else n), n
    args.stride_a_batch, args.stride_b_batch, args.stride_c_batch = m * k, n * k, m * n
    if scale_mode == L.SCALE_BLOCK:
        args.ptr_sfa, args.ptr_sfb = sfa.ctypes.data, sfb.ctypes.data
        args.stride_sfa, args.stride_sfb = m, k // 128
        args.stride_sfa_batch, args.stride_sfb_batch = m * (k // 128), (n // 128) * (k // 128)
    elif scale_mode == L.SCALE_MX:
        args.ptr_sfa, args.ptr_sfb = sfa.ctypes.data, sfb.ctypes.data
        args.stride_sfa_batch, args.stride_sfb_batch = lib().b200_mx_sf_bytes(m, k), lib().b200_mx_sf_bytes(n, k)
    elif scale_mode == L.SCALE_TENSOR:
        if scale_a is not None:
            args.ptr_scale_a = scale_a.ctypes.data
        if scale_b is not None:
            args.ptr_scale_b = scale_b.ctypes.data
    args.scale_mode, args.b_layout, args.tile_hint = scale_mode, b_layout, tile
    args.out_dtype = L.OUT_F32 if c.dtype == np.float32 else L.OUT_BF16
    st = C.c_void_p(stream if stream is not None else torch.cuda.current_stream().cuda_stream)
    check(lib().b200_gemm_a8w8_host(C.byref(args), st), "b200_gemm_a8w8_host")
    return c


def last_status() -> int:
    return lib().b200_last_status()


def peek_status() -> int:
    """The device status word without synchronising the device and without clearing it."""
    return lib().b200_peek_status()


def launch_count() -> int:
    return lib().b200_launch_count()


def last_tail_split():
    """(first split tile, column parts per tile) of this thread's last pair-kernel launch, or None when that launch
    computed every tile whole."""
    v = (C.c_int32 * 2)()
    hit = lib().b200_last_tail_split(C.byref(v, 0), C.byref(v, 4))
    return (v[0], v[1]) if hit else None
