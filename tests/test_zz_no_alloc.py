"""GPU: the allocation-free skinny-M entry point, b200_gemm_a8w8_decode_static.

Some users of this library may not allocate device memory once they are running -- a serving loop with a
memory plan fixed at start-up, a latency-critical thread that cannot afford cudaMalloc's device-wide
synchronisation, a host that gives the library a fixed budget.  For them the split-K workspace of the skinny-M
kernel sits in a fixed 1 MiB array inside the library instead of in cudaMalloc'd memory.  This file checks,
through the C ABI, that the variant returns exactly what b200_gemm_a8w8 returns -- on two calls in a row that
share the array and leave different contents in it -- and that a problem whose partials do not fit is refused.
It is collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _args(a, b, sfa, sfb, out):
    from gcnasm_b200._lib import GemmArgs, OUT_F32, SCALE_BLOCK

    m, k = a.shape
    n = b.shape[0]
    g = GemmArgs()
    g.ptr_a, g.ptr_b, g.ptr_c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.m, g.n, g.k, g.batch = m, n, k, 1
    g.stride_a, g.stride_b, g.stride_c = k, k, n
    g.stride_a_batch, g.stride_b_batch, g.stride_c_batch = m * k, n * k, m * n
    g.ptr_sfa, g.ptr_sfb = sfa.data_ptr(), sfb.data_ptr()
    g.stride_sfa, g.stride_sfb = m, k // 128
    g.stride_sfa_batch, g.stride_sfb_batch = m * (k // 128), (n // 128) * (k // 128)
    g.scale_mode, g.out_dtype = SCALE_BLOCK, OUT_F32
    return g


def _problem(O, m, n, k, seed):
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(DEV)
    a = T(O.cast_e4m3(O.fill_uniform((m, k), seed, 0, 0.0, 1.0)))
    b = T(O.cast_e4m3(O.fill_uniform((n, k), seed, 1, -0.5, 0.5)))
    sfa = T(O.fill_uniform((k // 128, m), seed, 2, 0.8, 1.2))
    sfb = T(O.fill_uniform((n // 128, k // 128), seed, 3, 0.8, 1.2))
    return a, b, sfa, sfb


def test_static_scratch_variant_matches_regular_entry(native, O):
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # few weight panels and a long K: the launcher splits K, so the workspace is really used; the second
    # problem has another shape and other data, so it finds the first call's partials in the array
    for call, (m, n, k, seed) in enumerate([(16, 1024, 4096, 21), (5, 512, 2048, 22)]):
        a, b, sfa, sfb = _problem(O, m, n, k, seed)
        want = torch.full((m, n), -7.0, dtype=torch.float32, device=DEV)
        got = torch.full((m, n), 9.0, dtype=torch.float32, device=DEV)
        assert native.b200_gemm_a8w8(C.byref(_args(a, b, sfa, sfb, want)), stream) == 0
        assert native.b200_gemm_a8w8_decode_static(C.byref(_args(a, b, sfa, sfb, got)), stream) == 0
        torch.cuda.synchronize()
        assert native.b200_last_status() == 0
        # same kernels, same order of additions: bit-identical, well inside the suite's 1e-2 * max|ref| bound
        assert torch.equal(got, want), f"call {call}: static-scratch result differs from b200_gemm_a8w8"
        ref = O.gemm_ref_blockscale(a.cpu().numpy(), b.cpu().numpy(), sfa.cpu().numpy(), sfb.cpu().numpy())
        err, mref = O.max_err(ref, got.cpu().numpy())
        assert err <= 1e-2 * mref


def test_static_scratch_variant_refuses_what_does_not_fit(native, O):
    from gcnasm_b200 import _lib as L

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 8 weight panels -> 16 K splits -> 16 * 64 * 1024 partials = 4 MiB, more than the 1 MiB array
    a, b, sfa, sfb = _problem(O, 64, 1024, 8192, 23)
    out = torch.zeros((64, 1024), dtype=torch.float32, device=DEV)
    assert native.b200_gemm_a8w8_decode_static(C.byref(_args(a, b, sfa, sfb, out)), stream) == L.ERR_TOO_LARGE
    torch.cuda.synchronize()
    assert torch.all(out == 0)                         # nothing was launched
    # a shape that does not go to the skinny-M kernel at all
    a, b, sfa, sfb = _problem(O, 128, 256, 256, 24)
    out = torch.zeros((128, 256), dtype=torch.float32, device=DEV)
    assert native.b200_gemm_a8w8_decode_static(C.byref(_args(a, b, sfa, sfb, out)), stream) == L.ERR_UNSUPPORTED
