"""CPU: the C-ABI surface -- the library loads, exports every symbol the header declares, the Python
struct mirrors the C struct, argument validation returns the documented codes, and nothing computes
without a GPU."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "b200gemm.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native):
    from gcnasm_b200 import _lib

    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(native, name), f"{name} declared in include/b200gemm.h but not exported"
    assert sorted(_lib.EXPORTS) == declared


def test_struct_layout_matches_c(native):
    from gcnasm_b200._lib import GemmArgs

    fields = [f[0] for f in GemmArgs._fields_]
    prog = '#include <stdio.h>\n#include <stddef.h>\n#include "b200gemm.h"\nint main(){printf("%zu", sizeof(b200_gemm_args));' + "".join(
        f'printf(" %zu", offsetof(b200_gemm_args, {f}));' for f in fields) + "return 0;}"
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.c")
        open(src, "w").write(prog)
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), src, "-o", os.path.join(d, "t")])
        out = subprocess.check_output([os.path.join(d, "t")]).decode().split()
    assert int(out[0]) == C.sizeof(GemmArgs)
    for f, off in zip(fields, out[1:]):
        assert getattr(GemmArgs, f).offset == int(off), f


def _args(**kw):
    from gcnasm_b200._lib import GemmArgs

    a = GemmArgs()
    a.ptr_a, a.ptr_b, a.ptr_c = 0x1000, 0x2000, 0x3000
    a.m, a.n, a.k, a.batch = 256, 512, 1024, 1
    a.stride_a, a.stride_b, a.stride_c = 1024, 1024, 512
    a.stride_a_batch, a.stride_b_batch, a.stride_c_batch = 256 * 1024, 512 * 1024, 256 * 512
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_validation_codes(native):
    from gcnasm_b200 import _lib as L

    tile = C.c_int32(0)
    chk = lambda a: native.b200_gemm_check(C.byref(a), C.byref(tile))
    assert chk(_args()) == L.OK and tile.value in (L.TILE_128x128, L.TILE_128x256, L.TILE_PAIR_256x128)
    assert native.b200_gemm_check(None, None) == L.ERR_BAD_ARG
    assert chk(_args(ptr_a=0)) == L.ERR_BAD_ARG
    # non-positive sizes are rejected like the reference's "Invalid problem size" (gemm_a8w8_8wave.cc:685-688)
    for f in ("m", "n", "k", "batch"):
        assert chk(_args(**{f: 0})) == L.ERR_BAD_ARG
        assert chk(_args(**{f: -4})) == L.ERR_BAD_ARG
    assert chk(_args(scale_mode=9)) == L.ERR_BAD_ARG
    assert chk(_args(stride_a=1000)) == L.ERR_BAD_ARG            # row pitch smaller than K
    assert chk(_args(k=1000, stride_a=1000, stride_b=1000)) == L.ERR_UNSUPPORTED   # K % 16 != 0
    assert chk(_args(ptr_a=0x1004)) == L.ERR_UNSUPPORTED          # TMA base alignment
    # block scale: N % 128 and K % 128 as gemm_a8w8_blockscale_host.cc:183, M arbitrary
    bs = dict(scale_mode=L.SCALE_BLOCK, ptr_sfa=0x4000, ptr_sfb=0x5000, stride_sfa=256, stride_sfb=8)
    assert chk(_args(**bs)) == L.OK
    assert chk(_args(**{**bs, "m": 77, "stride_sfa": 77})) == L.OK
    assert chk(_args(**{**bs, "n": 500, "stride_c": 500})) == L.ERR_UNSUPPORTED
    assert chk(_args(**{**bs, "k": 1040, "stride_a": 1040, "stride_b": 1040, "stride_sfb": 9})) == L.ERR_UNSUPPORTED
    assert chk(_args(**{**bs, "ptr_sfa": 0})) == L.ERR_BAD_ARG
    # flat B: whole 16x16 blocks (asserts at flatmm_a8w8_gfx950.cc:650-651)
    assert chk(_args(b_layout=L.B_FLAT_16x16)) == L.OK
    assert chk(_args(b_layout=L.B_FLAT_16x16, n=500, stride_c=500)) == L.ERR_UNSUPPORTED
    # tile selection: skinny M goes to the decode kernel, MX to 128x128
    assert chk(_args(m=16)) == L.OK and tile.value == L.TILE_DECODE
    assert chk(_args(**{**bs, "m": 64, "stride_sfa": 64})) == L.OK and tile.value == L.TILE_DECODE
    assert chk(_args(m=65)) == L.OK and tile.value != L.TILE_DECODE
    assert chk(_args(m=4096, n=7168, k=2048, stride_a=2048, stride_b=2048, stride_c=7168)) == L.OK and tile.value == L.TILE_PAIR_256x224
    bs2 = dict(scale_mode=L.SCALE_BLOCK, ptr_sfa=0x4000, ptr_sfb=0x5000, stride_sfa=4096, stride_sfb=16)
    assert chk(_args(m=4096, n=7168, k=2048, stride_a=2048, stride_b=2048, stride_c=7168, **bs2)) == L.OK and tile.value == L.TILE_PAIR_256x256
    assert chk(_args(m=8192, n=8192, k=8192, stride_a=8192, stride_b=8192, stride_c=8192)) == L.OK and tile.value == L.TILE_PAIR_256x256
    assert chk(_args(m=128, tile_hint=L.TILE_DECODE)) == L.ERR_UNSUPPORTED
    mx = dict(scale_mode=L.SCALE_MX, ptr_sfa=0x4000, ptr_sfb=0x5000)
    assert chk(_args(**mx)) == L.OK and tile.value in (L.TILE_128x128, L.TILE_PAIR_256x256)
    assert chk(_args(**mx, tile_hint=L.TILE_128x256)) == L.ERR_UNSUPPORTED
    assert chk(_args(**mx, k=1056, stride_a=1056, stride_b=1056)) == L.ERR_UNSUPPORTED


def test_helpers_and_strings(native):
    assert native.b200_strerror(0) == b"ok"
    assert b"unsupported" in native.b200_strerror(-2)
    assert native.b200_version().startswith(b"b200gemm")
    assert native.b200_mx_sf_bytes(8192, 8192) == 64 * 64 * 512
    assert native.b200_mx_sf_bytes(129, 128) == 2 * 512
    assert native.b200_quantize_tensor_workspace() >= 4
    assert native.b200_launch_count() >= 0


def test_layout_and_quantiser_argument_checks(native):
    from gcnasm_b200 import _lib as L

    assert native.b200_shuffle_b(0x1000, 0x2000, 24, 16, 1, None) == L.ERR_UNSUPPORTED
    assert native.b200_shuffle_b(0x1000, 0x2000, 16, 24, 1, None) == L.ERR_UNSUPPORTED
    assert native.b200_shuffle_b(None, 0x2000, 16, 16, 1, None) == L.ERR_BAD_ARG
    assert native.b200_quantize_1x128(0x1000, 0x2000, 0x3000, 4, 100, None) == L.ERR_UNSUPPORTED
    assert native.b200_quantize_128x128(0x1000, 0x2000, 0x3000, 100, 128, None) == L.ERR_UNSUPPORTED
    assert native.b200_quantize_mx32(0x1000, 0x2000, 0x3000, 4, 48, None) == L.ERR_UNSUPPORTED
    assert native.b200_mx_sf_relayout(0x1000, 0x2000, 4, 96, None) == L.ERR_UNSUPPORTED


def test_host_generators_match_oracle(native, O):
    from gcnasm_b200 import api

    for seed, tid in ((1234, 0), (7, 9)):
        assert np.array_equal(api.fill_uniform(10007, seed, tid, -1.0, 1.0), O.fill_uniform(10007, seed, tid, -1.0, 1.0))
        assert np.array_equal(api.fill_normal(10007, seed, tid), O.fill_normal(10007, seed, tid))


def test_no_gpu_means_error_not_fallback(native):
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for GPU-less machines")
    from gcnasm_b200 import _lib as L

    assert native.b200_gemm_a8w8(C.byref(_args()), None) in (L.ERR_NO_DEVICE, L.ERR_CUDA)
    assert native.b200_sm_count() < 0


def test_missing_library_fails_loudly(monkeypatch):
    from gcnasm_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libb200gemm.so")
    with pytest.raises(ImportError):
        _lib.lib()


def test_sibling_entry_argument_checks(native):
    """a16w16 check, bf16 shuffle, fused activation quantisers, bandwidth probe: validation only (no launch)."""
    from gcnasm_b200 import _lib as L

    tile = C.c_int32(0)
    chk = lambda a: native.b200_gemm_a16w16_check(C.byref(a), C.byref(tile))
    assert chk(_args()) == L.OK and tile.value in (L.TILE_128x128, L.TILE_128x256, L.TILE_PAIR_256x256)
    assert chk(_args(m=16)) == L.OK and tile.value != L.TILE_DECODE               # no bf16 skinny-M kernel
    assert chk(_args(m=8192, n=8192, k=8192, stride_a=8192, stride_b=8192, stride_c=8192)) == L.OK
    assert tile.value == L.TILE_PAIR_256x256
    assert chk(_args(k=1004, stride_a=1004, stride_b=1004)) == L.ERR_UNSUPPORTED   # K % 8 != 0 (bf16 rows of 16-byte units)
    assert chk(_args(k=1032, stride_a=1032, stride_b=1032)) == L.OK
    assert chk(_args(scale_mode=L.SCALE_BLOCK, ptr_sfa=0x4000, ptr_sfb=0x5000, stride_sfa=256, stride_sfb=8)) == L.ERR_UNSUPPORTED
    assert chk(_args(scale_mode=L.SCALE_TENSOR)) == L.OK
    assert chk(_args(b_layout=L.B_FLAT_16x16, k=1056, stride_a=1056)) == L.ERR_UNSUPPORTED     # flat bf16 needs K % 64 == 0
    assert chk(_args(b_layout=L.B_FLAT_16x16)) == L.OK
    assert chk(_args(tile_hint=L.TILE_PAIR_256x224)) == L.ERR_UNSUPPORTED
    assert native.b200_gemm_a16w16_check(None, None) == L.ERR_BAD_ARG

    assert native.b200_shuffle_b_bf16(0x1000, 0x2000, 24, 16, 1, None) == L.ERR_UNSUPPORTED
    assert native.b200_shuffle_b_bf16(0x1000, 0x2000, 16, 12, 1, None) == L.ERR_UNSUPPORTED
    assert native.b200_shuffle_b_bf16(None, 0x2000, 16, 16, 1, None) == L.ERR_BAD_ARG

    q = native.b200_quantize_act_bf16_1x128
    assert q(0x1000, 256, 0x2000, 256, 0x3000, 8, 8, 200, None) == L.ERR_UNSUPPORTED      # K % 128
    assert q(0x1000, 100, 0x2000, 256, 0x3000, 8, 8, 256, None) == L.ERR_BAD_ARG           # ldx < K
    assert q(0x1000, 256, 0x2000, 256, 0x3000, 4, 8, 256, None) == L.ERR_BAD_ARG           # stride_sfa < M
    assert q(0x1008, 256, 0x2000, 256, 0x3000, 8, 8, 256, None) == L.ERR_UNSUPPORTED      # 16-byte loads
    assert q(None, 256, 0x2000, 256, 0x3000, 8, 8, 256, None) == L.ERR_BAD_ARG
    assert native.b200_quantize_act_bf16_mx32(0x1000, 256, 0x2000, 256, 0x3000, 8, 200, None) == L.ERR_UNSUPPORTED

    assert native.b200_membw_read(0x1000, 20, 0x2000, None) == L.ERR_UNSUPPORTED          # bytes % 16
    assert native.b200_membw_copy(0x1000, None, 32, None) == L.ERR_BAD_ARG


def test_batch_ready_and_shared_b_validation(native):
    """B200_GEMM_BATCH_READY (slabs that are still arriving) and a B shared by all batches: 2-CTA tile kernels only."""
    from gcnasm_b200 import _lib as L

    tile = C.c_int32(0)
    chk = lambda a: native.b200_gemm_check(C.byref(a), C.byref(tile))
    bs = dict(scale_mode=L.SCALE_BLOCK, ptr_sfa=0x4000, ptr_sfb=0x5000, stride_sfa=2048, stride_sfb=64)
    big = dict(m=2048, n=7168, k=8192, batch=8, stride_a=8192, stride_b=8192, stride_c=7168,
               stride_a_batch=2048 * 8192 + 64 * 2048 * 4, stride_b_batch=0, stride_c_batch=2048 * 7168,
               stride_sfa_batch=(2048 * 8192 + 64 * 2048 * 4) // 4, stride_sfb_batch=0)
    pair_tiles = (L.TILE_PAIR_256x256, L.TILE_PAIR_256x224, L.TILE_PAIR_256x192, L.TILE_PAIR_256x128)
    # shared B without ready words
    assert chk(_args(**big, **bs)) == L.OK and tile.value in pair_tiles
    # ready words
    rdy = dict(flags=L.GEMM_BATCH_READY, ptr_batch_ready=0x6000, batch_epoch=3)
    assert chk(_args(**big, **bs, **rdy)) == L.OK and tile.value in pair_tiles
    assert chk(_args(**big, **bs, flags=L.GEMM_BATCH_READY)) == L.ERR_BAD_ARG                       # no ready words given
    assert chk(_args(**{**big, "m": 128}, **bs, **rdy)) == L.ERR_UNSUPPORTED                          # needs the pair tiles
    assert chk(_args(**big, **bs, **rdy, tile_hint=L.TILE_128x256)) == L.ERR_UNSUPPORTED
    assert chk(_args(**big, **bs, **rdy, tile_hint=L.TILE_PAIR_256x256)) == L.OK
    assert chk(_args(**big, **{**bs, "scale_mode": L.SCALE_MX}, **rdy)) == L.ERR_UNSUPPORTED
    assert chk(_args(**{**big, "stride_sfb_batch": 448}, **bs)) == L.ERR_BAD_ARG                      # B shared, SFB not
    # small shapes keep their single-CTA tiles when nothing asks for the pair kernels
    assert chk(_args(m=256, n=512, k=1024, batch=2)) == L.OK
    assert native.b200_flag_write(None, 1, None) == L.ERR_BAD_ARG
    assert native.b200_flag_write(0x1002, 1, None) == L.ERR_BAD_ARG


def test_host_entry_rejects_bad_arguments_before_touching_the_device(native):
    from gcnasm_b200 import _lib as L

    assert native.b200_gemm_a8w8_host(None, None) == L.ERR_BAD_ARG
    assert native.b200_gemm_a8w8_host(C.byref(_args(ptr_c=0)), None) == L.ERR_BAD_ARG
    assert native.b200_gemm_a8w8_host(C.byref(_args(flags=L.GEMM_BATCH_READY, ptr_batch_ready=0x100)), None) == L.ERR_UNSUPPORTED


class _FakeTensor:
    """Just enough of a tensor for the device check (no GPU needed)."""

    def __init__(self, index):
        import torch

        self.is_cuda = True
        self.device = torch.device("cuda", index)


def test_operands_must_share_the_current_device(monkeypatch):
    import torch

    from gcnasm_b200 import api

    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    assert api._same_device(_FakeTensor(0), None, _FakeTensor(0)) == torch.device("cuda", 0)
    with pytest.raises(ValueError, match="different devices"):
        api._same_device(_FakeTensor(0), _FakeTensor(1))
    with pytest.raises(ValueError, match="current device"):
        api._same_device(_FakeTensor(1), _FakeTensor(1))
    cpu = _FakeTensor(0)
    cpu.is_cuda = False
    with pytest.raises(ValueError, match="CUDA tensors"):
        api._same_device(cpu)
