"""GPU parity: a16w16 siblings (bf16 operands) -- GEMM within 1e-2*max|ref| of the oracle, bf16 shuffle bit-exact."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from test_gpu_gemm import DEV, assert_close

pytestmark = pytest.mark.gpu


def bf16_bits(O, shape, seed, tid, lo, hi):
    return O.f32_to_bf16_bits(O.fill_uniform(shape, seed, tid, lo, hi))


def to_dev(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).to(DEV).view(torch.bfloat16)


def from_dev(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("m,n,k,tile", [
    (256, 512, 256, 0),            # the reference's default shape
    (128, 128, 64, 1), (100, 200, 328, 1), (300, 520, 1032, 2), (512, 512, 512, 4), (700, 1000, 776, 4),
    (1, 16, 8, 0), (64, 256, 4096, 0), (2048, 2048, 2048, 0),
])
def test_gemm_a16w16_nt(api, O, m, n, k, tile):
    a = bf16_bits(O, (m, k), 41, 0, 0.0, 1.0)
    b = bf16_bits(O, (n, k), 41, 1, -0.5, 0.5)
    ref = O.gemm_ref_nt_bf16(a, b, out_bf16=False)
    got = api.gemm_a16w16(to_dev(a), to_dev(b), out_dtype=torch.float32, tile=tile)
    assert_close(O, got.cpu().numpy(), ref, f"a16w16 {m}x{n}x{k} tile {tile}")
    got16 = api.gemm_a16w16(to_dev(a), to_dev(b), tile=tile)                # bf16 out, what the reference writes
    assert_close(O, got16.float().cpu().numpy(), ref, "a16w16 bf16 out")
    assert api.last_status() == 0


def test_gemm_a16w16_golden(api, O):
    G = np.load(os.path.join(GOLDEN, "golden.npz"))
    got = api.gemm_a16w16(to_dev(G["bf_a"]), to_dev(G["bf_b"]), out_dtype=torch.float32)
    assert_close(O, got.cpu().numpy(), G["bf_c_f32"], "a16w16 golden")


def test_gemm_a16w16_batched_strided_scaled(api, O):
    batch, m, n, k = 3, 130, 272, 264
    a = bf16_bits(O, (batch, m, k + 24), 42, 0, -1.0, 1.0)          # padded rows: stride_a = k + 24
    b = bf16_bits(O, (batch, n, k), 42, 1, -1.0, 1.0)
    ta = to_dev(a)[:, :, :k]
    sa = torch.tensor([0.5], device=DEV)
    sb = torch.tensor([3.0], device=DEV)
    got = api.gemm_a16w16(ta, to_dev(b), sa, sb, out_dtype=torch.float32)
    for i in range(batch):
        ref = O.gemm_ref_nt_bf16(np.ascontiguousarray(a[i, :, :k]), b[i], out_bf16=False) * np.float32(1.5)
        assert_close(O, got[i].cpu().numpy(), ref, f"batch {i}")


@pytest.mark.parametrize("n,k", [(16, 8), (48, 64), (272, 1040), (1024, 512)])
def test_shuffle_b_bf16_bit_exact(api, O, n, k):
    w = (np.arange(k * n, dtype=np.uint64) * 2654435761 >> 9).astype(np.uint16).reshape(k, n)
    want = O.shuffle_b_bf16(w)
    f_kn = api.shuffle_b_bf16(to_dev(w), "kn")
    f_nk = api.shuffle_b_bf16(to_dev(np.ascontiguousarray(w.T)), "nk")
    assert np.array_equal(from_dev(f_kn), want) and np.array_equal(from_dev(f_nk), want)
    assert np.array_equal(from_dev(api.unshuffle_b_bf16(f_kn, n, k, "kn")), w)
    assert np.array_equal(from_dev(api.unshuffle_b_bf16(f_kn, n, k, "nk")), w.T)


def test_shuffle_b_bf16_golden(api):
    G = np.load(os.path.join(GOLDEN, "golden.npz"))
    assert np.array_equal(from_dev(api.shuffle_b_bf16(to_dev(G["bf_shuffle_in_kn"]), "kn")), G["bf_shuffle_out"])


@pytest.mark.parametrize("m,n,k,tile", [(256, 512, 256, 0), (40, 272, 192, 1), (600, 1024, 1024, 4), (300, 768, 512, 2)])
def test_flatmm_a16w16(api, O, m, n, k, tile):
    """B given as [K,N] (the reference's orientation), shuffled on the device, GEMM reads the flat image; the host
    reference reads the unshuffled matrix (flatmm_a16w16_gfx950.cc:571-582)."""
    a = bf16_bits(O, (m, k), 43, 0, 0.0, 1.0)
    b_kn = bf16_bits(O, (k, n), 43, 1, -0.5, 0.5)
    flat = api.shuffle_b_bf16(to_dev(b_kn), "kn")
    got = api.gemm_a16w16(to_dev(a), flat, n=n, flat=True, out_dtype=torch.float32, tile=tile)
    assert_close(O, got.cpu().numpy(), O.gemm_ref_kn_bf16(a, b_kn, out_bf16=False), f"flat a16w16 {m}x{n}x{k}")
    assert api.last_status() == 0


def test_a16w16_rejects(api):
    from gcnasm_b200 import B200Error

    a = torch.zeros(64, 36, dtype=torch.bfloat16, device=DEV)             # K % 8 != 0
    b = torch.zeros(64, 36, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(B200Error):
        api.gemm_a16w16(a, b)
    with pytest.raises(TypeError):
        api.gemm_a16w16(a.float(), b)
    with pytest.raises(B200Error):                                         # a tile that is not built for bf16
        api.gemm_a16w16(torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV),
                        torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV), tile=7)
