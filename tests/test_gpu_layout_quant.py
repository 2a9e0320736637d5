"""GPU parity, bit-exact: weight pre-shuffle (and inverse), quantisers and the MX scale re-layout."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from test_gpu_gemm import DEV, T, e4m3

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k", [(16, 16), (48, 64), (512, 256), (272, 1040), (1040, 272), (4096, 4096)])
def test_shuffle_b_bit_exact(api, O, n, k):
    b_kn = e4m3(O, (k, n), 9, 0, -400.0, 400.0)
    want = O.shuffle_b(b_kn)
    f_kn = api.shuffle_b(T(b_kn), "kn")
    f_nk = api.shuffle_b(T(np.ascontiguousarray(b_kn.T)), "nk")
    assert np.array_equal(f_kn.cpu().numpy(), want)
    assert np.array_equal(f_nk.cpu().numpy(), want)
    assert np.array_equal(api.unshuffle_b(f_kn, n, k, "kn").cpu().numpy(), b_kn)
    assert np.array_equal(api.unshuffle_b(f_kn, n, k, "nk").cpu().numpy(), b_kn.T)


def test_shuffle_b_golden(api):
    G = np.load(os.path.join(GOLDEN, "golden.npz"))
    assert np.array_equal(api.shuffle_b(T(G["shuffle_in_kn"]), "kn").cpu().numpy(), G["shuffle_out"])


def test_shuffle_b_full_decode_weight(api, O):
    n, k = 18432, 7168
    b = O.cast_e4m3(O.fill_uniform((n, k), 4, 0, -448.0, 448.0))
    f = api.shuffle_b(T(b), "nk")
    assert np.array_equal(f.cpu().numpy(), O.shuffle_b_nk(b))
    assert torch.equal(api.unshuffle_b(f, n, k, "nk"), T(b))


def test_shuffle_rejects_ragged(api):
    from gcnasm_b200 import B200Error

    with pytest.raises(B200Error):
        api.shuffle_b(torch.zeros(16, 24, dtype=torch.uint8, device=DEV), "kn")


def _x(O, shape, seed):
    x = O.fill_normal(shape, seed, 0) * 3.0
    x[3, :40] = 0.0
    if shape[0] >= 228 and shape[1] >= 256:
        x[100:228, 128:256] = 0.0
    return x


@pytest.mark.parametrize("shape", [(512, 1024), (8, 256), (130, 384)])
def test_quantisers_bit_exact(api, O, shape):
    x = _x(O, shape, 11)
    q, s = api.quantize_tensor(T(x))
    qr, sr = O.quant_tensor(x)
    assert np.array_equal(q.cpu().numpy(), qr) and s.item() == sr[0]
    q, s = api.quantize_1x128(T(x))
    qr, sr = O.quant_1x128(x)
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr)
    q, s, _ = api.quantize_mx32(T(x))
    qr, sr = O.quant_mx32(x)
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr)
    assert np.array_equal(api.cast_e4m3(T(x * 100)).cpu().numpy(), O.cast_e4m3(x * 100))
    if shape[0] % 128 == 0:
        q, s = api.quantize_128x128(T(x))
        qr, sr = O.quant_128x128(x)
        assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr)


def test_quantisers_golden(api):
    G = np.load(os.path.join(GOLDEN, "golden.npz"))
    x = T(G["q_in"])
    q, s = api.quantize_tensor(x)
    assert np.array_equal(q.cpu().numpy(), G["q_tensor_q"]) and s.item() == G["q_tensor_scale"][0]
    q, s = api.quantize_1x128(x)
    assert np.array_equal(q.cpu().numpy(), G["q_1x128_q"]) and np.array_equal(s.cpu().numpy(), G["q_1x128_sfa"])
    q, s, _ = api.quantize_mx32(x)
    assert np.array_equal(q.cpu().numpy(), G["q_mx_q"]) and np.array_equal(s.cpu().numpy(), G["q_mx_sf"])


def test_quantiser_extremes(api, O):
    x = np.zeros((4, 128), np.float32)
    x[1, 5] = 1e-30
    x[2, :] = 3e38
    x[3, 7] = -2.0 ** -140           # float subnormal
    q, s = api.quantize_1x128(T(x))
    qr, sr = O.quant_1x128(x)
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr)
    q, s, _ = api.quantize_mx32(T(x))
    qr, sr = O.quant_mx32(x)
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr)


def test_mx_sf_relayout_atoms(api):
    rows, k = 200, 384
    sf = np.arange(rows * (k // 32), dtype=np.uint32).astype(np.uint8).reshape(rows, k // 32)
    sf[sf == 255] = 0
    atoms = api.mx_sf_relayout(T(sf), rows, k).cpu().numpy().reshape(k // 128, 2, 32, 4, 4)
    for r in (0, 1, 31, 32, 100, 127, 128, 199):
        for kb in range(k // 32):
            assert atoms[kb // 4, r // 128, r % 32, (r % 128) // 32, kb % 4] == sf[r, kb]
    assert atoms[0, 1, 8, 2, 0] == 127        # row 128 + 72 = 200 is padding -> scale 1.0
