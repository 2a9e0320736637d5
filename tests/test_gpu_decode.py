"""GPU parity: the skinny-M weight-streaming kernel (row-major and pre-shuffled weights, block scales, K splits)."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from test_gpu_gemm import DEV, T, e4m3, status_ok

pytestmark = pytest.mark.gpu
DECODE = 3


@pytest.mark.parametrize("m,n,k", [(1, 1024, 1024), (16, 256, 512), (33, 272, 640), (64, 384, 2048), (8, 512, 8192), (64, 16, 128)])
def test_decode_rowmajor_unscaled(api, O, m, n, k):
    a = e4m3(O, (m, k), 1, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 1, 1, -0.5, 0.5)
    c = api.gemm_a8w8(T(a), T(b), out_dtype=torch.float32, tile=DECODE)
    status_ok(api)
    ref = O.gemm_ref_nt(a, b)
    assert_close(O, c.cpu().numpy(), ref, "decode nk")
    assert O.valid_vector(ref, c.cpu().numpy(), 0.1)


@pytest.mark.parametrize("m,n,k", [(1, 512, 1024), (16, 256, 512), (64, 1024, 1024), (40, 144, 256)])
def test_decode_flat_unscaled(api, O, m, n, k):
    a = e4m3(O, (m, k), 3, 0, 0.0, 1.0)
    b_kn = e4m3(O, (k, n), 3, 1, -0.5, 0.5)
    c = api.flatmm_a8w8(T(a), api.shuffle_b(T(b_kn), "kn"), n, out_dtype=torch.float32, tile=DECODE)
    status_ok(api)
    assert_close(O, c.cpu().numpy(), O.gemm_ref_kn(a, b_kn), "decode flat")


@pytest.mark.parametrize("flat", [False, True])
@pytest.mark.parametrize("m,n,k", [(1, 512, 1024), (16, 256, 512), (16, 1024, 4096), (64, 2304, 1792), (50, 128, 128)])
def test_decode_blockscale(api, O, m, n, k, flat):
    a = e4m3(O, (m, k), 2, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 2, 1, -0.5, 0.5)
    sfa = O.fill_uniform((k // 128, m), 2, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 2, 3, 0.8, 1.2)
    if flat:
        c = api.gemm_a8w8_blockscale(T(a), api.shuffle_b(T(b), "nk"), T(sfa), T(sfb), out_dtype=torch.float32, b_flat_n=n)
    else:
        c = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=torch.float32)
    status_ok(api)
    assert_close(O, c.cpu().numpy(), O.gemm_ref_blockscale(a, b, sfa, sfb), "decode block")


@pytest.mark.parametrize("m", [1, 16, 64])
def test_decode_config4_full_size(api, O, m):
    """BASELINE config 4 in full: N=18432, K=7168, pre-shuffled weights, U[-1,1] data quantised with
    1x128 / 128x128 amax/448 scales, bf16 output; checked against the oracle on every element."""
    n, k = 18432, 7168
    xa = O.fill_uniform((m, k), 1234, 0, -1.0, 1.0)
    xb = O.fill_uniform((n, k), 1234, 1, -1.0, 1.0)
    qa, sfa = O.quant_1x128(xa)
    qb, sfb = O.quant_128x128(xb)
    flat = api.shuffle_b(T(qb), "nk")
    assert np.array_equal(flat.cpu().numpy(), O.shuffle_b_nk(qb))
    c = api.gemm_a8w8_blockscale(T(qa), flat, T(sfa), T(sfb), out_dtype=torch.bfloat16, b_flat_n=n)
    status_ok(api)
    ref = O.bf16_bits_to_f32(O.gemm_ref_blockscale(qa, qb, sfa, sfb, out_bf16=True))
    assert_close(O, c.float().cpu().numpy(), ref, f"config 4 M={m}")
    # same weights row-major: identical arithmetic, bit-identical result
    c2 = api.gemm_a8w8_blockscale(T(qa), T(qb), T(sfa), T(sfb), out_dtype=torch.bfloat16)
    assert torch.equal(c, c2)


def test_decode_batched_and_scaled(api, O):
    B, m, n, k = 2, 16, 256, 512
    a = e4m3(O, (B, m, k), 5, 0, 0.0, 1.0)
    b = e4m3(O, (B, n, k), 5, 1, -0.5, 0.5)
    sa = torch.tensor([0.25], device=DEV)
    sb = torch.tensor([3.0], device=DEV)
    c = api.gemm_a8w8(T(a), T(b), sa, sb, out_dtype=torch.bfloat16, tile=DECODE).float().cpu().numpy()
    status_ok(api)
    for i in range(B):
        assert_close(O, c[i], O.gemm_ref_nt(a[i], b[i], 0.25, 3.0), f"batch {i}")
