"""GPU parity, bit-exact: fused activation quantisers (bf16 in, e4m3 + scales in the GEMM's layout out).

The oracle quantises fp32; a bf16 value converts to fp32 exactly, so the expected result is the oracle run on the
widened input."""
import numpy as np
import pytest
import torch

from test_gpu_gemm import DEV, T, assert_close

pytestmark = pytest.mark.gpu


def _bf16_input(O, shape, seed, scale=3.0):
    """(torch bf16 tensor on the device, the same values as fp32 numpy)"""
    x = O.fill_normal(shape, seed, 0) * scale
    x[min(3, shape[0] - 1), :40] = 0.0
    if shape[0] >= 228 and shape[1] >= 256:
        x[100:228, 128:256] = 0.0                    # whole zero groups -> scale 1.0, zero bytes
    bits = O.f32_to_bf16_bits(x)
    xb = torch.from_numpy(bits.view(np.int16)).to(DEV).view(torch.bfloat16)
    return xb, O.bf16_bits_to_f32(bits)


@pytest.mark.parametrize("shape", [(512, 1024), (1, 128), (31, 256), (33, 1152), (130, 384), (4096, 2048)])
def test_act_quant_1x128_bit_exact(api, O, shape):
    xb, xf = _bf16_input(O, shape, 21)
    q, sfa = api.quantize_act_bf16_1x128(xb)
    qr, sr = O.quant_1x128(xf)
    assert np.array_equal(q.cpu().numpy(), qr)
    assert np.array_equal(sfa.cpu().numpy(), sr)


def test_act_quant_1x128_matches_fp32_quantiser(api, O):
    xb, xf = _bf16_input(O, (256, 512), 22)
    q, sfa = api.quantize_act_bf16_1x128(xb)
    q2, sfa2 = api.quantize_1x128(T(xf))
    assert torch.equal(q, q2) and torch.equal(sfa, sfa2)


def test_act_quant_1x128_strided_into_broadcast_buffer(api, O):
    """Input rows taken from a wider activation matrix; outputs written into one flat buffer [A bytes | SFA floats],
    the form the sharded path broadcasts."""
    m, k, wide = 96, 384, 640
    xb_w, xf_w = _bf16_input(O, (m, wide), 23)
    xb = xb_w[:, 128:128 + k]
    xf = np.ascontiguousarray(xf_w[:, 128:128 + k])
    buf = torch.zeros(m * k + 4 * (k // 128) * m, dtype=torch.uint8, device=DEV)
    q = buf[:m * k].view(m, k)
    sfa = buf[m * k:].view(torch.float32).view(k // 128, m)
    api.quantize_act_bf16_1x128(xb, q=q, sfa=sfa)
    qr, sr = O.quant_1x128(xf)
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(sfa.cpu().numpy(), sr)


def test_act_quant_1x128_extremes(api, O):
    x = np.zeros((4, 256), np.float32)
    x[1, 5] = 1e-30
    x[2, :] = 3e38
    x[3, 7] = -2.0 ** -130                           # bf16 subnormal
    x[3, 200] = 448.0
    bits = O.f32_to_bf16_bits(x)
    xb = torch.from_numpy(bits.view(np.int16)).to(DEV).view(torch.bfloat16)
    q, sfa = api.quantize_act_bf16_1x128(xb)
    qr, sr = O.quant_1x128(O.bf16_bits_to_f32(bits))
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(sfa.cpu().numpy(), sr)


def test_act_quant_1x128_wide_dynamic_range(api, O):
    """Row r is scaled by 2^e(r), e from -125 to 120: group scales inside and outside the range where the kernel
    replaces the IEEE division by reciprocal + FMA correction; every byte must still match the divided oracle."""
    m, k = 2048, 512
    x = O.fill_normal((m, k), 27, 0)
    e = np.linspace(-125, 120, m).astype(np.int32)
    x = np.ldexp(x, e[:, None]).astype(np.float32)
    bits = O.f32_to_bf16_bits(x)
    xb = torch.from_numpy(bits.view(np.int16)).to(DEV).view(torch.bfloat16)
    q, sfa = api.quantize_act_bf16_1x128(xb)
    qr, sr = O.quant_1x128(O.bf16_bits_to_f32(bits))
    assert np.array_equal(sfa.cpu().numpy(), sr)
    assert np.array_equal(q.cpu().numpy(), qr)


@pytest.mark.parametrize("shape", [(256, 512), (200, 384), (1, 128), (129, 256), (2048, 1024)])
def test_act_quant_mx32_bit_exact(api, O, shape):
    xb, xf = _bf16_input(O, shape, 24)
    q, atoms = api.quantize_act_bf16_mx32(xb)
    qr, sr = O.quant_mx32(xf)
    assert np.array_equal(q.cpu().numpy(), qr)
    want_atoms = api.mx_sf_relayout(T(sr), shape[0], shape[1])     # the re-layout itself is pinned by its own test
    assert torch.equal(atoms, want_atoms)


def test_act_quant_rejects_bad_arguments(api):
    from gcnasm_b200 import B200Error

    with pytest.raises(B200Error):
        api.quantize_act_bf16_1x128(torch.zeros(8, 192, dtype=torch.bfloat16, device=DEV))       # K % 128 != 0
    with pytest.raises(ValueError):
        api.quantize_act_bf16_1x128(torch.zeros(8, 128, dtype=torch.float32, device=DEV))
    with pytest.raises(B200Error):
        api.quantize_act_bf16_1x128(torch.zeros(8, 130, dtype=torch.bfloat16, device=DEV)[:, 1:129])  # misaligned rows


def test_act_quant_feeds_blockscale_gemm(api, O):
    """bf16 activations -> fused quantiser -> block-scale GEMM, against the oracle on the same quantised operands."""
    m, n, k = 384, 512, 1024
    xb, xf = _bf16_input(O, (m, k), 25, scale=1.0)
    w = O.fill_normal((n, k), 26, 1)
    qb, sfb = O.quant_128x128(w)
    qa, sfa = api.quantize_act_bf16_1x128(xb)
    out = api.gemm_a8w8_blockscale(qa, T(qb), sfa, T(sfb), out_dtype=torch.bfloat16)
    ref = O.gemm_ref_blockscale(qa.cpu().numpy(), qb, sfa.cpu().numpy(), sfb)
    assert_close(O, out.float().cpu().numpy(), ref)


def test_sharded_forward_bf16_single_gpu(api, O):
    """The sharded operator's bf16 entry on one GPU (world 1): fused quantise into the broadcast buffer, GEMM on
    its views."""
    from gcnasm_b200.sharded import ColumnShardedGemm

    m, n, k = 256, 384, 512
    xb, xf = _bf16_input(O, (m, k), 28, scale=1.0)
    qb, sfb = O.quant_128x128(O.fill_normal((n, k), 29, 1))
    op = ColumnShardedGemm(T(qb), T(sfb), n)
    out = op.forward_bf16(xb, m, k, DEV)
    qa, sfa = O.quant_1x128(xf)
    _, va, vs = op.activation_buffer(m, k, DEV)
    assert np.array_equal(va.cpu().numpy(), qa) and np.array_equal(vs.cpu().numpy(), sfa)
    assert_close(O, out.float().cpu().numpy(), O.gemm_ref_blockscale(qa, qb, sfa, sfb))
