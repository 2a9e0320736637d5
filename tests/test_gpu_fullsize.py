"""GPU: the BASELINE configurations at full size.  The CPU oracle cannot finish these in seconds, so they are
checked (a) on sampled rows against the oracle, (b) on row slabs against the one-thread-per-output device
kernel (itself bit-identical to the oracle on small shapes), and (c) through size-independent properties:
run-to-run determinism, exact power-of-two scale linearity and shard/slice consistency."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from test_gpu_gemm import DEV, T, status_ok

pytestmark = pytest.mark.gpu


def _rows(m, count, seed):
    rng = np.random.default_rng(seed)
    return np.sort(rng.choice(m, count, replace=False))


@pytest.fixture(scope="module")
def config2(api, O):
    m, n, k = 4096, 7168, 2048
    xa = torch.from_numpy(api.fill_normal((m, k), 1234, 0)).to(DEV)
    xb = torch.from_numpy(api.fill_normal((n, k), 1234, 1)).to(DEV)
    qa, sfa = api.quantize_1x128(xa)
    qb, sfb = api.quantize_128x128(xb)
    return m, n, k, qa, qb, sfa, sfb


@pytest.mark.parametrize("tile", [2, 4, 7])
def test_config2_blockscale_full(api, O, config2, tile):
    m, n, k, qa, qb, sfa, sfb = config2
    c = api.gemm_a8w8_blockscale(qa, qb, sfa, sfb, out_dtype=torch.bfloat16, tile=tile)
    status_ok(api)
    # (a) sampled rows on the CPU oracle
    rows = _rows(m, 6, 2)
    ha, hb = qa.cpu().numpy(), qb.cpu().numpy()
    hsa, hsb = sfa.cpu().numpy(), sfb.cpu().numpy()
    for r in rows:
        ref = O.bf16_bits_to_f32(O.gemm_ref_blockscale(ha, hb, hsa, hsb, out_bf16=True, rows=(int(r), int(r) + 1)))
        assert_close(O, c[r:r + 1].float().cpu().numpy(), ref, f"row {r}")
    # (b) two 128-row slabs on the device checker
    for r0 in (0, 3968):
        ref = api.gemm_a8w8_blockscale(qa[r0:r0 + 128], qb, sfa[:, r0:r0 + 128].contiguous(), sfb,
                                       out_dtype=torch.bfloat16, simple=True)
        assert_close(O, c[r0:r0 + 128].float().cpu().numpy(), ref.float().cpu().numpy(), f"slab {r0}")
    # (c) determinism and N-shard consistency: computing a column shard alone gives the same bits
    c2 = api.gemm_a8w8_blockscale(qa, qb, sfa, sfb, out_dtype=torch.bfloat16, tile=tile)
    assert torch.equal(c, c2)
    shard = api.gemm_a8w8_blockscale(qa, qb[1792:3584], sfa, sfb[14:28].contiguous(), out_dtype=torch.bfloat16, tile=tile)
    assert torch.equal(shard, c[:, 1792:3584])


def test_config3_mxfp8_full(api, O):
    m = n = k = 8192
    xa = torch.from_numpy(api.fill_normal((m, k), 1234, 0)).to(DEV)
    xb = torch.from_numpy(api.fill_normal((n, k), 1234, 1)).to(DEV)
    qa, ea, sa = api.quantize_mx32(xa)
    qb, eb, sb = api.quantize_mx32(xb)
    del xa, xb
    c = api.gemm_a8w8_mx(qa, qb, sa, sb, out_dtype=torch.bfloat16)
    status_ok(api)
    hb, heb = qb.cpu().numpy(), eb.cpu().numpy()
    for r in _rows(m, 3, 3):
        ref = O.gemm_ref_mx(qa[r:r + 1].cpu().numpy(), hb, ea[r:r + 1].cpu().numpy(), heb)
        assert_close(O, c[r:r + 1].float().cpu().numpy(), O.bf16_bits_to_f32(O.f32_to_bf16_bits(ref)), f"row {r}")
    # a 128-row slab on the device checker (needs that slab's own scale atoms)
    r0 = 4096
    sa_slab = api.mx_sf_relayout(ea[r0:r0 + 128].contiguous(), 128, k)
    ref = api.gemm_a8w8_mx(qa[r0:r0 + 128], qb, sa_slab, sb, out_dtype=torch.float32, simple=True)
    assert_close(O, c[r0:r0 + 128].float().cpu().numpy(), ref.cpu().numpy(), "slab")
    assert torch.equal(c, api.gemm_a8w8_mx(qa, qb, sa, sb, out_dtype=torch.bfloat16))


def test_blockscale_8192_cube_sampled(api, O):
    """the shape the throughput target is quoted on"""
    m = n = k = 8192
    xa = torch.from_numpy(api.fill_normal((m, k), 7, 0)).to(DEV)
    xb = torch.from_numpy(api.fill_normal((n, k), 7, 1)).to(DEV)
    qa, sfa = api.quantize_1x128(xa)
    qb, sfb = api.quantize_128x128(xb)
    del xa, xb
    c = api.gemm_a8w8_blockscale(qa, qb, sfa, sfb, out_dtype=torch.bfloat16)
    status_ok(api)
    r0 = 8064
    ref = api.gemm_a8w8_blockscale(qa[r0:r0 + 128], qb, sfa[:, r0:r0 + 128].contiguous(), sfb, out_dtype=torch.float32, simple=True)
    assert_close(O, c[r0:r0 + 128].float().cpu().numpy(), ref.cpu().numpy(), "slab")
    ha, hb, hsa, hsb = qa.cpu().numpy(), qb.cpu().numpy(), sfa.cpu().numpy(), sfb.cpu().numpy()
    for r in _rows(m, 2, 5):
        ref = O.bf16_bits_to_f32(O.gemm_ref_blockscale(ha, hb, hsa, hsb, out_bf16=True, rows=(int(r), int(r) + 1)))
        assert_close(O, c[r:r + 1].float().cpu().numpy(), ref, f"row {r}")


def test_scale_linearity_exact(api, O):
    """power-of-two per-tensor scales only shift exponents: results scale exactly"""
    m, n, k = 512, 1024, 1024
    a = T(O.cast_e4m3(O.fill_uniform((m, k), 1, 0, 0.0, 1.0)))
    b = T(O.cast_e4m3(O.fill_uniform((n, k), 1, 1, -0.5, 0.5)))
    base = api.gemm_a8w8(a, b, out_dtype=torch.float32)
    s2 = api.gemm_a8w8(a, b, torch.tensor([4.0], device=DEV), torch.tensor([0.125], device=DEV), out_dtype=torch.float32)
    assert torch.equal(s2, base * 0.5)
    # block scales all equal to 1 reproduce the unscaled product bit for bit
    ones_a = torch.ones(k // 128, m, device=DEV)
    ones_b = torch.ones(n // 128, k // 128, device=DEV)
    bs = api.gemm_a8w8_blockscale(a, b, ones_a, ones_b, out_dtype=torch.float32)
    assert_close(O, bs.cpu().numpy(), base.cpu().numpy(), "unit block scales")
    status_ok(api)


def test_config5_activation_quantise_full(api, O):
    """Fused bf16 quantiser on config 5's activation matrix (16384 x 8192): sampled row blocks bit-exact against the
    oracle, and the size-independent properties -- every scale is its group's amax/448, the largest magnitude of every
    non-zero group encodes as +-448, the result does not change from run to run."""
    m, k = 16384, 8192
    x = torch.randn(m, k, device=DEV, dtype=torch.float32).mul_(2.0).to(torch.bfloat16)
    x[100:228, 1024:1152] = 0                                       # whole zero groups
    q, sfa = api.quantize_act_bf16_1x128(x)
    q2, sfa2 = api.quantize_act_bf16_1x128(x)
    assert torch.equal(q, q2) and torch.equal(sfa, sfa2)
    for r0 in (0, 96, 8000, 16352):
        bits = x[r0:r0 + 32].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        qr, sr = O.quant_1x128(O.bf16_bits_to_f32(bits))
        assert np.array_equal(q[r0:r0 + 32].cpu().numpy(), qr), f"rows {r0}"
        assert np.array_equal(sfa[:, r0:r0 + 32].cpu().numpy(), sr), f"scales of rows {r0}"
    amax = x.float().abs().view(m, k // 128, 128).amax(dim=2)                       # [M, K/128]
    # amax is exact; the division is done by numpy (IEEE fp32) -- torch's GPU division by a constant is not
    # correctly rounded and differs in the last bit for some values
    am = amax.cpu().numpy()
    want = np.where(am > 0, am / np.float32(448.0), np.float32(1.0)).astype(np.float32).T
    assert np.array_equal(sfa.cpu().numpy(), want)
    mag = (q.view(m, k // 128, 128) & 0x7F).amax(dim=2)                             # e4m3 magnitude bits
    assert torch.equal(mag[amax > 0], torch.full_like(mag[amax > 0], 0x7E))          # 448 = 0x7E
    assert int(mag[amax == 0].max()) == 0


def test_a16w16_large_sampled_rows(api, O):
    """bf16 sibling at 4096^3: sampled rows against the oracle, determinism, N-shard consistency."""
    m = n = k = 4096
    a = (torch.randn(m, k, device=DEV) * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, device=DEV) * 0.5).to(torch.bfloat16)
    c = api.gemm_a16w16(a, b, out_dtype=torch.float32)
    status_ok(api)
    hb = b.view(torch.int16).cpu().numpy().view(np.uint16)
    for r in _rows(m, 4, 5):
        ha = a[r:r + 1].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        assert_close(O, c[r:r + 1].cpu().numpy(), O.gemm_ref_nt_bf16(ha, hb, out_bf16=False), f"row {r}")
    assert torch.equal(c, api.gemm_a16w16(a, b, out_dtype=torch.float32))
    shard = api.gemm_a16w16(a, b[1024:2048], out_dtype=torch.float32)
    assert torch.equal(shard, c[:, 1024:2048])


def test_config5_per_rank_gemm_full(api, O):
    """BASELINE config 5 as one of 8 ranks runs it: M=16384, K=8192, a 7168-column weight shard, through the slab
    pipeline of the sharded operator (8 slabs of 2048 rows as batches of one launch, one B, ready words).  Sampled rows on
    the CPU oracle, two row blocks on the device checker, and the whole result bit-identical to the plain (unbatched)
    launch of the same problem and from run to run."""
    from gcnasm_b200.sharded import ColumnShardedGemm

    m, n, k = 16384, 7168, 8192
    qb, sfb = api.quantize_128x128(torch.from_numpy(api.fill_normal((n, k), 1234, 16)).to(DEV))
    qa, sfa = api.quantize_1x128(torch.from_numpy(api.fill_normal((m, k), 1234, 0)).to(DEV))
    op = ColumnShardedGemm(qb, sfb, n)
    plan = op.plan_slabs(m, k, DEV)
    assert (plan.slabs, plan.rows) == (8, 2048)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    op.step(0, out, a=qa, sfa=sfa)
    status_ok(api)
    hb, hsb = qb.cpu().numpy(), sfb.cpu().numpy()
    for r in _rows(m, 4, 9):
        ha = qa[r:r + 1].cpu().numpy()
        hsa = sfa[:, r:r + 1].contiguous().cpu().numpy()
        ref = O.bf16_bits_to_f32(O.gemm_ref_blockscale(ha, hb, hsa, hsb, out_bf16=True))
        assert_close(O, out[r:r + 1].float().cpu().numpy(), ref, f"row {r}")
    for row0 in (1920, 14336 + 512):
        err, ref = op.check_rows(0, out, row0, 128)
        assert err <= 1e-2 * ref, (row0, err, ref)
    plain = api.gemm_a8w8_blockscale(qa, qb, sfa, sfb, out_dtype=torch.bfloat16)
    assert torch.equal(plain, out)                       # the same tiles, the same order of additions
    out2 = torch.zeros_like(out)
    op.step(1, out2, a=qa, sfa=sfa)
    status_ok(api)
    assert torch.equal(out2, out)
