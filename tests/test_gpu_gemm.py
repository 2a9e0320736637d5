"""GPU parity: the tcgen05 GEMM kernels through the C ABI against the oracle on the same seeded inputs.
Tolerance is the benchmark's: max|err| <= 1e-2 * max|ref| (fp32 accumulation); most cases are far inside it."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def T(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def e4m3(O, shape, seed, tid, lo, hi):
    return O.cast_e4m3(O.fill_uniform(shape, seed, tid, lo, hi))


def status_ok(api):
    torch.cuda.synchronize()
    assert api.last_status() == 0, "a bounded device wait expired"


# reference default shape (256x512x256), BASELINE config 1 (256x512x1024), tile edges, K not a multiple of 128
NT_SHAPES = [(256, 512, 256), (256, 512, 1024), (128, 128, 128), (200, 136, 144), (129, 72, 1040), (1024, 2048, 2048),
             (65, 16, 16), (300, 400, 272)]


@pytest.mark.parametrize("tile", [1, 2, 4, 6, 7, 8])
@pytest.mark.parametrize("m,n,k", NT_SHAPES)
def test_nt_unscaled_fp32(api, O, m, n, k, tile):
    a = e4m3(O, (m, k), 1, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 1, 1, -0.5, 0.5)
    c = api.gemm_a8w8(T(a), T(b), out_dtype=torch.float32, tile=tile)
    status_ok(api)
    ref = O.gemm_ref_nt(a, b)
    got = c.cpu().numpy()
    assert_close(O, got, ref, f"nt {m}x{n}x{k} tile {tile}")
    assert O.valid_vector(ref, got, 0.1)                 # the reference's own criterion (gemm_a8w8_8wave.cc:757)


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (129, 72, 1040)])
def test_nt_per_tensor_scale_bf16(api, O, m, n, k):
    """BASELINE config 1: U[-1,1] data, per-tensor amax/448 quantisation, bf16 output."""
    xa = O.fill_uniform((m, k), 1234, 0, -1.0, 1.0)
    xb = O.fill_uniform((n, k), 1234, 1, -1.0, 1.0)
    qa, sa = O.quant_tensor(xa)
    qb, sb = O.quant_tensor(xb)
    c = api.gemm_a8w8(T(qa), T(qb), T(sa), T(sb), out_dtype=torch.bfloat16)
    status_ok(api)
    ref = O.bf16_bits_to_f32(O.gemm_ref_nt(qa, qb, sa[0], sb[0], out_bf16=True))
    assert_close(O, c.float().cpu().numpy(), ref, "per-tensor bf16")
    # and against the unquantised fp32 product: quantisation noise only
    full = xa.astype(np.float64) @ xb.astype(np.float64).T
    assert np.max(np.abs(c.float().cpu().numpy() - full)) <= 0.05 * np.max(np.abs(full))


def test_nt_batched(api, O):
    """batch > 1 with the reference's strides (gemm_a8w8_8wave.cc:725-727), default problem of the reference."""
    B, m, n, k = 8, 256, 512, 256
    a = e4m3(O, (B, m, k), 5, 0, 0.0, 1.0)
    b = e4m3(O, (B, n, k), 5, 1, -0.5, 0.5)
    for tile in (1, 2, 4, 7):
        c = api.gemm_a8w8(T(a), T(b), out_dtype=torch.float32, tile=tile).cpu().numpy()
        status_ok(api)
        for i in range(B):
            assert_close(O, c[i], O.gemm_ref_nt(a[i], b[i]), f"batch {i}")


def test_nt_strided_views(api, O):
    """row pitch larger than K and an output with a row pitch larger than N."""
    m, n, k = 192, 160, 256
    a_full = e4m3(O, (m, 384), 6, 0, 0.0, 1.0)
    b_full = e4m3(O, (n, 512), 6, 1, -0.5, 0.5)
    ta, tb = T(a_full)[:, :k], T(b_full)[:, 128:128 + k]
    out = torch.zeros(m, 256, dtype=torch.float32, device=DEV)
    api.gemm_a8w8(ta, tb, out=out[:, :n])
    status_ok(api)
    ref = O.gemm_ref_nt(np.ascontiguousarray(a_full[:, :k]), np.ascontiguousarray(b_full[:, 128:128 + k]))
    assert_close(O, out[:, :n].cpu().numpy(), ref, "strided")
    assert torch.all(out[:, n:] == 0)                     # nothing written outside the N columns


BS_SHAPES = [(128, 128, 256, 1), (256, 512, 1024, 1), (128, 256, 256, 2), (384, 640, 1024, 2), (77, 384, 512, 2),
             (2048, 4096, 1024, 2), (130, 128, 128, 1),
             # CTA-pair tiles: 256x256, 256x128, 256x224 (tiles straddle the 128-column scale blocks), 256x192
             (256, 256, 256, 4), (512, 768, 1024, 4), (300, 640, 512, 4), (2048, 4096, 1024, 4), (77, 384, 512, 4),
             (512, 768, 1024, 6), (512, 896, 1024, 7), (300, 640, 512, 7), (2048, 3584, 1024, 7), (512, 768, 1024, 8),
             (1000, 1152, 384, 8), (4096, 7168, 256, 0)]


@pytest.mark.parametrize("m,n,k,tile", BS_SHAPES)
def test_blockscale_reference_inputs(api, O, m, n, k, tile):
    """The reference's own inputs: A~U[0,1), B~U[-.5,.5), scales U[.8,1.2] (gemm_a8w8_blockscale_host.cc:207-210)
    and its own criterion, abs diff <= 1e-3 on fp32 output (:274) -- relaxed to 2e-3 at K >= 1024 where the
    order of fp32 additions differs -- plus the relative bound."""
    a = e4m3(O, (m, k), 2, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 2, 1, -0.5, 0.5)
    sfa = O.fill_uniform((k // 128, m), 2, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 2, 3, 0.8, 1.2)
    c = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=torch.float32, tile=tile)
    status_ok(api)
    ref = O.gemm_ref_blockscale(a, b, sfa, sfb)
    got = c.cpu().numpy()
    assert_close(O, got, ref, f"block {m}x{n}x{k}")
    assert O.valid_vector(ref, got, 1e-3 if k < 1024 else 2e-3)


def test_blockscale_quantised_normal_bf16(api, O):
    """BASELINE config 2 recipe at a CPU-checkable size: N(0,1) data, 1x128 / 128x128 amax/448 scales, bf16 out."""
    m, n, k = 512, 768, 2048
    xa = O.fill_normal((m, k), 1234, 0)
    xb = O.fill_normal((n, k), 1234, 1)
    qa, sfa = O.quant_1x128(xa)
    qb, sfb = O.quant_128x128(xb)
    ref = O.bf16_bits_to_f32(O.gemm_ref_blockscale(qa, qb, sfa, sfb, out_bf16=True))
    for tile in (1, 2, 4, 6, 7, 8):
        c = api.gemm_a8w8_blockscale(T(qa), T(qb), T(sfa), T(sfb), out_dtype=torch.bfloat16, tile=tile)
        status_ok(api)
        assert_close(O, c.float().cpu().numpy(), ref, f"config-2 recipe tile {tile}")
    full = xa.astype(np.float64) @ xb.astype(np.float64).T
    assert np.max(np.abs(c.float().cpu().numpy() - full)) <= 0.05 * np.max(np.abs(full))


def test_blockscale_batched(api, O):
    B, m, n, k = 3, 160, 256, 384
    a = e4m3(O, (B, m, k), 8, 0, 0.0, 1.0)
    b = e4m3(O, (B, n, k), 8, 1, -0.5, 0.5)
    sfa = O.fill_uniform((B, k // 128, m), 8, 2, 0.8, 1.2)
    sfb = O.fill_uniform((B, n // 128, k // 128), 8, 3, 0.8, 1.2)
    c = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=torch.float32).cpu().numpy()
    status_ok(api)
    for i in range(B):
        assert_close(O, c[i], O.gemm_ref_blockscale(a[i], b[i], sfa[i], sfb[i]), f"batch {i}")


@pytest.mark.parametrize("m,n,k,tile", [(256, 512, 256, 1), (200, 272, 384, 2), (256, 512, 256, 2), (96, 1024, 1024, 0),
                                        (256, 512, 256, 4), (300, 672, 384, 7), (512, 384, 256, 8), (256, 512, 256, 6)])
def test_flatmm_reference_semantics(api, O, m, n, k, tile):
    """flatmm_a8w8: B created as [K,N], shuffled, host check on the unshuffled matrix, threshold 0.1
    (opus_fmm/flatmm_a8w8_gfx950.cc:732-742,586-597,798)."""
    a = e4m3(O, (m, k), 3, 0, 0.0, 1.0)
    b_kn = e4m3(O, (k, n), 3, 1, -0.5, 0.5)
    flat = api.shuffle_b(T(b_kn), "kn")
    assert np.array_equal(flat.cpu().numpy(), O.shuffle_b(b_kn))
    c = api.flatmm_a8w8(T(a), flat, n, out_dtype=torch.float32, tile=tile)
    status_ok(api)
    ref = O.gemm_ref_kn(a, b_kn)
    assert_close(O, c.cpu().numpy(), ref, "flatmm")
    assert O.valid_vector(ref, c.cpu().numpy(), 0.1)


def test_flatmm_batched_default_problem(api, O):
    B, m, n, k = 8, 256, 512, 256                           # the reference's default run (:704-707)
    a = e4m3(O, (B, m, k), 4, 0, 0.0, 1.0)
    b_kn = e4m3(O, (B, k, n), 4, 1, -0.5, 0.5)
    flat = torch.stack([api.shuffle_b(T(b_kn[i]), "kn") for i in range(B)])
    c = api.flatmm_a8w8(T(a), flat, n, out_dtype=torch.float32).cpu().numpy()
    status_ok(api)
    for i in range(B):
        assert_close(O, c[i], O.gemm_ref_kn(a[i], b_kn[i]), f"batch {i}")


def test_flat_blockscale(api, O):
    m, n, k = 256, 512, 512
    a = e4m3(O, (m, k), 9, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 9, 1, -0.5, 0.5)
    sfa = O.fill_uniform((k // 128, m), 9, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 9, 3, 0.8, 1.2)
    flat = api.shuffle_b(T(b), "nk")
    for tile in (1, 2, 4, 7):
        c = api.gemm_a8w8_blockscale(T(a), flat, T(sfa), T(sfb), out_dtype=torch.float32, tile=tile, b_flat_n=n)
        status_ok(api)
        assert_close(O, c.cpu().numpy(), O.gemm_ref_blockscale(a, b, sfa, sfb), "flat block")


@pytest.mark.parametrize("m,n,k", [(256, 384, 512), (128, 128, 128), (200, 72, 256), (1024, 1024, 2048)])
def test_mxfp8(api, O, m, n, k):
    """BASELINE config 3 recipe at CPU-checkable sizes: N(0,1) data, E8M0 per 1x32, e = floor(log2 amax) - 8."""
    xa = O.fill_normal((m, k), 1234, 0)
    xb = O.fill_normal((n, k), 1234, 1)
    qa, ea = O.quant_mx32(xa)
    qb, eb = O.quant_mx32(xb)
    sa = api.mx_sf_relayout(T(ea), m, k)
    sb = api.mx_sf_relayout(T(eb), n, k)
    ref = O.gemm_ref_mx(qa, qb, ea, eb)
    for tile in (1, 4, 0):
        c = api.gemm_a8w8_mx(T(qa), T(qb), sa, sb, out_dtype=torch.float32, tile=tile)
        status_ok(api)
        assert_close(O, c.cpu().numpy(), ref, f"mx tile {tile}")
    cb = api.gemm_a8w8_mx(T(qa), T(qb), sa, sb, out_dtype=torch.bfloat16)
    status_ok(api)
    assert_close(O, cb.float().cpu().numpy(), O.bf16_bits_to_f32(O.f32_to_bf16_bits(ref)), "mx bf16")
    full = xa.astype(np.float64) @ xb.astype(np.float64).T
    assert np.max(np.abs(c.cpu().numpy() - full)) <= 0.05 * np.max(np.abs(full))


def test_mx_wide_exponent_range(api, O):
    """block exponents spread over many binades, including all-zero blocks (E8M0 byte 0)."""
    m, n, k = 128, 128, 512
    xa = O.fill_normal((m, k), 77, 0) * np.exp2(np.floor(O.fill_uniform((m, k // 32), 77, 2, -20, 20))).repeat(32, axis=1)
    xb = O.fill_normal((n, k), 77, 1) * np.exp2(np.floor(O.fill_uniform((n, k // 32), 77, 3, -20, 20))).repeat(32, axis=1)
    xa[5, 64:128] = 0.0
    xb[9, :32] = 0.0
    qa, ea = O.quant_mx32(xa.astype(np.float32))
    qb, eb = O.quant_mx32(xb.astype(np.float32))
    c = api.gemm_a8w8_mx(T(qa), T(qb), api.mx_sf_relayout(T(ea), m, k), api.mx_sf_relayout(T(eb), n, k),
                         out_dtype=torch.float32)
    status_ok(api)
    assert_close(O, c.cpu().numpy(), O.gemm_ref_mx(qa, qb, ea, eb), "mx wide")


def test_simple_kernel_matches_oracle_bitwise(api, O):
    """the one-thread-per-output checker kernel mirrors the host loops operation for operation."""
    a = e4m3(O, (64, 256), 2, 0, 0.0, 1.0)
    b = e4m3(O, (256, 256), 2, 1, -0.5, 0.5)
    sfa = O.fill_uniform((2, 64), 2, 2, 0.8, 1.2)
    sfb = O.fill_uniform((2, 2), 2, 3, 0.8, 1.2)
    c = api.gemm_a8w8(T(a), T(b), out_dtype=torch.float32, simple=True).cpu().numpy()
    assert np.array_equal(c, O.gemm_ref_nt(a, b))
    c = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=torch.float32, simple=True).cpu().numpy()
    assert np.array_equal(c, O.gemm_ref_blockscale(a, b, sfa, sfb))


def test_golden_fixtures_through_cuda(api, O):
    G = np.load(os.path.join(GOLDEN, "golden.npz"))
    c = api.gemm_a8w8(T(G["nt_a"]), T(G["nt_b"]), out_dtype=torch.float32, tile=1)
    assert_close(O, c.cpu().numpy(), G["nt_c"], "golden nt")
    c = api.gemm_a8w8_blockscale(T(G["bs_a"]), T(G["bs_b"]), T(G["bs_sfa"]), T(G["bs_sfb"]), out_dtype=torch.float32)
    assert_close(O, c.cpu().numpy(), G["bs_c"], "golden block")
    m, k = G["mx_a"].shape
    n = G["mx_b"].shape[0]
    c = api.gemm_a8w8_mx(T(G["mx_a"]), T(G["mx_b"]), api.mx_sf_relayout(T(G["mx_sfa"]), m, k),
                         api.mx_sf_relayout(T(G["mx_sfb"]), n, k), out_dtype=torch.float32, tile=1)
    assert_close(O, c.cpu().numpy(), G["mx_c"], "golden mx")
    status_ok(api)


def test_error_behaviour_on_device(api, O):
    from gcnasm_b200 import B200Error

    a = T(e4m3(O, (128, 128), 1, 0, 0, 1))
    b = T(e4m3(O, (100, 128), 1, 1, 0, 1))
    with pytest.raises(B200Error) as ei:                    # K = 24 is not a multiple of 16: TMA row pitch
        api.gemm_a8w8(T(e4m3(O, (128, 24), 1, 0, 0, 1)), T(e4m3(O, (100, 24), 1, 1, 0, 1)))
    assert ei.value.code == -2
    with pytest.raises(B200Error):                          # flat layout needs K % 128 == 0
        api.flatmm_a8w8(T(e4m3(O, (128, 64), 1, 0, 0, 1)), T(e4m3(O, (64 * 128,), 1, 1, 0, 1)), 128)
    with pytest.raises(TypeError):
        api.gemm_a8w8(a.float(), b)
    with pytest.raises(ValueError):
        api.gemm_a8w8(a, T(e4m3(O, (128, 256), 1, 1, 0, 1)))


def test_host_buffer_entry_point(api, O):
    """b200_gemm_a8w8_host: copy-in, launch, copy-out; bit-identical to the device-resident path."""
    from gcnasm_b200 import _lib as L

    m, n, k = 256, 512, 1024
    a = e4m3(O, (m, k), 11, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 11, 1, -0.5, 0.5)
    sfa = O.fill_uniform((k // 128, m), 11, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 11, 3, 0.8, 1.2)
    c = np.zeros((m, n), np.float32)
    api.gemm_a8w8_host(a, b, c, sfa=sfa, sfb=sfb, scale_mode=L.SCALE_BLOCK)
    dev = api.gemm_a8w8_blockscale(T(a), T(b), T(sfa), T(sfb), out_dtype=torch.float32).cpu().numpy()
    assert np.array_equal(c, dev)
    assert_close(O, c, O.gemm_ref_blockscale(a, b, sfa, sfb), "host entry")
    c2 = np.zeros((m, n), np.uint16)
    api.gemm_a8w8_host(a, b, c2, scale_a=np.array([0.5], np.float32), scale_b=np.array([3.0], np.float32),
                       scale_mode=L.SCALE_TENSOR)
    assert_close(O, O.bf16_bits_to_f32(c2), O.gemm_ref_nt(a, b, 0.5, 3.0), "host entry tensor")


@pytest.mark.parametrize("m", [2048, 2300, 4096])
def test_host_buffer_entry_point_row_slabs(api, O, m):
    """Large M: the host entry runs row slabs with the copy-back on a second stream.  Every row of C must arrive and
    equal the device-resident result bit for bit (same kernels, same tiles within a slab boundary of 256 rows)."""
    from gcnasm_b200 import _lib as L

    n, k = 640, 512
    a = e4m3(O, (m, k), 12, 0, 0.0, 1.0)
    b = e4m3(O, (n, k), 12, 1, -0.5, 0.5)
    sfa = O.fill_uniform((k // 128, m), 12, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 12, 3, 0.8, 1.2)
    c = np.full((m, n), 0xFFFF, np.uint16)                           # poison: a missed slab would keep NaN bits
    for _ in range(2):                                               # second call reuses streams, events and buffers
        c[:] = 0xFFFF
        api.gemm_a8w8_host(a, b, c, sfa=sfa, sfb=sfb, scale_mode=L.SCALE_BLOCK)
        got = O.bf16_bits_to_f32(c)
        assert not np.isnan(got).any()
        rows = slice(0, m, 37)
        ref = O.gemm_ref_blockscale(a, b, sfa, sfb)
        assert_close(O, got[rows], ref[rows], f"host slabs m={m}")
        assert_close(O, got[-64:], ref[-64:], "last rows")
    cu = np.zeros((m, n), np.float32)
    api.gemm_a8w8_host(a, b, cu)                                     # unscaled, fp32 out
    assert_close(O, cu[::53], O.gemm_ref_nt(a, b)[::53], "host slabs unscaled")


def test_chained_launches_with_inputs_ready(api, O):
    """B200_GEMM_INPUTS_READY lets a launch start before its predecessor has finished.  Results must not change, and
    two launches that write the same C must still land in order."""
    m, n, k = 1024, 1792, 1024
    sets = []
    for j in range(3):
        a, b = e4m3(O, (m, k), 20 + j, 0, 0.0, 1.0), e4m3(O, (n, k), 20 + j, 1, -0.5, 0.5)
        sfa = O.fill_uniform((k // 128, m), 20 + j, 2, 0.8, 1.2)
        sfb = O.fill_uniform((n // 128, k // 128), 20 + j, 3, 0.8, 1.2)
        sets.append((T(a), T(b), T(sfa), T(sfb)))
    want = [api.gemm_a8w8_blockscale(*s, out_dtype=torch.bfloat16) for s in sets]
    torch.cuda.synchronize()
    outs = [torch.empty_like(w) for w in want]
    for rep in range(4):                                       # 12 launches back to back, no host synchronisation
        for j, s in enumerate(sets):
            api.gemm_a8w8_blockscale(*s, out=outs[j], inputs_ready=True)
    status_ok(api)
    for j in range(3):
        assert torch.equal(outs[j], want[j]), f"set {j} changed under overlapped launches"
    # same C written by consecutive launches of different problems: the last one wins
    shared = torch.empty_like(want[0])
    for rep in range(3):
        for j, s in enumerate(sets):
            api.gemm_a8w8_blockscale(*s, out=shared, inputs_ready=True)
    status_ok(api)
    assert torch.equal(shared, want[2])
    # unscaled and MX kernels take the same launch path
    c0 = api.gemm_a8w8(sets[0][0], sets[0][1], out_dtype=torch.float32)
    c1 = api.gemm_a8w8(sets[0][0], sets[0][1], out_dtype=torch.float32, inputs_ready=True)
    assert torch.equal(c0, c1)
