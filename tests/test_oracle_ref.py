"""CPU: the C restatement (oracle/oracle.c) against the REFERENCE'S OWN host checkers.

Two layers.  (1) ``tests/golden/ref_golden.npz`` holds outputs of the reference's functions run through
``oracle/_ref`` (made by tests/golden/make_ref_golden.py); the restatement must reproduce them bit for bit.
These tests run everywhere.  (2) Where ``oracle/_ref`` itself is present (it is built whenever a reference
checkout is at hand, and travels with the tree as a binary), restatement and reference run side by side on fresh
seeded inputs: shuffles and valid_vector bit-exact, GEMMs bit-exact against the IEEE build and within
1e-6 * max|ref| of the build that uses the reference Makefiles' -ffast-math.
"""
import os

import numpy as np
import pytest

from conftest import GOLDEN


@pytest.fixture(scope="module")
def RG():
    return np.load(os.path.join(GOLDEN, "ref_golden.npz"))


@pytest.fixture(scope="module")
def R():
    from oracle import ref

    if not ref.build():
        pytest.skip("oracle/_ref is not built (no reference checkout on this machine)")
    return ref


# ---- layer 1: committed outputs of the reference's code ------------------------------------------------
def test_restated_gemm_refs_reproduce_reference_outputs(O, RG):
    assert np.array_equal(O.gemm_ref_nt(RG["nt_a"], RG["nt_b"]), RG["nt_c"])
    assert np.array_equal(O.gemm_ref_kn(RG["nt_a"], RG["kn_b"]), RG["kn_c"])
    c = O.gemm_ref_blockscale(RG["bs_a"], RG["bs_b"], RG["bs_sfa"], RG["bs_sfb"])
    assert np.array_equal(c, RG["bs_c"])
    e, r = O.max_err(RG["bs_c_fastmath"], c)
    assert e <= 1e-6 * r
    assert np.array_equal(O.gemm_ref_blockscale(RG["bs_a"], RG["bs_b"], RG["bs_sfa"], RG["bs_sfb"], rows=(3, 17)), RG["bs_c"][3:17])


def test_restated_shuffles_reproduce_reference_outputs(O, RG):
    assert np.array_equal(O.shuffle_b(RG["shuffle_in_kn"]), RG["shuffle_out"])
    assert np.array_equal(O.shuffle_b_bf16(RG["bf_shuffle_in_kn"]), RG["bf_shuffle_out"])


def test_restated_bf16_gemm_refs_reproduce_reference_outputs(O, RG):
    assert np.array_equal(O.gemm_ref_nt_bf16(RG["bf_a"], RG["bf_b"], out_bf16=True), RG["bf_c_nt"])
    assert np.array_equal(O.gemm_ref_kn_bf16(RG["bf_a"], np.ascontiguousarray(RG["bf_b"].T), out_bf16=True), RG["bf_c_kn"])


def test_e4m3_codec_of_the_shim(O, RG):
    """The operand type is third party in the reference (hip/hip_fp8.h); the shim binds NVIDIA's host type."""
    t = O.e4m3_decode_table()
    ok = ~np.isnan(RG["e4m3_decode"])
    assert np.array_equal(t[ok].view(np.uint32), RG["e4m3_decode"][ok].view(np.uint32))
    assert np.array_equal(np.isnan(t), ~ok)
    assert np.array_equal(O.cast_e4m3(RG["e4m3_cast_in"]), RG["e4m3_cast_out"])


# ---- layer 2: side by side with oracle/_ref ------------------------------------------------------------
@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (17, 33, 128), (64, 96, 1024)])
def test_live_gemm_nt_and_kn(O, R, m, n, k):
    a = O.cast_e4m3(O.fill_uniform((m, k), 100 + m, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((n, k), 100 + m, 1, -0.5, 0.5))
    want = R.gemm_ref_nt(a, b)
    assert np.array_equal(O.gemm_ref_nt(a, b), want)
    e, r = O.max_err(R.gemm_ref_nt(a, b, flavour="fast"), want)
    assert e <= 1e-6 * r
    b_kn = np.ascontiguousarray(b.T)
    assert np.array_equal(O.gemm_ref_kn(a, b_kn), R.gemm_ref_kn(a, b_kn))
    assert np.array_equal(R.gemm_ref_kn(a, b_kn), want)     # same sums in the same order


@pytest.mark.parametrize("m,n,k", [(5, 128, 128), (37, 256, 512), (130, 384, 1024)])
def test_live_gemm_blockscale(O, R, m, n, k):
    a = O.cast_e4m3(O.fill_uniform((m, k), 200 + m, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((n, k), 200 + m, 1, -0.5, 0.5))
    sfa = O.fill_uniform((k // 128, m), 200 + m, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), 200 + m, 3, 0.8, 1.2)
    want = R.gemm_ref_blockscale(a, b, sfa, sfb)
    assert np.array_equal(O.gemm_ref_blockscale(a, b, sfa, sfb), want)
    fast = R.gemm_ref_blockscale(a, b, sfa, sfb, flavour="fast")
    e, r = O.max_err(fast, want)
    assert e <= 1e-6 * r
    # the benchmark configurations' data: N(0,1) quantised with amax/448 scales
    qa, sa = O.quant_1x128(O.fill_normal((m, k), 300 + m, 0))
    qb, sb = O.quant_128x128(O.fill_normal((n, k), 300 + m, 1))
    assert np.array_equal(O.gemm_ref_blockscale(qa, qb, sa, sb), R.gemm_ref_blockscale(qa, qb, sa, sb))


@pytest.mark.parametrize("n,k", [(16, 16), (48, 64), (272, 400), (512, 1024)])
def test_live_shuffle_b(O, R, n, k):
    rng = np.random.default_rng(n * 7 + k)
    w = rng.integers(0, 256, (k, n), dtype=np.uint8)
    assert np.array_equal(O.shuffle_b(w), R.shuffle_b(w))
    if k % 8 == 0:
        w16 = rng.integers(0, 65536, (k, n), dtype=np.uint16)
        assert np.array_equal(O.shuffle_b_bf16(w16), R.shuffle_b_bf16(w16))


def test_live_bf16_gemm_refs(O, R):
    a = O.f32_to_bf16_bits(O.fill_uniform((21, 160), 400, 0, 0.0, 1.0))
    b = O.f32_to_bf16_bits(O.fill_uniform((35, 160), 400, 1, -0.5, 0.5))
    assert np.array_equal(O.gemm_ref_nt_bf16(a, b, out_bf16=True), R.gemm_ref_nt_bf16(a, b))
    b_kn = np.ascontiguousarray(b.T)
    assert np.array_equal(O.gemm_ref_kn_bf16(a, b_kn, out_bf16=True), R.gemm_ref_kn_bf16(a, b_kn))


def test_live_valid_vector(O, R):
    rng = np.random.default_rng(9)
    ref = rng.standard_normal(4096).astype(np.float32)
    for thr in (0.1, 1e-3):
        for bump in (0.0, thr * 0.999, thr, thr * 1.001, 1.0):
            res = ref.copy()
            res[123] += np.float32(bump)
            for which in ("a8w8", "bs"):
                assert O.valid_vector(ref, res, thr) == R.valid_vector(ref, res, thr, which), (thr, bump, which)


def test_live_e4m3_cast(O, R):
    xs = np.concatenate([O.fill_uniform(2000, 500, 0, -500.0, 500.0), O.fill_uniform(2000, 500, 1, -1.0, 1.0),
                         O.fill_uniform(500, 500, 2, -0.02, 0.02)])
    assert np.array_equal(O.cast_e4m3(xs), R.cast_e4m3(xs))
