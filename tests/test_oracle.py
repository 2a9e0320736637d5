"""CPU: the oracle against the golden fixtures (made by independent implementations, see
tests/golden/make_golden.py) and against ml_dtypes / numpy on fresh seeded inputs."""
import os

import ml_dtypes
import numpy as np
import pytest

from conftest import GOLDEN


@pytest.fixture(scope="module")
def G():
    return np.load(os.path.join(GOLDEN, "golden.npz"))


def test_e4m3_decode_table(O, G):
    t = O.e4m3_decode_table()
    ok = ~np.isnan(G["e4m3_decode"])
    assert np.array_equal(t[ok].view(np.uint32), G["e4m3_decode"][ok].view(np.uint32))
    assert np.isnan(t[0x7F]) and np.isnan(t[0xFF]) and t[0x7E] == 448.0 and t[0xFE] == -448.0


def test_e4m3_encode_known_answers(O, G):
    assert np.array_equal(O.cast_e4m3(G["e4m3_kat_in"]), G["e4m3_kat_out"])
    assert np.array_equal(O.cast_e4m3(G["e4m3_rand_in"]), G["e4m3_rand_out"])
    # saturate-to-finite facts of the HIP / NVIDIA fp8 casts: 460 -> 0x7E, -500 -> 0xFE, 17 -> 16, 19 -> 20
    q = O.cast_e4m3(np.array([460.0, -500.0, 17.0, 19.0, np.nan], np.float32))
    t = O.e4m3_decode_table()
    assert q[0] == 0x7E and q[1] == 0xFE and t[q[2]] == 16.0 and t[q[3]] == 20.0 and (q[4] & 0x7F) == 0x7F


def test_e4m3_encode_exhaustive_midpoints(O):
    """every representable value, every midpoint between neighbours and a hair either side."""
    t = O.e4m3_decode_table()
    vals = np.sort(t[:0x7F].astype(np.float64))
    mids = (vals[:-1] + vals[1:]) / 2
    xs = np.concatenate([vals, mids, np.nextafter(mids.astype(np.float32), np.float32(1e9)),
                         np.nextafter(mids.astype(np.float32), np.float32(-1e9))]).astype(np.float32)
    xs = np.concatenate([xs, -xs])
    want = np.clip(xs, -448, 448).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(O.cast_e4m3(xs), want)


def test_bf16_and_e8m0(O, G):
    assert np.array_equal(O.f32_to_bf16_bits(G["e4m3_rand_in"]), G["bf16_rand_out"])
    L = O.lib()
    got = np.array([L.orc_f32_to_bf16(float(x)) for x in G["e4m3_rand_in"][:512]], np.uint16)
    assert np.array_equal(got, G["bf16_rand_out"][:512])
    e = np.array([L.orc_e8m0_to_f32(i) for i in range(255)], np.float32)
    assert np.array_equal(e, G["e8m0_decode"])
    assert np.isnan(L.orc_e8m0_to_f32(255))


def test_seeded_generators(O, G):
    assert np.array_equal(O.fill_uniform(64, 1234, 0, -1.0, 1.0), G["gen_uniform_1234_0"])
    assert np.array_equal(O.fill_uniform(64, 7, 5, 0.8, 1.2), G["gen_uniform_7_5"])
    assert np.array_equal(O.fill_normal(64, 1234, 1), G["gen_normal_1234_1"])
    assert np.array_equal(O.fill_normal(64, 99, 3), G["gen_normal_99_3"])
    # counter based: any prefix/slice is reproducible, tensors and seeds are independent streams
    big = O.fill_normal(1 << 16, 1234, 1)
    assert np.array_equal(big[:64], G["gen_normal_1234_1"])
    assert abs(float(big.mean())) < 0.02 and abs(float(big.std()) - 1.0) < 0.02
    assert not np.array_equal(O.fill_normal(64, 1234, 2), G["gen_normal_1234_1"])


def test_shuffle_b_golden_and_roundtrip(O, G):
    assert np.array_equal(O.shuffle_b(G["shuffle_in_kn"]), G["shuffle_out"])
    assert np.array_equal(O.unshuffle_b(G["shuffle_out"], 48, 64), G["shuffle_in_kn"])
    assert np.array_equal(O.shuffle_b_nk(np.ascontiguousarray(G["shuffle_in_kn"].T)), G["shuffle_out"])


@pytest.mark.parametrize("n,k", [(16, 16), (32, 128), (272, 400), (512, 256)])
def test_shuffle_b_vs_numpy_reshape(O, n, k):
    rng = np.random.default_rng(n * 1000 + k)
    b_kn = rng.integers(0, 256, (k, n), dtype=np.uint8)
    # [K,N] -> [K/16, 16, N/16, 16] -> [N/16, K/16, n16, k16]
    want = b_kn.reshape(k // 16, 16, n // 16, 16).transpose(2, 0, 3, 1).reshape(-1)
    assert np.array_equal(O.shuffle_b(b_kn), want)
    assert np.array_equal(O.unshuffle_b(want, n, k), b_kn)


def test_shuffle_b_rejects_ragged(O):
    with pytest.raises(ValueError):
        O.shuffle_b(np.zeros((16, 24), np.uint8))
    with pytest.raises(ValueError):
        O.shuffle_b(np.zeros((24, 16), np.uint8))


def test_gemm_refs_golden(O, G):
    e, r = O.max_err(G["nt_c"], O.gemm_ref_nt(G["nt_a"], G["nt_b"]))
    assert e <= 1e-5 * r
    e, r = O.max_err(G["bs_c"], O.gemm_ref_blockscale(G["bs_a"], G["bs_b"], G["bs_sfa"], G["bs_sfb"]))
    assert e <= 1e-5 * r
    e, r = O.max_err(G["mx_c"], O.gemm_ref_mx(G["mx_a"], G["mx_b"], G["mx_sfa"], G["mx_sfb"]))
    assert e <= 1e-5 * r
    # flat reference reads the UNSHUFFLED [K,N] matrix
    e, r = O.max_err(G["nt_c"], O.gemm_ref_kn(G["nt_a"], np.ascontiguousarray(G["nt_b"].T)))
    assert e <= 1e-5 * r


def test_gemm_ref_variants_consistent(O):
    a = O.cast_e4m3(O.fill_uniform((33, 256), 3, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((128, 256), 3, 1, -0.5, 0.5))
    plain = O.gemm_ref_nt(a, b)
    ones_a = np.ones((2, 33), np.float32)
    ones_b = np.ones((1, 2), np.float32)
    assert np.array_equal(O.gemm_ref_blockscale(a, b, ones_a, ones_b), plain)          # unit scales = unscaled
    assert np.array_equal(O.gemm_ref_blockscale(a, b, ones_a, ones_b, rows=(5, 20)), plain[5:20])
    sc = O.gemm_ref_nt(a, b, 0.5, 4.0)
    assert np.array_equal(sc, plain * np.float32(2.0))
    bf = O.gemm_ref_nt(a, b, out_bf16=True)
    assert np.array_equal(bf, O.f32_to_bf16_bits(plain))
    sf = np.full((33, 8), 127, np.uint8)
    sfb = np.full((128, 8), 127, np.uint8)
    e, r = O.max_err(plain, O.gemm_ref_mx(a, b, sf, sfb))
    assert e <= 1e-5 * r


def test_quantisers_golden(O, G):
    q, s = O.quant_tensor(G["q_in"])
    assert np.array_equal(q, G["q_tensor_q"]) and s[0] == G["q_tensor_scale"][0]
    q, s = O.quant_1x128(G["q_in"])
    assert np.array_equal(q, G["q_1x128_q"]) and np.array_equal(s, G["q_1x128_sfa"])
    q, s = O.quant_mx32(G["q_in"])
    assert np.array_equal(q, G["q_mx_q"]) and np.array_equal(s, G["q_mx_sf"])


def test_quantiser_properties(O):
    x = O.fill_normal((256, 512), 21, 0)
    x[7] = 0.0
    t = O.e4m3_decode_table()
    q, sfa = O.quant_1x128(x)
    assert sfa.shape == (4, 256) and np.all(sfa[:, 7] == 1.0)
    deq = t[q].reshape(256, 4, 128) * sfa.T[:, :, None]
    assert np.max(np.abs(deq.reshape(256, 512) - x)) <= np.max(np.abs(x)) * 2 ** -4
    assert np.abs(t[q]).max() == 448.0                    # every non-zero group reaches the format maximum
    q, sfb = O.quant_128x128(x)
    assert sfb.shape == (2, 4)
    for nb in range(2):
        for g in range(4):
            blk = x[nb * 128:(nb + 1) * 128, g * 128:(g + 1) * 128]
            assert sfb[nb, g] == np.float32(np.abs(blk).max()) / np.float32(448.0)
    q, e = O.quant_mx32(x)
    assert e.shape == (256, 16) and np.all(e[7] == 0) and np.all(q[7] == 0)
    amax = np.abs(x.reshape(256, 16, 32)).max(axis=2)
    live = amax > 0
    assert np.array_equal(e[live].astype(np.int32) - 127, np.floor(np.log2(amax[live])).astype(np.int32) - 8)


def test_valid_vector_semantics(O):
    ref = np.zeros(100, np.float32)
    res = ref.copy()
    assert O.valid_vector(ref, res, 0.1)
    res[3] = 0.1000001
    assert not O.valid_vector(ref, res, 0.1)
    res[3] = 0.1
    assert O.valid_vector(ref, res, 0.1)                  # strictly greater than the threshold fails
    res[50] = np.nan
    assert not O.valid_vector(ref, res, 0.1)
    e, r = O.max_err(np.array([1.0, -4.0], np.float32), np.array([1.5, -4.0], np.float32))
    assert e == 0.5 and r == 4.0


def test_bf16_siblings_golden(O, G):
    """a16w16 references and the bf16 shuffle against ml_dtypes / numpy-reshape fixtures."""
    c = O.gemm_ref_nt_bf16(G["bf_a"], G["bf_b"], out_bf16=False)
    e, r = O.max_err(G["bf_c_f32"], c)
    assert e <= 1e-5 * r                                        # float64 vs sequential fp32 sums
    cb = O.gemm_ref_nt_bf16(G["bf_a"], G["bf_b"], out_bf16=True)
    diff = np.abs(cb.astype(np.int32) - G["bf_c_bf16"].astype(np.int32))
    assert diff.max() <= 1                                      # at most one bf16 ulp where the fp32 sums differ
    assert (diff == 0).mean() > 0.97
    ck = O.gemm_ref_kn_bf16(G["bf_a"], np.ascontiguousarray(G["bf_b"].T), out_bf16=False)
    assert np.array_equal(ck, c)                                # same sums in the same order
    assert np.array_equal(O.shuffle_b_bf16(G["bf_shuffle_in_kn"]), G["bf_shuffle_out"])
    assert np.array_equal(O.unshuffle_b_bf16(G["bf_shuffle_out"], 32, 40), G["bf_shuffle_in_kn"])
    with pytest.raises(ValueError):
        O.shuffle_b_bf16(np.zeros((12, 16), np.uint16))         # K % 8 != 0


def test_bf16_shuffle_is_the_byte_shuffle_of_the_nk_view(O):
    """In bytes the bf16 flat image equals the 8-bit flat image of the [N][2K]-byte matrix."""
    k, n = 64, 48
    w = (np.arange(k * n, dtype=np.uint32) * 2654435761 >> 7).astype(np.uint16).reshape(k, n)
    flat16 = O.shuffle_b_bf16(w)
    nk_bytes = np.ascontiguousarray(w.T).view(np.uint8).reshape(n, 2 * k)
    assert np.array_equal(flat16.view(np.uint8), O.shuffle_b_nk(nk_bytes))
