"""Generates the golden fixtures in this directory:  python tests/golden/make_golden.py

The reference (carlushuang/gcnasm) holds no golden vectors for the FP8 GEMM path -- its inputs come from
std::random_device and it cannot be built or imported here (HIP-only) -- so the fixtures are produced by
implementations that are INDEPENDENT of oracle/oracle.c:
  * E4M3 / bf16 / E8M0 codecs ....... ml_dtypes
  * seeded generator ................. pure-Python integers and math (the hash written out literally)
  * shuffle_b ........................ literal Python loops over the reference's index formula
                                       out[d0][d2][d1][d3] = in[(d2*16+d3)*N + d0*16+d1]
                                       (opus_fmm/flatmm_a8w8_gfx950.cc:670-677)
  * GEMM results ..................... numpy float64 on ml_dtypes-decoded operands
  * quantisers ....................... numpy float32 + ml_dtypes casts
The CPU test-suite checks the oracle against these files; the GPU suite checks the CUDA path against the
oracle and against the same files.
"""
import math
import os

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
M64 = (1 << 64) - 1


def mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def draw64(seed, tid, i):
    key = mix64(seed ^ (tid << 32) ^ 0xA8F8A8F8)
    return mix64((key + i * 0xD1342543DE82EF95) & M64)


def py_uniform(n, seed, tid, lo, hi):
    out = np.empty(n, np.float32)
    for i in range(n):
        u = np.float32((draw64(seed, tid, i) >> 40) * (1.0 / 16777216.0))
        out[i] = np.float32(lo) + np.float32(np.float32(hi) - np.float32(lo)) * u
    return out


def py_normal(n, seed, tid):
    out = np.empty(n, np.float32)
    for i in range(n):
        d = draw64(seed, tid, i)
        u1 = ((d >> 40) + 1.0) * (1.0 / 16777216.0)
        u2 = ((d >> 8) & 0xFFFFFF) * (1.0 / 16777216.0)
        out[i] = np.float32(math.sqrt(-2.0 * math.log(u1)) * math.cos(6.283185307179586 * u2))
    return out


def e4m3_bytes(x):
    return np.clip(x, -448, 448).astype(ml_dtypes.float8_e4m3fn).view(np.uint8)


def e4m3_f64(b):
    return b.view(ml_dtypes.float8_e4m3fn).astype(np.float64)


def main():
    rng = np.random.default_rng(20261125)
    out = {}

    # ---- codecs ----
    out["e4m3_decode"] = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    kat = np.array([0.0, -0.0, 1.0, -1.0, 448.0, 449.0, 460.0, 463.9, 464.0, 480.0, 1e9, -500.0, np.inf, -np.inf,
                    17.0, 19.0, 0.0155, 2.0 ** -9, 2.0 ** -10, 2.0 ** -10 * 1.0001, 1.5 * 2.0 ** -9, 2.5 * 2.0 ** -9,
                    3.5 * 2.0 ** -9, 0.9375 * 2.0 ** -6, 0.96875 * 2.0 ** -6, 0.3, -0.7, 100.0, 104.0, 108.0, 120.0, 248.0],
                   np.float32)
    out["e4m3_kat_in"] = kat
    out["e4m3_kat_out"] = e4m3_bytes(kat)
    xs = (rng.standard_normal(4096) * rng.choice([1e-3, 0.05, 1.0, 30.0, 400.0], 4096)).astype(np.float32)
    out["e4m3_rand_in"] = xs
    out["e4m3_rand_out"] = e4m3_bytes(xs)
    out["bf16_rand_out"] = xs.astype(ml_dtypes.bfloat16).view(np.uint16)
    out["e8m0_decode"] = np.arange(255, dtype=np.uint8).view(ml_dtypes.float8_e8m0fnu).astype(np.float32)

    # ---- seeded generator ----
    out["gen_uniform_1234_0"] = py_uniform(64, 1234, 0, -1.0, 1.0)
    out["gen_uniform_7_5"] = py_uniform(64, 7, 5, 0.8, 1.2)
    out["gen_normal_1234_1"] = py_normal(64, 1234, 1)
    out["gen_normal_99_3"] = py_normal(64, 99, 3)

    # ---- shuffle_b ----
    N, K = 48, 64
    b_kn = rng.integers(0, 256, (K, N), dtype=np.uint8)
    flat = np.zeros(N * K, np.uint8)
    dim0, dim1, dim2, dim3 = N // 16, 16, K // 16, 16
    for d0 in range(dim0):
        for d2 in range(dim2):
            for d1 in range(dim1):
                for d3 in range(dim3):
                    flat[d0 * (dim2 * dim1 * dim3) + d2 * (dim1 * dim3) + d1 * dim3 + d3] = b_kn[d2 * 16 + d3, d0 * 16 + d1]
    out["shuffle_in_kn"] = b_kn
    out["shuffle_out"] = flat

    # ---- GEMM: unscaled NT (reference semantics), the reference's default value ranges ----
    m, n, k = 40, 48, 256
    a = e4m3_bytes(rng.uniform(0.0, 1.0, (m, k)).astype(np.float32))
    b = e4m3_bytes(rng.uniform(-0.5, 0.5, (n, k)).astype(np.float32))
    out["nt_a"], out["nt_b"] = a, b
    out["nt_c"] = (e4m3_f64(a) @ e4m3_f64(b).T).astype(np.float32)

    # ---- GEMM: block scale (SFA [K/128][M], SFB [N/128][K/128]) ----
    m, n, k = 24, 256, 384
    a = e4m3_bytes(rng.uniform(0.0, 1.0, (m, k)).astype(np.float32))
    b = e4m3_bytes(rng.uniform(-0.5, 0.5, (n, k)).astype(np.float32))
    sfa = rng.uniform(0.8, 1.2, (k // 128, m)).astype(np.float32)
    sfb = rng.uniform(0.8, 1.2, (n // 128, k // 128)).astype(np.float32)
    c = np.zeros((m, n), np.float64)
    for g in range(k // 128):
        part = e4m3_f64(a[:, g * 128:(g + 1) * 128]) @ e4m3_f64(b[:, g * 128:(g + 1) * 128]).T
        scale = sfa[g].astype(np.float64)[:, None] * np.repeat(sfb[:, g].astype(np.float64), 128)[None, :]
        c += part * scale
    out["bs_a"], out["bs_b"], out["bs_sfa"], out["bs_sfb"] = a, b, sfa, sfb
    out["bs_c"] = c.astype(np.float32)

    # ---- quantisers (numpy restatement of the benchmark configurations' rules) ----
    x = (rng.standard_normal((8, 256)) * 3.0).astype(np.float32)
    x[2, :128] = 0.0
    out["q_in"] = x
    amax = np.abs(x).max()
    s = np.float32(amax) / np.float32(448.0)
    out["q_tensor_scale"] = np.array([s], np.float32)
    out["q_tensor_q"] = e4m3_bytes((x / s).astype(np.float32))
    g = x.reshape(8, 2, 128)
    ga = np.abs(g).max(axis=2)
    gs = np.where(ga > 0, ga / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    out["q_1x128_sfa"] = np.ascontiguousarray(gs.T)                       # [K/128][M]
    out["q_1x128_q"] = e4m3_bytes((g / gs[:, :, None]).astype(np.float32)).reshape(8, 256)
    blk = x.reshape(8, 8, 32)
    ba = np.abs(blk).max(axis=2)
    e = np.where(ba > 0, np.floor(np.log2(np.where(ba > 0, ba, 1.0))).astype(np.int32) - 8, -127)
    byte = np.clip(e + 127, 0, 254).astype(np.uint8)
    out["q_mx_sf"] = byte
    out["q_mx_q"] = e4m3_bytes(np.ldexp(blk, -(byte.astype(np.int32) - 127)[:, :, None]).astype(np.float32)).reshape(8, 256)

    # ---- GEMM: MXFP8 ----
    m, n, k = 16, 32, 128
    xa = rng.standard_normal((m, k)).astype(np.float32)
    xb = rng.standard_normal((n, k)).astype(np.float32)

    def mxq(x):
        blk = x.reshape(x.shape[0], -1, 32)
        ba = np.abs(blk).max(axis=2)
        by = np.clip(np.floor(np.log2(ba)).astype(np.int32) - 8 + 127, 0, 254).astype(np.uint8)
        q = e4m3_bytes(np.ldexp(blk, -(by.astype(np.int32) - 127)[:, :, None]).astype(np.float32)).reshape(x.shape)
        return q, by

    qa, ea = mxq(xa)
    qb, eb = mxq(xb)
    da = e4m3_f64(qa).reshape(m, -1, 32) * np.exp2(ea.astype(np.float64) - 127)[:, :, None]
    db = e4m3_f64(qb).reshape(n, -1, 32) * np.exp2(eb.astype(np.float64) - 127)[:, :, None]
    out["mx_a"], out["mx_b"], out["mx_sfa"], out["mx_sfb"] = qa, qb, ea, eb
    out["mx_c"] = (da.reshape(m, k) @ db.reshape(n, k).T).astype(np.float32)

    # ---- a16w16 siblings: bf16 operands (ml_dtypes bfloat16), float64 GEMM, numpy-reshape shuffle ----
    m, n, k = 24, 48, 128
    a16 = rng.uniform(0.0, 1.0, (m, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    b16 = rng.uniform(-0.5, 0.5, (n, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    out["bf_a"], out["bf_b"] = a16.view(np.uint16), b16.view(np.uint16)
    c64 = a16.astype(np.float64) @ b16.astype(np.float64).T
    out["bf_c_f32"] = c64.astype(np.float32)
    out["bf_c_bf16"] = c64.astype(np.float32).astype(ml_dtypes.bfloat16).view(np.uint16)
    kk, nn = 40, 32                                                      # [K, N] -> [N/16][K/8][16][8]
    w = rng.integers(0, 65536, (kk, nn)).astype(np.uint16)
    out["bf_shuffle_in_kn"] = w
    out["bf_shuffle_out"] = np.ascontiguousarray(w.reshape(kk // 8, 8, nn // 16, 16).transpose(2, 0, 3, 1)).reshape(-1)

    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote golden.npz with", len(out), "arrays,", os.path.getsize(os.path.join(HERE, "golden.npz")), "bytes")


if __name__ == "__main__":
    main()
