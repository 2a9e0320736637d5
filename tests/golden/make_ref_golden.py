"""Generates ``ref_golden.npz``: outputs of the REFERENCE'S OWN host checkers, run here.

    python oracle/ref_build.py <reference checkout>      # compiles the reference's functions into oracle/_ref
    python tests/golden/make_ref_golden.py

``oracle/_ref`` holds gemm_ref (x5), shuffle_b (x2) and valid_vector exactly as the reference wrote them
(oracle/ref_build.py cuts them out of the reference's files; oracle/_ref/MANIFEST.json names the lines), compiled
with g++ in IEEE order.  This script feeds them small seeded inputs in the reference's own value ranges
(A ~ U[0,1), B ~ U[-0.5,0.5), scales ~ U[0.8,1.2): gemm_a8w8_blockscale_host.cc:207-210) and stores inputs and
outputs.  The CPU test-suite then requires the C restatement (oracle/oracle.c) to reproduce every stored output
BIT FOR BIT, which pins the restatement to the reference's code on machines that have no reference checkout.
The inputs are stored next to the outputs, so nothing depends on how they were drawn.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402  (only to draw seeded inputs and encode them)
from oracle import ref as R  # noqa: E402


def main():
    if not R.build():
        raise SystemExit("oracle/_ref is not built and no reference checkout was found")
    g = {}
    # plain NT gemm_ref (gemm_a8w8_8wave.cc:601-612), ragged sizes
    a = O.cast_e4m3(O.fill_uniform((24, 192), 11, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((40, 192), 11, 1, -0.5, 0.5))
    g["nt_a"], g["nt_b"], g["nt_c"] = a, b, R.gemm_ref_nt(a, b)
    # flat-matmul gemm_ref on the unshuffled [K,N] matrix (flatmm_a8w8_gfx950.cc:586-597)
    b_kn = O.cast_e4m3(O.fill_uniform((192, 48), 11, 2, -0.5, 0.5))
    g["kn_b"], g["kn_c"] = b_kn, R.gemm_ref_kn(a, b_kn)
    # block-scale gemm_ref (gemm_a8w8_blockscale_host.cc:66-90): 3 K groups, 2 N blocks, 1x128x128 groups
    a = O.cast_e4m3(O.fill_uniform((20, 384), 12, 0, 0.0, 1.0))
    b = O.cast_e4m3(O.fill_uniform((256, 384), 12, 1, -0.5, 0.5))
    sfa = O.fill_uniform((3, 20), 12, 2, 0.8, 1.2)
    sfb = O.fill_uniform((2, 3), 12, 3, 0.8, 1.2)
    g["bs_a"], g["bs_b"], g["bs_sfa"], g["bs_sfb"] = a, b, sfa, sfb
    g["bs_c"] = R.gemm_ref_blockscale(a, b, sfa, sfb)
    g["bs_c_fastmath"] = R.gemm_ref_blockscale(a, b, sfa, sfb, flavour="fast")      # the reference's build flags
    # shuffle_b<fp8> (flatmm_a8w8_gfx950.cc:638-681)
    rng = np.random.default_rng(5)
    w = rng.integers(0, 256, (64, 48), dtype=np.uint8)
    g["shuffle_in_kn"], g["shuffle_out"] = w, R.shuffle_b(w)
    # bf16 siblings (gemm_a16w16_8wave.cc:585-596, flatmm_a16w16_gfx950.cc:571-582, 623-666)
    a16 = O.f32_to_bf16_bits(O.fill_uniform((18, 96), 13, 0, 0.0, 1.0))
    b16 = O.f32_to_bf16_bits(O.fill_uniform((24, 96), 13, 1, -0.5, 0.5))
    b16_kn = np.ascontiguousarray(b16.T)
    g["bf_a"], g["bf_b"] = a16, b16
    g["bf_c_nt"] = R.gemm_ref_nt_bf16(a16, b16)
    g["bf_c_kn"] = R.gemm_ref_kn_bf16(a16, b16_kn)
    w16 = rng.integers(0, 65536, (40, 32), dtype=np.uint16)
    g["bf_shuffle_in_kn"], g["bf_shuffle_out"] = w16, R.shuffle_b_bf16(w16)
    # the e4m3 codec the shim binds host_fp8_t to (third party in the reference: hip/hip_fp8.h)
    g["e4m3_decode"] = R.e4m3_decode_table()
    xs = np.concatenate([O.fill_uniform(256, 14, 0, -500.0, 500.0), O.fill_uniform(256, 14, 1, -2.0, 2.0),
                         np.array([0.0, -0.0, 448.0, 449.0, 464.0, 465.0, 1e9, -1e9, 2 ** -9, 2 ** -10, 1.5 * 2 ** -10], np.float32)])
    g["e4m3_cast_in"], g["e4m3_cast_out"] = xs, R.cast_e4m3(xs)
    np.savez_compressed(os.path.join(HERE, "ref_golden.npz"), **g)
    print("wrote ref_golden.npz:", ", ".join(sorted(g)))


if __name__ == "__main__":
    main()
