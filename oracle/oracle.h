/*
 * CPU oracle for the A8W8 FP8 (OCP E4M3) GEMM family.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the host-side reference loops of carlushuang/gcnasm
 * (opus_gemm/gemm_a8w8_8wave.cc, opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_host.cc,
 * opus_fmm/flatmm_a8w8_gfx950.cc) plus the quantisers the benchmark configurations
 * specify.  It is the checker for the CUDA path: only the test-suite, the smoke check
 * and the CPU-baseline leg of the benchmark may link or load it.  Nothing in the
 * product library depends on it.
 *
 * Parity status: the three gemm_ref loops, shuffle_b and valid_vector follow the
 * reference source line by line (citations at each function) and are PINNED TO THE
 * REFERENCE'S OWN CODE: ref_build.py compiles those functions, cut unmodified out of a
 * reference checkout, into oracle/_ref, and the test-suite requires this restatement to
 * match them bit for bit -- live where oracle/_ref exists, and everywhere against the
 * committed outputs in tests/golden/ref_golden.npz.  The same holds for the a16w16 siblings
 * (opus_gemm/gemm_a16w16_8wave.cc:585-596, opus_fmm/flatmm_a16w16_gfx950.cc:571-582,623-666).
 * The reference builds its checkers with -ffast-math; against that build the restatement
 * agrees to 1e-6 * max|ref|.  The e4m3 type itself is third party in the reference
 * (ROCm hip/hip_fp8.h); NVIDIA's host __nv_fp8_e4m3 stands in for it (same OCP encoding).
 * The quantisers, the per-tensor-scale epilogue, bf16 output of the fp8 GEMMs and MXFP8 do
 * not exist in the reference at all: for them PARITY IS UNPINNED by the reference and is
 * pinned instead by a second independent implementation (numpy + ml_dtypes and NVIDIA's
 * host cuda_fp8.h) in the test-suite.
 */
#ifndef B200GEMM_ORACLE_H
#define B200GEMM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar codecs ---------------------------------------------------------------- */
float    orc_e4m3_to_f32(uint8_t v);          /* OCP E4M3: bias 7, max 448, NaN 0x7F/0xFF */
uint8_t  orc_f32_to_e4m3(float x);            /* RNE, saturate-to-finite, NaN -> 0x7F     */
uint16_t orc_f32_to_bf16(float x);            /* RNE, NaN kept quiet                      */
float    orc_bf16_to_f32(uint16_t v);
float    orc_e8m0_to_f32(uint8_t v);          /* 2^(v-127); 255 = NaN                     */

/* ---- seeded counter-based generators --------------------------------------------- */
void orc_fill_uniform(float *out, size_t n, uint64_t seed, uint32_t tensor_id, float lo, float hi);
void orc_fill_normal(float *out, size_t n, uint64_t seed, uint32_t tensor_id);

/* ---- quantisers -------------------------------------------------------------------- */
/* direct cast, what the reference's rand_vector does with static_cast<fp8>(float)      */
void orc_cast_e4m3(const float *x, size_t n, uint8_t *q);
/* one fp32 scale = amax/448 for the whole tensor; q = e4m3(x/scale)                    */
void orc_quant_tensor(const float *x, size_t n, uint8_t *q, float *scale);
/* A side: one scale per row per 128 K.  sfa is [K/128][M] (K-group major, M contiguous) */
void orc_quant_1x128(const float *x, int M, int K, uint8_t *q, float *sfa);
/* B side: one scale per 128x128 block.  sfb is [N/128][K/128]                           */
void orc_quant_128x128(const float *x, int N, int K, uint8_t *q, float *sfb);
/* MX: one E8M0 byte per row per 32 K.  sf is [R][K/32]                                  */
void orc_quant_mx32(const float *x, int R, int K, uint8_t *q, uint8_t *sf);

/* ---- GEMM references --------------------------------------------------------------- */
/* out_bf16 == 0: c is float*; out_bf16 == 1: c is uint16_t* (bf16 bits, RNE of the sum) */
void orc_gemm_ref_nt(const uint8_t *a, const uint8_t *b, void *c, int m, int n, int k,
                     int64_t lda, int64_t ldb, int64_t ldc, float scale_a, float scale_b,
                     int out_bf16);
void orc_gemm_ref_blockscale(const uint8_t *a, const uint8_t *b, const float *sfa,
                             const float *sfb, void *c, int m, int n, int k, int64_t lda,
                             int64_t ldb, int64_t ldc, int64_t stride_sfa, int64_t stride_sfb,
                             int group_m, int group_n, int group_k, int out_bf16);
void orc_gemm_ref_kn(const uint8_t *a, const uint8_t *b_kn, void *c, int m, int n, int k,
                     int64_t lda, int64_t ldb, int64_t ldc, int out_bf16);
void orc_gemm_ref_mx(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb,
                     void *c, int m, int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                     int out_bf16);
/* rows [m0, m1) only: lets the tests sample big problems */
void orc_gemm_ref_blockscale_rows(const uint8_t *a, const uint8_t *b, const float *sfa,
                                  const float *sfb, void *c, int m0, int m1, int n, int k,
                                  int64_t lda, int64_t ldb, int64_t ldc, int64_t stride_sfa,
                                  int64_t stride_sfb, int out_bf16);

/* ---- layout transforms ------------------------------------------------------------- */
/* [K,N] row-major -> flat [N/16][K/16][16 n][16 k] */
int orc_shuffle_b(const uint8_t *b_kn, uint8_t *out, int N, int K);
int orc_unshuffle_b(const uint8_t *flat, uint8_t *b_kn, int N, int K);
/* [N,K] row-major -> the same flat layout */
int orc_shuffle_b_nk(const uint8_t *b_nk, uint8_t *out, int N, int K);

/* ---- a16w16 siblings: bf16 operands as uint16_t bit patterns ------------------------------ */
void orc_gemm_ref_nt_bf16(const uint16_t *a, const uint16_t *b, void *c, int m, int n, int k, int64_t lda,
                          int64_t ldb, int64_t ldc, int out_bf16);
void orc_gemm_ref_kn_bf16(const uint16_t *a, const uint16_t *b_kn, void *c, int m, int n, int k, int64_t lda,
                          int64_t ldb, int64_t ldc, int out_bf16);
/* [K,N] row-major -> flat [N/16][K/8][16 n][8 k] */
int orc_shuffle_b_bf16(const uint16_t *b_kn, uint16_t *out, int N, int K);
int orc_unshuffle_b_bf16(const uint16_t *flat, uint16_t *b_kn, int N, int K);

/* ---- checker ------------------------------------------------------------------------ */
/* returns 1 when no |ref-res| exceeds threshold; prints up to 10 offenders if verbose   */
int orc_valid_vector(const float *ref, const float *res, int64_t n, float threshold, int verbose);
/* max|ref-res| and max|ref| over n floats */
void orc_max_err(const float *ref, const float *res, int64_t n, float *max_err, float *max_ref);

int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
