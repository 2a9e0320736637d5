/*
 * CPU oracle for the A8W8 FP8 GEMM family -- TEST INFRASTRUCTURE ONLY (see oracle.h).
 * Plain C11 + OpenMP.  Build with -ffp-contract=off and WITHOUT -ffast-math so every
 * float operation is the IEEE one written here.
 */
#include "oracle.h"

#include <math.h>
#include <stdio.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------ */
/* scalar codecs                                                                         */
/* ------------------------------------------------------------------------------------ */

static inline uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* OCP E4M3 ("e4m3fn"): 1-4-3, bias 7, no infinities, 0x7F/0xFF are NaN, max finite 448.
 * This is the encoding of __hip_fp8_e4m3 on gfx950 (the reference states max 0x7E=448 and
 * NaN 0x7F at wmma_opus_rdna4/opus/opus.hpp:858-865) and of NVIDIA's __nv_fp8_e4m3.      */
float orc_e4m3_to_f32(uint8_t v) {
    const uint32_t sign = (uint32_t)(v & 0x80u) << 24;
    const int e = (v >> 3) & 0xF;
    const int m = v & 7;
    if (e == 0xF && m == 7) return bits_f32(sign | 0x7FC00000u);
    if (e == 0) {
        /* subnormal: m * 2^-9 */
        const float mag = (float)m * (1.0f / 512.0f);
        return bits_f32(f32_bits(mag) | sign);
    }
    return bits_f32(sign | ((uint32_t)(e - 7 + 127) << 23) | ((uint32_t)m << 20));
}

/* float -> E4M3 with round-to-nearest-even and saturation to +-448, the behaviour of
 * static_cast<__hip_fp8_e4m3>(float) used by the reference's rand_vector
 * (opus_gemm/gemm_a8w8_8wave.cc:576, gemm_a8w8_blockscale_host.cc:41).                   */
uint8_t orc_f32_to_e4m3(float x) {
    const uint32_t bits = f32_bits(x);
    const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
    const uint32_t abits = bits & 0x7FFFFFFFu;
    if (abits > 0x7F800000u) return (uint8_t)(sign | 0x7F);       /* NaN */
    const float a = bits_f32(abits);
    if (a > 448.0f) return (uint8_t)(sign | 0x7E);                /* saturate (inf too) */
    if (a < 0.015625f) {                                          /* below 2^-6: subnormal grid 2^-9 */
        const float q = nearbyintf(a * 512.0f);                   /* exact scale, RNE */
        return (uint8_t)(sign | (uint8_t)q);                      /* q==8 is 0x08 = 2^-6 */
    }
    uint32_t r = abits;
    const uint32_t lsb = (r >> 20) & 1u;
    r += 0x7FFFFu + lsb;                                          /* RNE on the 20 dropped bits */
    const uint32_t e = (r >> 23) - 127u + 7u;
    const uint32_t m = (r >> 20) & 7u;
    uint32_t byte = (e << 3) | m;
    if (byte > 0x7Eu) byte = 0x7Eu;
    return (uint8_t)(sign | byte);
}

/* float -> bf16, round-to-nearest-even: what static_cast<bf16_t>(sum) does in the bf16
 * sibling (opus_gemm/gemm_a16w16_8wave.cc:593; bit recipe at
 * wmma_opus_rdna4/opus/opus.hpp:944-950).                                                */
uint16_t orc_f32_to_bf16(float x) {
    uint32_t u = f32_bits(x);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float orc_bf16_to_f32(uint16_t v) { return bits_f32((uint32_t)v << 16); }

/* E8M0: value 2^(v-127), 0xFF is NaN ("127 = 1.0", wmma_opus_rdna4/opus/opus.hpp:1786).   */
float orc_e8m0_to_f32(uint8_t v) {
    if (v == 0xFF) return bits_f32(0x7FC00000u);
    if (v == 0) return bits_f32(0x00400000u);                     /* 2^-127 is a float subnormal */
    return bits_f32((uint32_t)v << 23);
}

/* ------------------------------------------------------------------------------------ */
/* seeded generators                                                                     */
/* ------------------------------------------------------------------------------------ */
/* The reference seeds from std::random_device (gemm_a8w8_8wave.cc:570-571), so it has no
 * reproducible inputs.  This counter-based generator replaces it: element i of tensor t
 * depends only on (seed, t, i), so any slice can be regenerated independently.           */

static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline uint64_t stream_key(uint64_t seed, uint32_t tensor_id) {
    return mix64(seed ^ ((uint64_t)tensor_id << 32) ^ 0xA8F8A8F8ull);
}

static inline uint64_t draw64(uint64_t key, uint64_t idx) { return mix64(key + idx * 0xD1342543DE82EF95ull); }

void orc_fill_uniform(float *out, size_t n, uint64_t seed, uint32_t tensor_id, float lo, float hi) {
    const uint64_t key = stream_key(seed, tensor_id);
    const float span = hi - lo;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        const uint32_t r = (uint32_t)(draw64(key, (uint64_t)i) >> 40);   /* 24 bits */
        const float u = (float)r * (1.0f / 16777216.0f);                  /* [0,1) exact */
        out[i] = lo + span * u;
    }
}

void orc_fill_normal(float *out, size_t n, uint64_t seed, uint32_t tensor_id) {
    const uint64_t key = stream_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        const uint64_t d = draw64(key, (uint64_t)i);
        const uint32_t r1 = (uint32_t)(d >> 40);                          /* 24 bits */
        const uint32_t r2 = (uint32_t)(d >> 8) & 0xFFFFFFu;               /* 24 other bits */
        const double u1 = ((double)r1 + 1.0) * (1.0 / 16777216.0);        /* (0,1] */
        const double u2 = (double)r2 * (1.0 / 16777216.0);                /* [0,1) */
        out[i] = (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2));
    }
}

/* ------------------------------------------------------------------------------------ */
/* quantisers (specified by the benchmark configurations, absent from the reference)     */
/* ------------------------------------------------------------------------------------ */

void orc_cast_e4m3(const float *x, size_t n, uint8_t *q) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) q[i] = orc_f32_to_e4m3(x[i]);
}

/* scale = amax/448 (1.0 when the group is all zero), q = e4m3(x / scale) */
static inline float scale_from_amax(float amax) { return amax > 0.0f ? amax / 448.0f : 1.0f; }

void orc_quant_tensor(const float *x, size_t n, uint8_t *q, float *scale) {
    float amax = 0.0f;
#pragma omp parallel for reduction(max : amax) schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        const float a = fabsf(x[i]);
        if (a > amax) amax = a;
    }
    const float s = scale_from_amax(amax);
    *scale = s;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) q[i] = orc_f32_to_e4m3(x[i] / s);
}

/* SFA is stored K-group major with M contiguous, the reference's layout
 * (sfa[k_group_idx*stride_sfa + m_group], gemm_a8w8_blockscale_host.cc:78; stride_sfa =
 * num_groups_m at :244).                                                                 */
void orc_quant_1x128(const float *x, int M, int K, uint8_t *q, float *sfa) {
    const int KG = K / 128;
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < M; ++i) {
        for (int g = 0; g < KG; ++g) {
            const float *src = x + (size_t)i * K + (size_t)g * 128;
            float amax = 0.0f;
            for (int p = 0; p < 128; ++p) amax = fmaxf(amax, fabsf(src[p]));
            const float s = scale_from_amax(amax);
            sfa[(size_t)g * M + i] = s;
            uint8_t *dst = q + (size_t)i * K + (size_t)g * 128;
            for (int p = 0; p < 128; ++p) dst[p] = orc_f32_to_e4m3(src[p] / s);
        }
    }
}

/* SFB is [N/128][K/128] (sfb[n_group*stride_sfb + k_group_idx], host.cc:79; stride_sfb =
 * num_groups_k at :245).                                                                 */
void orc_quant_128x128(const float *x, int N, int K, uint8_t *q, float *sfb) {
    const int NG = N / 128, KG = K / 128;
#pragma omp parallel for collapse(2) schedule(static)
    for (int nb = 0; nb < NG; ++nb) {
        for (int g = 0; g < KG; ++g) {
            float amax = 0.0f;
            for (int r = 0; r < 128; ++r) {
                const float *src = x + (size_t)(nb * 128 + r) * K + (size_t)g * 128;
                for (int p = 0; p < 128; ++p) amax = fmaxf(amax, fabsf(src[p]));
            }
            const float s = scale_from_amax(amax);
            sfb[(size_t)nb * KG + g] = s;
            for (int r = 0; r < 128; ++r) {
                const float *src = x + (size_t)(nb * 128 + r) * K + (size_t)g * 128;
                uint8_t *dst = q + (size_t)(nb * 128 + r) * K + (size_t)g * 128;
                for (int p = 0; p < 128; ++p) dst[p] = orc_f32_to_e4m3(src[p] / s);
            }
        }
    }
}

/* MX 1x32: shared exponent e = floor(log2(amax)) - 8 (8 = emax of E4M3), stored as the
 * E8M0 byte clamp(e+127, 0, 254); elements are e4m3(x * 2^-e) with saturation.  An
 * all-zero block stores byte 0 and zero elements.  (The repository's only E8M0 code,
 * mla_agentic_v0/flash_mla/quant.py:28-37, rounds the exponent UP and is not followed.)   */
void orc_quant_mx32(const float *x, int R, int K, uint8_t *q, uint8_t *sf) {
    const int KB = K / 32;
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < R; ++i) {
        for (int b = 0; b < KB; ++b) {
            const float *src = x + (size_t)i * K + (size_t)b * 32;
            uint8_t *dst = q + (size_t)i * K + (size_t)b * 32;
            float amax = 0.0f;
            for (int p = 0; p < 32; ++p) amax = fmaxf(amax, fabsf(src[p]));
            if (!(amax > 0.0f)) {
                sf[(size_t)i * KB + b] = 0;
                for (int p = 0; p < 32; ++p) dst[p] = (uint8_t)((f32_bits(src[p]) >> 24) & 0x80u);
                continue;
            }
            int ex;
            (void)frexpf(amax, &ex);                 /* amax = f * 2^ex, f in [0.5,1) */
            int e = (ex - 1) - 8;                    /* floor(log2(amax)) - emax */
            int byte = e + 127;
            if (byte < 0) byte = 0;
            if (byte > 254) byte = 254;
            e = byte - 127;
            sf[(size_t)i * KB + b] = (uint8_t)byte;
            for (int p = 0; p < 32; ++p) dst[p] = orc_f32_to_e4m3(ldexpf(src[p], -e));
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* GEMM references                                                                       */
/* ------------------------------------------------------------------------------------ */

static float g_lut[256];
static int g_lut_ready = 0;
static void lut_init(void) {
    if (g_lut_ready) return;
#pragma omp critical(orc_lut)
    {
        if (!g_lut_ready) {
            for (int i = 0; i < 256; ++i) g_lut[i] = orc_e4m3_to_f32((uint8_t)i);
            g_lut_ready = 1;
        }
    }
}

static inline void store_out(void *c, int64_t idx, float v, int out_bf16) {
    if (out_bf16) ((uint16_t *)c)[idx] = orc_f32_to_bf16(v);
    else ((float *)c)[idx] = v;
}

/* Plain NT reference: opus_gemm/gemm_a8w8_8wave.cc:601-612 -- sum += float(a[i*lda+p]) *
 * float(b[j*ldb+p]), sequential p, fp32, collapse(2) over (i,j).  The reference has no
 * scale; scale_a*scale_b (per-tensor) multiplies the finished sum, so 1,1 reproduces it.  */
void orc_gemm_ref_nt(const uint8_t *a, const uint8_t *b, void *c, int m, int n, int k,
                     int64_t lda, int64_t ldb, int64_t ldc, float scale_a, float scale_b,
                     int out_bf16) {
    lut_init();
    const float s = scale_a * scale_b;
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int p = 0; p < k; ++p) sum += g_lut[a[i * lda + p]] * g_lut[b[j * ldb + p]];
            store_out(c, i * ldc + j, (scale_a == 1.0f && scale_b == 1.0f) ? sum : sum * s, out_bf16);
        }
    }
}

/* Block-scale reference: gemm_a8w8_blockscale_host.cc:66-90.  The scale product is
 * applied to every term inside the inner loop (:84) and SFA is indexed K-group major
 * (:78).  The reference builds this loop with -ffast-math (Makefile:5); here it is
 * evaluated in strict IEEE order.                                                         */
void orc_gemm_ref_blockscale_rows(const uint8_t *a, const uint8_t *b, const float *sfa,
                                  const float *sfb, void *c, int m0, int m1, int n, int k,
                                  int64_t lda, int64_t ldb, int64_t ldc, int64_t stride_sfa,
                                  int64_t stride_sfb, int out_bf16) {
    lut_init();
    const int group_m = 1, group_n = 128, group_k = 128;
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = m0; i < m1; ++i) {
        for (int j = 0; j < n; ++j) {
            const uint8_t *a_row = a + i * lda;
            const uint8_t *b_row = b + j * ldb;
            const int m_group = i / group_m;
            const int n_group = j / group_n;
            float sum = 0.0f;
            for (int g = 0; g < k / group_k; ++g) {
                const float scale = sfa[g * stride_sfa + m_group] * sfb[n_group * stride_sfb + g];
                for (int p = g * group_k; p < (g + 1) * group_k; ++p)
                    sum += g_lut[a_row[p]] * g_lut[b_row[p]] * scale;
            }
            store_out(c, i * ldc + j, sum, out_bf16);
        }
    }
}

void orc_gemm_ref_blockscale(const uint8_t *a, const uint8_t *b, const float *sfa,
                             const float *sfb, void *c, int m, int n, int k, int64_t lda,
                             int64_t ldb, int64_t ldc, int64_t stride_sfa, int64_t stride_sfb,
                             int group_m, int group_n, int group_k, int out_bf16) {
    lut_init();
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            const uint8_t *a_row = a + i * lda;
            const uint8_t *b_row = b + j * ldb;
            const int m_group = i / group_m;
            const int n_group = j / group_n;
            float sum = 0.0f;
            for (int g = 0; g < k / group_k; ++g) {
                const float scale_a = sfa[g * stride_sfa + m_group];
                const float scale_b = sfb[n_group * stride_sfb + g];
                const float scale = scale_a * scale_b;
                const int p_begin = g * group_k;
                const int p_end = p_begin + group_k;
                for (int p = p_begin; p < p_end; ++p)
                    sum += g_lut[a_row[p]] * g_lut[b_row[p]] * scale;
            }
            store_out(c, i * ldc + j, sum, out_bf16);
        }
    }
}

/* Flat-matmul reference: opus_fmm/flatmm_a8w8_gfx950.cc:586-597 -- B is the UNSHUFFLED
 * [K,N] matrix, read as b[p*ldb + j].                                                     */
void orc_gemm_ref_kn(const uint8_t *a, const uint8_t *b_kn, void *c, int m, int n, int k,
                     int64_t lda, int64_t ldb, int64_t ldc, int out_bf16) {
    lut_init();
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int p = 0; p < k; ++p) sum += g_lut[a[i * lda + p]] * g_lut[b_kn[p * ldb + j]];
            store_out(c, i * ldc + j, sum, out_bf16);
        }
    }
}

/* MXFP8 reference (no counterpart in the reference): per 32-wide K block a sequential
 * fp32 partial, multiplied by 2^(ea-127) * 2^(eb-127) and added to the running sum.       */
void orc_gemm_ref_mx(const uint8_t *a, const uint8_t *b, const uint8_t *sfa, const uint8_t *sfb,
                     void *c, int m, int n, int k, int64_t lda, int64_t ldb, int64_t ldc,
                     int out_bf16) {
    lut_init();
    const int KB = k / 32;
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int blk = 0; blk < KB; ++blk) {
                float part = 0.0f;
                for (int p = blk * 32; p < blk * 32 + 32; ++p)
                    part += g_lut[a[i * lda + p]] * g_lut[b[j * ldb + p]];
                const float s = orc_e8m0_to_f32(sfa[(int64_t)i * KB + blk]) *
                                orc_e8m0_to_f32(sfb[(int64_t)j * KB + blk]);
                sum += part * s;
            }
            store_out(c, i * ldc + j, sum, out_bf16);
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* layout transforms                                                                     */
/* ------------------------------------------------------------------------------------ */

/* shuffle_b for 1-byte elements: opus_fmm/flatmm_a8w8_gfx950.cc:638-681 with W_N = 16,
 * W_K = 128, warp 64 -> ItemsPerAccess = min(16, 128/(64/16)) = 16 (:642-647).
 * out[d0][d2][d1][d3] = in[(d2*16+d3)*N + d0*16+d1], dims [N/16][K/16][16][16] (:670-677). */
int orc_shuffle_b(const uint8_t *b_kn, uint8_t *out, int N, int K) {
    if (N % 16 != 0 || K % 16 != 0) return -1;        /* the asserts at :650-651 */
    const int dim0 = N / 16, dim2 = K / 16;
#pragma omp parallel for collapse(2) schedule(static)
    for (int d0 = 0; d0 < dim0; ++d0) {
        for (int d2 = 0; d2 < dim2; ++d2) {
            for (int d1 = 0; d1 < 16; ++d1) {
                const uint8_t *src = b_kn + (size_t)(d2 * 16) * N + (d0 * 16 + d1);
                uint8_t *dst = out + (size_t)d0 * ((size_t)dim2 * 256) + (size_t)d2 * 256 + d1 * 16;
                for (int d3 = 0; d3 < 16; ++d3) dst[d3] = src[(size_t)d3 * N];
            }
        }
    }
    return 0;
}

int orc_unshuffle_b(const uint8_t *flat, uint8_t *b_kn, int N, int K) {
    if (N % 16 != 0 || K % 16 != 0) return -1;
    const int dim2 = K / 16;
#pragma omp parallel for schedule(static)
    for (int kk = 0; kk < K; ++kk) {
        for (int nn = 0; nn < N; ++nn) {
            const size_t off = (size_t)(nn / 16) * ((size_t)dim2 * 256) + (size_t)(kk / 16) * 256 +
                               (size_t)(nn % 16) * 16 + (kk % 16);
            b_kn[(size_t)kk * N + nn] = flat[off];
        }
    }
    return 0;
}

int orc_shuffle_b_nk(const uint8_t *b_nk, uint8_t *out, int N, int K) {
    if (N % 16 != 0 || K % 16 != 0) return -1;
    const int dim2 = K / 16;
#pragma omp parallel for schedule(static)
    for (int nn = 0; nn < N; ++nn) {
        for (int kk = 0; kk < K; ++kk) {
            const size_t off = (size_t)(nn / 16) * ((size_t)dim2 * 256) + (size_t)(kk / 16) * 256 +
                               (size_t)(nn % 16) * 16 + (kk % 16);
            out[off] = b_nk[(size_t)nn * K + kk];
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------ */
/* a16w16 siblings (bf16 operands)                                                       */
/* ------------------------------------------------------------------------------------ */

/* gemm_ref of opus_gemm/gemm_a16w16_8wave.cc:584-595: both operands widened to float, sequential fp32 sum over p,
 * result rounded to bf16 (`static_cast<bf16_t>(sum)`, RNE).  out_bf16 == 0 keeps the fp32 sum.                    */
void orc_gemm_ref_nt_bf16(const uint16_t *a, const uint16_t *b, void *c, int m, int n, int k, int64_t lda,
                          int64_t ldb, int64_t ldc, int out_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int p = 0; p < k; ++p) sum += orc_bf16_to_f32(a[i * lda + p]) * orc_bf16_to_f32(b[j * ldb + p]);
            store_out(c, i * ldc + j, sum, out_bf16);
        }
    }
}

/* gemm_ref of opus_fmm/flatmm_a16w16_gfx950.cc:571-582: B is the UNSHUFFLED [K,N] matrix, b[p*ldb + j].            */
void orc_gemm_ref_kn_bf16(const uint16_t *a, const uint16_t *b_kn, void *c, int m, int n, int k, int64_t lda,
                          int64_t ldb, int64_t ldc, int out_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int p = 0; p < k; ++p) sum += orc_bf16_to_f32(a[i * lda + p]) * orc_bf16_to_f32(b_kn[p * ldb + j]);
            store_out(c, i * ldc + j, sum, out_bf16);
        }
    }
}

/* shuffle_b<bf16> of opus_fmm/flatmm_a16w16_gfx950.cc:623-666: ItemsPerAccess = min(16/sizeof(bf16), K_Warp_Tile/KLane)
 * = 8 for the shipped traits (:627-629), N_Warp_Tile = 16; out[d0][d2][d1][d3] = in[(d2*8+d3)*N + d0*16+d1] with
 * d0 = n/16, d1 = n%16, d2 = k/8, d3 = k%8.  Needs N % 16 == 0 and K % 8 == 0 (:631-633).                          */
int orc_shuffle_b_bf16(const uint16_t *b_kn, uint16_t *out, int N, int K) {
    if (N % 16 != 0 || K % 8 != 0) return -1;
    const int dim0 = N / 16, dim2 = K / 8;
#pragma omp parallel for collapse(2) schedule(static)
    for (int d0 = 0; d0 < dim0; ++d0) {
        for (int d2 = 0; d2 < dim2; ++d2) {
            for (int d1 = 0; d1 < 16; ++d1) {
                const uint16_t *src = b_kn + (size_t)(d2 * 8) * N + (d0 * 16 + d1);
                uint16_t *dst = out + (size_t)d0 * ((size_t)dim2 * 128) + (size_t)d2 * 128 + d1 * 8;
                for (int d3 = 0; d3 < 8; ++d3) dst[d3] = src[(size_t)d3 * N];
            }
        }
    }
    return 0;
}

int orc_unshuffle_b_bf16(const uint16_t *flat, uint16_t *b_kn, int N, int K) {
    if (N % 16 != 0 || K % 8 != 0) return -1;
    const int dim2 = K / 8;
#pragma omp parallel for schedule(static)
    for (int kk = 0; kk < K; ++kk)
        for (int nn = 0; nn < N; ++nn)
            b_kn[(size_t)kk * N + nn] = flat[(size_t)(nn / 16) * ((size_t)dim2 * 128) + (size_t)(kk / 8) * 128 +
                                             (size_t)(nn % 16) * 8 + (kk % 8)];
    return 0;
}

/* ------------------------------------------------------------------------------------ */
/* checker                                                                               */
/* ------------------------------------------------------------------------------------ */

/* valid_vector: opus_gemm/gemm_a8w8_8wave.cc:583-598 -- absolute difference above the
 * threshold is an error, at most 10 are printed, scanning stops at the 10th.              */
int orc_valid_vector(const float *ref, const float *res, int64_t n, float threshold, int verbose) {
    int errors = 0;
    for (int64_t i = 0; i < n; ++i) {
        const float diff = fabsf(ref[i] - res[i]);
        if (diff > threshold || diff != diff) {
            if (errors < 10 && verbose)
                printf("Error at %lld: ref=%.6f, result=%.6f, diff=%.6f\n", (long long)i, ref[i], res[i], diff);
            ++errors;
            if (errors >= 10) break;
        }
    }
    return errors == 0;
}

void orc_max_err(const float *ref, const float *res, int64_t n, float *max_err, float *max_ref) {
    float me = 0.0f, mr = 0.0f;
    int bad = 0;
#pragma omp parallel for reduction(max : me, mr) reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float d = fabsf(ref[i] - res[i]);
        if (d != d) bad++;
        if (d > me) me = d;
        const float r = fabsf(ref[i]);
        if (r > mr) mr = r;
    }
    *max_err = bad ? INFINITY : me;
    *max_ref = mr;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
