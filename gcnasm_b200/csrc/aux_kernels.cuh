// Memory-bound helper kernels: weight pre-shuffle (and inverse), quantisers, MX scale re-layout and
// the one-thread-per-output checker GEMM.  All are byte/elementwise work bounded by HBM bandwidth;
// they use 16-byte accesses arranged so that both the read and the write side are coalesced.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace b200 {

__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t v) {
    const uint32_t sign = static_cast<uint32_t>(v & 0x80u) << 24;
    const int e = (v >> 3) & 0xF, m = v & 7;
    if (e == 0xF && m == 7) return __uint_as_float(sign | 0x7FC00000u);
    if (e == 0) return __uint_as_float(__float_as_uint(static_cast<float>(m) * (1.0f / 512.0f)) | sign);
    return __uint_as_float(sign | (static_cast<uint32_t>(e + 120) << 23) | (static_cast<uint32_t>(m) << 20));
}
__device__ __forceinline__ float e8m0_to_f32(uint8_t v) {
    if (v == 0xFF) return __uint_as_float(0x7FC00000u);
    if (v == 0) return __uint_as_float(0x00400000u);
    return __uint_as_float(static_cast<uint32_t>(v) << 23);
}

// byte offset of element (n, k) in the flat layout [N/16][K/16][16][16]
// (shuffle_b, opus_fmm/flatmm_a8w8_gfx950.cc:670-677)
__host__ __device__ __forceinline__ long long flat_offset(long long n, long long k, long long K) {
    return (n >> 4) * (K * 16) + (k >> 4) * 256 + (n & 15) * 16 + (k & 15);
}

// ---- [N][K] row-major <-> flat: whole 16-byte k-chunks move as units -------------------------
// block = 256 threads = 16 rows (d1) x 16 k-chunks; reads 16 rows x 256 B, writes 4 KB contiguous.
template <bool kToFlat>
__global__ void shuffle_nk_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long N, long long K) {
    const long long kchunks = K >> 4;
    const long long slab = blockIdx.y;                               // n / 16
    const long long kc = static_cast<long long>(blockIdx.x) * 16 + (threadIdx.x >> 4);
    const int d1 = threadIdx.x & 15;
    if (kc >= kchunks) return;
    const long long nk_idx = (slab * 16 + d1) * kchunks + kc;        // uint4 index in [N][K]
    const long long flat_idx = (slab * kchunks + kc) * 16 + d1;      // uint4 index in the flat image
    if (kToFlat) dst[flat_idx] = __ldg(src + nk_idx);
    else dst[nk_idx] = __ldg(src + flat_idx);
}

// ---- [K][N] row-major <-> flat: a 64(K) x 256(N) byte tile is transposed through shared memory -
template <bool kToFlat>
__global__ void shuffle_kn_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long N,
                                  long long K) {
    __shared__ __align__(16) uint8_t tile[64][256 + 16];
    const long long n0 = static_cast<long long>(blockIdx.x) * 256;
    const long long k0 = static_cast<long long>(blockIdx.y) * 64;
    const int t = threadIdx.x;                                       // 256 threads
    if (kToFlat) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = i * 16 + (t >> 4);
            const int nn = (t & 15) * 16;
            if (k0 + kk < K && n0 + nn < N)
                *reinterpret_cast<uint4*>(&tile[kk][nn]) =
                    __ldg(reinterpret_cast<const uint4*>(src + (k0 + kk) * N + n0 + nn));
        }
        __syncthreads();
        // thread -> (slab = t/16, d1 = t%16); for each of the 4 k-chunks gather 16 bytes down a column
        const int slab = t >> 4, d1 = t & 15;
        if (n0 + slab * 16 < N) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (k0 + c * 16 < K) {
                    uint32_t w[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        w[q] = 0;
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb)
                            w[q] |= static_cast<uint32_t>(tile[c * 16 + q * 4 + bb][slab * 16 + d1]) << (8 * bb);
                    }
                    uint8_t* o = dst + flat_offset(n0 + slab * 16 + d1, k0 + c * 16, K);
                    *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    } else {
        const int slab = t >> 4, d1 = t & 15;
        if (n0 + slab * 16 < N) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (k0 + c * 16 < K) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + flat_offset(n0 + slab * 16 + d1, k0 + c * 16, K)));
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb)
                            tile[c * 16 + q * 4 + bb][slab * 16 + d1] = static_cast<uint8_t>(w[q] >> (8 * bb));
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = i * 16 + (t >> 4);
            const int nn = (t & 15) * 16;
            if (k0 + kk < K && n0 + nn < N)
                *reinterpret_cast<uint4*>(dst + (k0 + kk) * N + n0 + nn) = *reinterpret_cast<const uint4*>(&tile[kk][nn]);
        }
    }
}

// ---- 16-bit elements, [K][N] row-major <-> flat [N/16][K/8][16 n][8 k] (16-byte items of 8 values, the reference's
// shuffle_b for bf16: opus_fmm/flatmm_a16w16_gfx950.cc:623-666).  In bytes the flat image has the geometry of the
// 8-bit one over a [N][2K]-byte matrix.  A 64(K) x 64(N) element tile goes through shared memory.
template <bool kToFlat>
__global__ void shuffle_kn16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, long long N, long long K) {
    __shared__ __align__(16) uint16_t tile[64][64 + 8];
    const long long n0 = static_cast<long long>(blockIdx.x) * 64;
    const long long k0 = static_cast<long long>(blockIdx.y) * 64;
    const int t = threadIdx.x;                                       // 256 threads
    // flat item (n, k8): element offset (n/16)*(K*16) + (k8)*128 + (n%16)*8
    if (kToFlat) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {                                // 64 rows x 8 uint4 (8 values each)
            const int kk = i * 32 + (t >> 3);
            const int nn = (t & 7) * 8;
            if (k0 + kk < K && n0 + nn < N)
                *reinterpret_cast<uint4*>(&tile[kk][nn]) = __ldg(reinterpret_cast<const uint4*>(src + (k0 + kk) * N + n0 + nn));
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {                                // 64 n x 8 k-chunks = 512 items
            const int item = i * 256 + t;
            const int c = item >> 6, nn = item & 63;
            if (n0 + nn < N && k0 + c * 8 < K) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    w[q] = static_cast<uint32_t>(tile[c * 8 + 2 * q][nn]) | (static_cast<uint32_t>(tile[c * 8 + 2 * q + 1][nn]) << 16);
                const long long n = n0 + nn, k8 = (k0 >> 3) + c;
                *reinterpret_cast<uint4*>(dst + (n >> 4) * (K * 16) + k8 * 128 + (n & 15) * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int item = i * 256 + t;
            const int c = item >> 6, nn = item & 63;
            if (n0 + nn < N && k0 + c * 8 < K) {
                const long long n = n0 + nn, k8 = (k0 >> 3) + c;
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (n >> 4) * (K * 16) + k8 * 128 + (n & 15) * 8));
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    tile[c * 8 + 2 * q][nn] = static_cast<uint16_t>(w[q]);
                    tile[c * 8 + 2 * q + 1][nn] = static_cast<uint16_t>(w[q] >> 16);
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int kk = i * 32 + (t >> 3);
            const int nn = (t & 7) * 8;
            if (k0 + kk < K && n0 + nn < N)
                *reinterpret_cast<uint4*>(dst + (k0 + kk) * N + n0 + nn) = *reinterpret_cast<const uint4*>(&tile[kk][nn]);
        }
    }
}

// ---- quantisers ----------------------------------------------------------------------------------
__global__ void cast_e4m3_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, long long count) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long n4 = count >> 2;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
        reinterpret_cast<uint32_t*>(q)[i] = f32x4_to_e4m3x4(v.x, v.y, v.z, v.w);
    }
    for (long long i = (n4 << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        q[i] = f32_to_e4m3(x[i]);
}

// pass 1 of the per-tensor quantiser: amax as the max of non-negative float bit patterns
__global__ void amax_kernel(const float* __restrict__ x, long long count, unsigned int* __restrict__ amax_bits) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    float m = 0.0f;
    const long long n4 = count >> 2;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    for (long long i = (n4 << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        m = fmaxf(m, fabsf(x[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    __shared__ float wm[32];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = (threadIdx.x < (blockDim.x >> 5)) ? wm[threadIdx.x] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(m));
    }
}
// pass 2: scale = amax/448 (1 when amax == 0), q = e4m3(x / scale)
__global__ void quant_tensor_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                                    long long count, const unsigned int* __restrict__ amax_bits) {
    const float amax = __uint_as_float(*amax_bits);
    const float s = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale = s;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long n4 = count >> 2;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
        reinterpret_cast<uint32_t*>(q)[i] =
            f32x4_to_e4m3x4(__fdiv_rn(v.x, s), __fdiv_rn(v.y, s), __fdiv_rn(v.z, s), __fdiv_rn(v.w, s));
    }
    for (long long i = (n4 << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        q[i] = f32_to_e4m3(__fdiv_rn(x[i], s));
}

// one warp per (row, 128-wide K group); sfa is [K/128][M]
__global__ void quant_1x128_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ sfa,
                                   long long M, long long K) {
    const long long KG = K >> 7;
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= M * KG) return;
    const long long row = wid / KG, g = wid - row * KG;
    const float4 v = __ldg(reinterpret_cast<const float4*>(x + row * K + g * 128) + lane);
    float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    const float s = m > 0.0f ? __fdiv_rn(m, 448.0f) : 1.0f;
    reinterpret_cast<uint32_t*>(q + row * K + g * 128)[lane] =
        f32x4_to_e4m3x4(__fdiv_rn(v.x, s), __fdiv_rn(v.y, s), __fdiv_rn(v.z, s), __fdiv_rn(v.w, s));
    if (lane == 0) sfa[g * M + row] = s;
}

// ---- self-test of the bounded waits ---------------------------------------------------------------------------
// Two threads wait on an mbarrier that nothing ever signals, with a short budget.  The first to run out sets the
// CTA's abort flag and the status word; the other leaves through the abort flag or its own budget.  The kernel
// then ends normally: this is how every pipeline wait in the GEMM kernels fails -- with a status, not a hang.
__global__ void selftest_bounded_wait_kernel(int* status, unsigned long long budget_ns, int polling, int* returned) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0 || threadIdx.x == 32) {
        ok = polling ? mbar_wait_poll<false, 64>(smem_u32(&bar), 0, &abort_flag, status, KSTAT_SELFTEST, budget_ns)
                     : mbar_wait<false, 0>(smem_u32(&bar), 0, &abort_flag, status, KSTAT_SELFTEST, budget_ns);
        atomicAdd(returned, ok ? 100 : 1);            // 2 when both waits gave up
    }
    __syncthreads();
}

// ---- HBM bandwidth probe ------------------------------------------------------------------------------------
// Read-only and read+write streams over a buffer, the same two measurements as the reference's
// bandwidth_memread/bandwidth_kernel.cu (memread_kernel :67-92, memcpy_kernel :94-118): persistent grid, 16-byte
// accesses, eight loads in flight per thread, streaming cache hints.  The read kernel folds everything it loads
// into a 32-bit word sum (so that the loads cannot be dropped, and so that a test can check every byte was read).
__global__ void __launch_bounds__(1024) membw_read_kernel(const uint4* __restrict__ src, unsigned long long n16,
                                                          unsigned int* __restrict__ word_sum) {
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    unsigned int acc = 0;
    for (; i + 7 * stride < n16; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __ldcs(src + i + j * stride);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += v[j].x + v[j].y + v[j].z + v[j].w;
    }
    for (; i < n16; i += stride) {
        const uint4 v = __ldcs(src + i);
        acc += v.x + v.y + v.z + v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if ((threadIdx.x & 31) == 0 && acc != 0) atomicAdd(word_sum, acc);
}

__global__ void __launch_bounds__(1024) membw_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                          unsigned long long n16) {
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
    unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 7 * stride < n16; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __ldcs(src + i + j * stride);
#pragma unroll
        for (int j = 0; j < 8; ++j) __stcs(dst + i + j * stride, v[j]);
    }
    for (; i < n16; i += stride) __stcs(dst + i, __ldcs(src + i));
}

// x / s, correctly rounded, for many x and one s.  With r = RN(1/s): q0 = RN(x*r), rem = x - q0*s (exact in an
// FMA), q = RN(q0 + rem*r) is the correctly rounded quotient when nothing overflows or loses bits to underflow
// (Markstein).  `fast` (uniform per group) says s is a normal number of moderate size; the callers guarantee
// |x| <= 448*s*(1+2^-23), and a quotient too small to be exact becomes a zero byte either way.  Everything else takes
// the IEEE division.
__device__ __forceinline__ float div_by_scale(float x, float s, float r, bool fast) {
    if (fast) {
        const float q0 = __fmul_rn(x, r);
        return __fmaf_rn(__fmaf_rn(-q0, s, x), r, q0);
    }
    return __fdiv_rn(x, s);
}

// Fused activation quantiser: bf16 [M][K] (row pitch ldx) -> e4m3 [M][K] (row pitch ldq) + fp32 scales in the
// GEMM's [K/128][M] layout (group pitch stride_sfa), one pass.  A block covers 32 rows x 16 K groups; warp w walks
// the 32 rows of groups g0+2w and g0+2w+1 (512 contiguous bytes per row: lanes 0-15 the first group, 16-31 the
// second, 16 bytes = 8 values per lane) and lane r keeps the two scales of row r, so that the scales leave as two
// 128-byte lines per warp.  Same arithmetic as the fp32 quantiser: scale = amax/448 (1 for an all-zero group),
// q = e4m3(x / scale), both divisions correctly rounded.
__global__ void __launch_bounds__(256) act_quant_bf16_1x128_kernel(const uint16_t* __restrict__ x, long long ldx,
                                                                   uint8_t* __restrict__ q, long long ldq,
                                                                   float* __restrict__ sfa, long long stride_sfa,
                                                                   long long M, long long K) {
    const long long KG = K >> 7;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gpair = (static_cast<long long>(blockIdx.x) * 8 + warp) * 2;     // first of the warp's two groups
    const long long row0 = static_cast<long long>(blockIdx.y) * 32;
    if (gpair >= KG) return;
    const bool live = gpair + (lane >> 4) < KG;                  // the second group may not exist
    const int nrows = (M - row0) < 32 ? static_cast<int>(M - row0) : 32;
    float my_a = 1.0f, my_b = 1.0f;
#pragma unroll 1
    for (int r0 = 0; r0 < nrows; r0 += 4) {
        uint4 raw[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            raw[i] = make_uint4(0u, 0u, 0u, 0u);
            if (live && r0 + i < nrows)
                raw[i] = __ldg(reinterpret_cast<const uint4*>(x + (row0 + r0 + i) * ldx + gpair * 128) + lane);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (r0 + i >= nrows) break;                                  // uniform across the warp
            const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
            float v[8];
            float m = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
                m = fmaxf(m, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            const float sc = m > 0.0f ? __fdiv_rn(m, 448.0f) : 1.0f;     // one per half-warp
            const float rc = __frcp_rn(sc);
            const bool fast = sc >= 0x1p-100f && sc <= 0x1p100f;
            auto dv = [&](float val) { return div_by_scale(val, sc, rc, fast); };
            uint2 out;
            out.x = f32x4_to_e4m3x4(dv(v[0]), dv(v[1]), dv(v[2]), dv(v[3]));
            out.y = f32x4_to_e4m3x4(dv(v[4]), dv(v[5]), dv(v[6]), dv(v[7]));
            if (live) reinterpret_cast<uint2*>(q + (row0 + r0 + i) * ldq + gpair * 128)[lane] = out;
            const float sa = __shfl_sync(0xFFFFFFFFu, sc, 0), sb = __shfl_sync(0xFFFFFFFFu, sc, 16);
            if (lane == r0 + i) {
                my_a = sa;
                my_b = sb;
            }
        }
    }
    if (lane < nrows) {
        sfa[gpair * stride_sfa + row0 + lane] = my_a;
        if (gpair + 1 < KG) sfa[(gpair + 1) * stride_sfa + row0 + lane] = my_b;
    }
}

// Fused MX activation quantiser: bf16 [rows][K] -> e4m3 [rows][K] + E8M0 scales written straight into the
// tensor-core atom order [K/128][ceil(rows/128)][32][4][4] (what quant_mx32 followed by mx_sf_relayout produce).
// Same block shape as above: warp w owns K group g0+w of the block's 32 rows; eight lanes share one 32-wide
// scale block; lane r keeps the four scale bytes of row r as one word.  Rows of the last atom beyond `rows`
// get 127 (scale 1.0).  grid.y covers ceil(rows/128)*4 row blocks.
__global__ void __launch_bounds__(256) act_quant_bf16_mx32_kernel(const uint16_t* __restrict__ x, long long ldx,
                                                                  uint8_t* __restrict__ q, long long ldq,
                                                                  uint32_t* __restrict__ atoms, long long rows,
                                                                  long long K) {
    const long long KG = K >> 7;
    const long long R128 = (rows + 127) >> 7;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long g = static_cast<long long>(blockIdx.x) * 8 + warp;
    const long long row0 = static_cast<long long>(blockIdx.y) * 32;
    if (g >= KG) return;
    const int nrows = row0 >= rows ? 0 : ((rows - row0) < 32 ? static_cast<int>(rows - row0) : 32);
    uint32_t my_word = 0x7F7F7F7Fu;
#pragma unroll 1
    for (int r0 = 0; r0 < nrows; r0 += 4) {
        uint2 raw[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            raw[i] = make_uint2(0u, 0u);
            if (r0 + i < nrows) raw[i] = __ldg(reinterpret_cast<const uint2*>(x + (row0 + r0 + i) * ldx + g * 128) + lane);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (r0 + i >= nrows) break;                                  // uniform across the warp
            const float a = __uint_as_float(raw[i].x << 16), b = __uint_as_float(raw[i].x & 0xFFFF0000u);
            const float c = __uint_as_float(raw[i].y << 16), d = __uint_as_float(raw[i].y & 0xFFFF0000u);
            float m = fmaxf(fmaxf(fabsf(a), fabsf(b)), fmaxf(fabsf(c), fabsf(d)));
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            uint32_t packed;
            int byte = 0;
            if (!(m > 0.0f)) {
                packed = ((__float_as_uint(a) >> 24) & 0x80u) | (((__float_as_uint(b) >> 24) & 0x80u) << 8) |
                         (((__float_as_uint(c) >> 24) & 0x80u) << 16) | (((__float_as_uint(d) >> 24) & 0x80u) << 24);
            } else {
                byte = ilogbf(m) - 8 + 127;
                byte = byte < 0 ? 0 : (byte > 254 ? 254 : byte);
                const int e = byte - 127;
                packed = f32x4_to_e4m3x4(scalbnf(a, -e), scalbnf(b, -e), scalbnf(c, -e), scalbnf(d, -e));
            }
            reinterpret_cast<uint32_t*>(q + (row0 + r0 + i) * ldq + g * 128)[lane] = packed;
            const uint32_t word = static_cast<uint32_t>(__shfl_sync(0xFFFFFFFFu, byte, 0)) |
                                  (static_cast<uint32_t>(__shfl_sync(0xFFFFFFFFu, byte, 8)) << 8) |
                                  (static_cast<uint32_t>(__shfl_sync(0xFFFFFFFFu, byte, 16)) << 16) |
                                  (static_cast<uint32_t>(__shfl_sync(0xFFFFFFFFu, byte, 24)) << 24);
            if (lane == r0 + i) my_word = word;
        }
    }
    const long long row = row0 + lane;                                   // row0 is a multiple of 32
    atoms[(g * R128 + (row >> 7)) * 128 + lane * 4 + ((row & 127) >> 5)] = my_word;
}

// one 256-thread block per 128x128 block; the block stays in registers between amax and quantise
__global__ void quant_128x128_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ sfb,
                                     long long N, long long K) {
    const long long KG = K >> 7;
    const long long nb = blockIdx.y, g = blockIdx.x;
    const int t = threadIdx.x;
    const int c4 = t & 31;                    // float4 column within the 128-wide row
    const int r0 = t >> 5;                    // 8 row phases
    float4 v[16];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const long long row = nb * 128 + r0 + i * 8;
        v[i] = __ldg(reinterpret_cast<const float4*>(x + row * K + g * 128) + c4);
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    __shared__ float wm[8];
    if ((t & 31) == 0) wm[t >> 5] = m;
    __syncthreads();
    m = wm[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, wm[i]);
    const float s = m > 0.0f ? __fdiv_rn(m, 448.0f) : 1.0f;
    if (t == 0) sfb[nb * KG + g] = s;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const long long row = nb * 128 + r0 + i * 8;
        reinterpret_cast<uint32_t*>(q + row * K + g * 128)[c4] =
            f32x4_to_e4m3x4(__fdiv_rn(v[i].x, s), __fdiv_rn(v[i].y, s), __fdiv_rn(v[i].z, s), __fdiv_rn(v[i].w, s));
    }
}

// 8 lanes per 1x32 block; sf is [rows][K/32] E8M0
__global__ void quant_mx32_kernel(const float* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                  long long rows, long long K) {
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long blk = tid >> 3;
    const int sub = static_cast<int>(tid & 7);
    const long long KB = K >> 5;
    const bool live = blk < rows * KB;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) v = __ldg(reinterpret_cast<const float4*>(x + blk * 32) + sub);
    float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (!live) return;
    if (!(m > 0.0f)) {
        reinterpret_cast<uint32_t*>(q + blk * 32)[sub] =
            ((__float_as_uint(v.x) >> 24) & 0x80u) | (((__float_as_uint(v.y) >> 24) & 0x80u) << 8) |
            (((__float_as_uint(v.z) >> 24) & 0x80u) << 16) | (((__float_as_uint(v.w) >> 24) & 0x80u) << 24);
        if (sub == 0) sf[blk] = 0;
        return;
    }
    int byte = ilogbf(m) - 8 + 127;
    byte = byte < 0 ? 0 : (byte > 254 ? 254 : byte);
    const int e = byte - 127;
    reinterpret_cast<uint32_t*>(q + blk * 32)[sub] =
        f32x4_to_e4m3x4(scalbnf(v.x, -e), scalbnf(v.y, -e), scalbnf(v.z, -e), scalbnf(v.w, -e));
    if (sub == 0) sf[blk] = static_cast<uint8_t>(byte);
}

// logical E8M0 [rows][K/32] -> atoms [K/128][R128][32][4][4]: byte (r%32)*16 + ((r%128)/32)*4 + (kb32%4)
// one thread per output 32-bit word (the 4 k-blocks of one row of one atom)
__global__ void mx_sf_relayout_kernel(const uint8_t* __restrict__ sf, uint32_t* __restrict__ atoms, long long rows,
                                      long long K) {
    const long long R128 = (rows + 127) >> 7;
    const long long KB128 = K >> 7;
    const long long KB32 = K >> 5;
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= KB128 * R128 * 128) return;
    const long long atom = i >> 7;
    const int w = static_cast<int>(i & 127);                 // word within atom = (r%32)*4 + (r%128)/32
    const int r_in = (w & 3) * 32 + (w >> 2);
    const long long kb = atom / R128, rb = atom - kb * R128;
    const long long r = rb * 128 + r_in;
    uint32_t word = 0x7F7F7F7Fu;
    if (r < rows) word = __ldg(reinterpret_cast<const uint32_t*>(sf + r * KB32 + kb * 4));
    atoms[i] = word;
}

// ---- checker GEMM: one thread per output element, the host gemm_ref loops on the device -----------
struct SimpleParams {
    const uint8_t* a;
    const uint8_t* b;
    void* c;
    const void* sfa;
    const void* sfb;
    const float* scale_a;
    const float* scale_b;
    long long m, n, k, batch;
    long long lda, ldb, ldc, a_batch, b_batch, c_batch;
    long long sfa_stride, sfb_stride, sfa_batch, sfb_batch;
    int scale_mode, b_layout, out_dtype;
};

__global__ void gemm_simple_kernel(const SimpleParams p) {
    __shared__ float lut[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = e4m3_to_f32(static_cast<uint8_t>(i));
    __syncthreads();
    const long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long i = blockIdx.y;
    const long long b = blockIdx.z;
    if (j >= p.n) return;
    const uint8_t* a_row = p.a + b * p.a_batch + i * p.lda;
    const uint8_t* bb = p.b + b * p.b_batch;
    float sum = 0.0f;
    auto bval = [&](long long kk) -> float {
        return lut[p.b_layout == 0 ? bb[j * p.ldb + kk] : bb[flat_offset(j, kk, p.k)]];
    };
    if (p.scale_mode == 2) {
        const float* sfa = reinterpret_cast<const float*>(p.sfa) + b * p.sfa_batch;
        const float* sfb = reinterpret_cast<const float*>(p.sfb) + b * p.sfb_batch;
        for (long long g = 0; g < p.k / 128; ++g) {
            const float scale = __fmul_rn(sfa[g * p.sfa_stride + i], sfb[(j / 128) * p.sfb_stride + g]);
            for (long long kk = g * 128; kk < (g + 1) * 128; ++kk)
                sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(lut[a_row[kk]], bval(kk)), scale));
        }
    } else if (p.scale_mode == 3) {
        const uint8_t* sfa = reinterpret_cast<const uint8_t*>(p.sfa) + b * p.sfa_batch;
        const uint8_t* sfb = reinterpret_cast<const uint8_t*>(p.sfb) + b * p.sfb_batch;
        for (long long blk = 0; blk < p.k / 32; ++blk) {
            float part = 0.0f;
            for (long long kk = blk * 32; kk < blk * 32 + 32; ++kk)
                part = __fadd_rn(part, __fmul_rn(lut[a_row[kk]], bval(kk)));
            const long long kb = blk >> 2;
            const int k4 = static_cast<int>(blk & 3);
            const uint8_t ea = sfa[((kb * p.sfa_stride + (i >> 7)) << 9) + (i & 31) * 16 + ((i & 127) >> 5) * 4 + k4];
            const uint8_t eb = sfb[((kb * p.sfb_stride + (j >> 7)) << 9) + (j & 31) * 16 + ((j & 127) >> 5) * 4 + k4];
            sum = __fadd_rn(sum, __fmul_rn(part, __fmul_rn(e8m0_to_f32(ea), e8m0_to_f32(eb))));
        }
    } else {
        for (long long kk = 0; kk < p.k; ++kk) sum = __fadd_rn(sum, __fmul_rn(lut[a_row[kk]], bval(kk)));
        if (p.scale_mode == 1) {
            const float sa = p.scale_a ? *p.scale_a : 1.0f, sb = p.scale_b ? *p.scale_b : 1.0f;
            if (!(sa == 1.0f && sb == 1.0f)) sum = __fmul_rn(sum, __fmul_rn(sa, sb));
        }
    }
    const long long o = b * p.c_batch + i * p.ldc + j;
    if (p.out_dtype == 1) reinterpret_cast<__nv_bfloat16*>(p.c)[o] = __float2bfloat16_rn(sum);
    else reinterpret_cast<float*>(p.c)[o] = sum;
}

}  // namespace b200
