// Skinny-M ("decode") A8W8 GEMM for sm_100a: C[M,N] = A[M,K] . W[N,K]^T with M <= 64.
//
// The reference runs its one 256x256x128 tile for every M (opus_fmm/flatmm_a8w8_gfx950.cc:684-687,
// out-of-range rows clamped at :268, stores predicated at :537-541); for M <= 64 that wastes the
// machine, and the job is purely a weight stream.  Here the operands are swapped: a 128(N) x 128(K)
// weight tile is the UMMA M-side operand and the (zero-padded) token block is the UMMA N-side
// operand, so D[n][token] lands in TMEM with one weight row per lane.  One CTA owns one 128-row
// weight panel (optionally one K slice of it) and streams it through a deep TMA ring; HBM is the bound.
//
// Weights are accepted row-major [N,K] (128-byte swizzled tiles) or in the reference's pre-shuffled
// flat layout [N/16][K/16][16][16] (shuffle_b, flatmm_a8w8_gfx950.cc:638-681).  A flat 16x16 block is
// two 8x16-byte UMMA core matrices back to back, so the TMA box {256 B, 8 slabs, 8 k-chunks} arrives
// in shared memory as [k-chunk][slab][256 B]: a canonical un-swizzled K-major operand with
// LBO = 2048 (next core matrix along K) and SBO = 128 (next 8 rows).  No re-layout pass is needed.
//
// Block scales (A: per token per 128 K, [K/128][M]; W: per 128x128 block, [N/128][K/128]) follow
// gemm_a8w8_blockscale_host.cc:66-90: every K group gets a fresh TMEM buffer and is folded into
// register accumulators as acc += partial * (sfa[g][token] * sfb[nblk][g]).
#pragma once

#include "gemm_sm100.cuh"

namespace b200 {

struct DecodeParams {
    CUtensorMap tmap_w;          // weights: 3-D [batch][N][K] swizzled, or the 4-D flat view
    CUtensorMap tmap_x;          // tokens:  3-D [batch][M][K], box 128 x MT, 128-byte swizzle
    void* c;
    float* partial;              // split-K workspace [splits][batch][M][N] fp32 (null when splits == 1)
    const float* sfa;
    const float* sfb;
    const float* scale_a;
    const float* scale_b;
    long long ldc, c_batch;
    long long sfa_stride, sfb_stride, sfa_batch, sfb_batch;
    int m, n, k, batch;
    int tiles_n, kblocks, splits, kb_per_split;
    int out_dtype;
    int inputs_ready;            // the weights are not written by work still in flight on the stream (b200_gemm_flags)
    int* status;
};

// Shared-memory bytes for the staged scales of one CTA.  16-token blocks already reach the ten-stage cap of the ring
// with 34 KB; wider token blocks get one more ring stage from a 24 KB area (config 4: 56 groups x 64 tokens = 14 KB).
__host__ __device__ constexpr int decode_sf_bytes(int mt) { return mt <= 16 ? 34 * 1024 : 24 * 1024; }

template <int MT_, int MODE_, int BLAYOUT_>
struct DecodeCfg {
    static constexpr int MT = MT_, MODE = MODE_, BLAYOUT = BLAYOUT_;
    static constexpr int BNW = 128, BK = 128;
    static constexpr int W_BYTES = BNW * BK;
    static constexpr int X_BYTES = MT * BK;
    static constexpr int STAGE_BYTES = ((W_BYTES + X_BYTES + 1023) / 1024) * 1024;
    // combined scales [K groups of this CTA][MT]; problems whose groups do not fit are split along K by the launcher
    static constexpr int SF_SMEM = decode_sf_bytes(MT_);
    static constexpr int STAGES_RAW = (225 * 1024 - 1024 - SF_SMEM) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + SF_SMEM + 1024;
    // Block-scale mode gives every K group its own TMEM buffer (a fresh accumulator per group), but hands the
    // buffers over in BATCHES of GB groups: one hand-off between the MMA issuer and the epilogue warps costs on
    // the order of a microsecond (commit -> barrier -> TMEM loads -> barrier), far more than the tiny MMAs of a
    // group, so it is paid once per GB groups.  Two batch sets ping-pong: TMEM holds 2 x GB x MT columns.
    static constexpr int GB = 4;
    static constexpr int NBUF = 2;
    static constexpr int TMEM_COLS = NBUF * GB * MT < 32 ? 32 : NBUF * GB * MT;
    static constexpr int THREADS = 192;
    static constexpr int MAX_SF_FLOATS = SF_SMEM / 4;
    static_assert(MT == 16 || MT == 32 || MT == 64, "token block is 16, 32 or 64");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1) decode_a8w8_sm100_kernel(const __grid_constant__ DecodeParams p) {
    constexpr int MT = Cfg::MT, BK = Cfg::BK, BNW = Cfg::BNW, STAGES = Cfg::STAGES, MODE = Cfg::MODE;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
    const uint32_t bar_full0 = smem_base + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_empty0 = bar_full0 + STAGES * 8;
    const uint32_t bar_accf0 = bar_empty0 + STAGES * 8;
    constexpr int NBUF = Cfg::NBUF;
    const uint32_t bar_acce0 = bar_accf0 + NBUF * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * NBUF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* sf_smem = reinterpret_cast<float*>(smem_gen + STAGES * Cfg::STAGE_BYTES + 1024);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // work item: (batch, n tile, k split)
    int w = blockIdx.x;
    const int split = w % p.splits;
    w /= p.splits;
    const int ni = w % p.tiles_n;
    const int b = w / p.tiles_n;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = (kb0 + p.kb_per_split < p.kblocks) ? kb0 + p.kb_per_split : p.kblocks;
    const int nkb = kb1 - kb0;

    // Consecutive decode GEMMs of a serving step are launched with programmatic serialization: this kernel may
    // start while its predecessor is still draining.  When the caller has vouched for the weights
    // (B200_GEMM_INPUTS_READY: resident, not written by anything still in flight) the first ring of weight tiles is
    // requested right away; otherwise the weights, like everything that may be the predecessor's output (tokens,
    // token scales) and every write to C, come after pdl_wait().
    pdl_launch_dependents();
    const int first = nkb < STAGES ? nkb : STAGES;
    auto request_weights = [&](int i) {
        const uint32_t sw = smem_base + i * Cfg::STAGE_BYTES;
        const uint32_t full = bar_full0 + i * 8;
        mbar_arrive_expect_tx(full, Cfg::W_BYTES + Cfg::X_BYTES);
        if constexpr (Cfg::BLAYOUT == BL_NK)
            tma_load_3d(sw, &p.tmap_w, full, (kb0 + i) * BK, ni * BNW, b);
        else
            tma_load_4d(sw, &p.tmap_w, full, 0, ni * (BNW / 16), (kb0 + i) * (BK / 16), b);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full0 + s * 8, 1);
            mbar_init(bar_empty0 + s * 8, 1);
        }
        for (int s = 0; s < NBUF; ++s) {
            mbar_init(bar_accf0 + s * 8, 1);
            mbar_init(bar_acce0 + s * 8, 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        if (p.inputs_ready)
            for (int i = 0; i < first; ++i) request_weights(i);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(tmem_slot), Cfg::TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();
    if (threadIdx.x == 0) {
        for (int i = 0; i < first; ++i) {
            if (!p.inputs_ready) request_weights(i);
            tma_load_3d(smem_base + i * Cfg::STAGE_BYTES + Cfg::W_BYTES, &p.tmap_x, bar_full0 + i * 8, (kb0 + i) * BK, 0, b);
        }
    }

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------ TMA producer ------------------------------
            for (int i = first; i < nkb; ++i) {
                const int kb = kb0 + i;
                const uint32_t s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!mbar_wait_poll<false, 64>(bar_empty0 + s * 8, ph ^ 1, abort_flag, p.status, KSTAT_TIMEOUT_EMPTY)) break;
                const uint32_t sw = smem_base + s * Cfg::STAGE_BYTES;
                const uint32_t sx = sw + Cfg::W_BYTES;
                const uint32_t full = bar_full0 + s * 8;
                mbar_arrive_expect_tx(full, Cfg::W_BYTES + Cfg::X_BYTES);
                if constexpr (Cfg::BLAYOUT == BL_NK)
                    tma_load_3d(sw, &p.tmap_w, full, kb * BK, ni * BNW, b);
                else
                    tma_load_4d(sw, &p.tmap_w, full, 0, ni * (BNW / 16), kb * (BK / 16), b);
                tma_load_3d(sx, &p.tmap_x, full, kb * BK, 0, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ------------------------------ UMMA issuer -------------------------------
            constexpr uint32_t idesc = make_idesc_f8(BNW, MT);
            uint32_t phase = 0;
            bool ok = true;
            if constexpr (MODE != MODE_BLOCK) {
                // the single accumulator buffer is free at kernel start
            }
            constexpr int GBATCH = (MODE == MODE_BLOCK) ? Cfg::GB : 1;
            for (int i0 = 0; i0 < nkb && ok; i0 += GBATCH, ++phase) {
                const int gb = (nkb - i0 < GBATCH) ? nkb - i0 : GBATCH;       // groups in this batch
                const uint32_t set = phase % NBUF;
                if constexpr (MODE == MODE_BLOCK) {
                    const uint32_t aph = (phase / NBUF) & 1;
                    if (!mbar_wait_poll<false, 20>(bar_acce0 + set * 8, aph ^ 1, abort_flag, p.status, KSTAT_TIMEOUT_ACC_E)) {
                        ok = false;
                        break;
                    }
                }
                for (int j = 0; j < gb && ok; ++j) {
                    const int i = i0 + j;
                    const uint32_t s = i % STAGES;
                    const uint32_t ph = (i / STAGES) & 1;
                    if (!mbar_wait_poll<false, 20>(bar_full0 + s * 8, ph, abort_flag, p.status, KSTAT_TIMEOUT_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sw = smem_base + s * Cfg::STAGE_BYTES;
                    const uint32_t sx = sw + Cfg::W_BYTES;
                    const uint32_t tacc = (MODE == MODE_BLOCK) ? tmem_base + (set * Cfg::GB + j) * MT : tmem_base;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) {
                        uint64_t dw;
                        if constexpr (Cfg::BLAYOUT == BL_NK) {
                            dw = make_smem_desc(sw + k * 32, 16, 1024, kSwizzle128B);
                        } else {
                            constexpr uint32_t LBO = (BNW / 16) * 256;
                            dw = make_smem_desc(sw + k * 2 * LBO, LBO, 128, kSwizzleNone);
                        }
                        const uint64_t dx = make_smem_desc(sx + k * 32, 16, 1024, kSwizzle128B);
                        const uint32_t accum = (MODE == MODE_BLOCK) ? (k > 0 ? 1u : 0u) : ((i > 0 || k > 0) ? 1u : 0u);
                        umma_f8<1>(tacc, dw, dx, idesc, accum);
                    }
                    umma_commit<1>(bar_empty0 + s * 8);
                }
                if (!ok) break;
                if constexpr (MODE == MODE_BLOCK) {
                    umma_commit<1>(bar_accf0 + set * 8);
                } else {
                    if (i0 + gb >= nkb) umma_commit<1>(bar_accf0);
                }
            }
        }
    } else {
        // ---------------------------------- epilogue ----------------------------------
        const int quad = warp & 3;
        const int et = (warp - 2) * 32 + lane;             // 0..127 over the four epilogue warps
        const int n_row = ni * BNW + quad * 32 + lane;
        const uint32_t tmem_lane = static_cast<uint32_t>(quad * 32) << 16;
        float acc[MT];
#pragma unroll
        for (int j = 0; j < MT; ++j) acc[j] = 0.0f;
        bool ok = true;

        if constexpr (MODE == MODE_BLOCK) {
            // stage this CTA's combined scales: sf_smem[i*MT + j] = sfa[kb0+i][j] * sfb[ni][kb0+i] (the product the
            // promotion multiplies by, formed once here instead of once per thread and group)
            const float* sfa_g = p.sfa + b * p.sfa_batch;
            const float* sfb_g = p.sfb + b * p.sfb_batch + static_cast<long long>(ni) * p.sfb_stride;
            // (U independent element loads in flight per thread: with one element per round trip this loop cost
            // 0.35 us per 128 x MT elements, 10 us of a 37 us launch at MT = 64.  Eight in flight cover a config-4 panel
            // in 1, 2 and 4 round trips at MT = 16, 32, 64; the wider token blocks therefore keep 16 and 28 in flight --
            // the accumulators are not live yet, so the registers are there.)
            constexpr int U = MT <= 16 ? 8 : (MT <= 32 ? 16 : 28);
            const int total = nkb * MT;
            for (int base = et; base < total; base += 128 * U) {
                float va[U], vb[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int idx = base + u * 128;
                    va[u] = 0.0f;
                    vb[u] = 0.0f;
                    if (idx < total) {
                        const int i = idx / MT, j = idx - i * MT;
                        if (j < p.m) {
                            va[u] = __ldg(sfa_g + static_cast<long long>(kb0 + i) * p.sfa_stride + j);
                            vb[u] = __ldg(sfb_g + kb0 + i);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int idx = base + u * 128;
                    if (idx < total) sf_smem[idx] = va[u] * vb[u];
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");   // epilogue warps only

            // packed accumulators (token pairs); the TMEM loads of group j+1 run behind the FMAs of group j
            unsigned long long acc2[MT / 2];
#pragma unroll
            for (int j = 0; j < MT / 2; ++j) acc2[j] = 0ull;
            float vbuf[2][MT];
            uint32_t phase = 0;
            for (int i0 = 0; i0 < nkb && ok; i0 += Cfg::GB, ++phase) {
                const int gb = (nkb - i0 < Cfg::GB) ? nkb - i0 : Cfg::GB;
                const uint32_t set = phase % NBUF;
                const uint32_t aph = (phase / NBUF) & 1;
                if (!mbar_wait(bar_accf0 + set * 8, aph, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tset = tmem_base + tmem_lane + set * Cfg::GB * MT;
#pragma unroll
                for (int c = 0; c < MT / 16; ++c) tmem_ld16(tset + c * 16, &vbuf[0][c * 16]);
#pragma unroll
                for (int j = 0; j < Cfg::GB; ++j) {
                    if (j < gb) {
                        tmem_ld_wait();                                  // group j is in vbuf[j & 1]
                        if (j + 1 < gb) {
#pragma unroll
                            for (int c = 0; c < MT / 16; ++c) tmem_ld16(tset + (j + 1) * MT + c * 16, &vbuf[(j + 1) & 1][c * 16]);
                        } else {
                            // the whole batch has left TMEM: the set goes back to the MMA issuer
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar_acce0 + set * 8);
                        }
                        const float4* s4 = reinterpret_cast<const float4*>(sf_smem + (i0 + j) * MT);
#pragma unroll
                        for (int jj = 0; jj < MT; jj += 4) {
                            const float4 sc = s4[jj / 4];
                            acc2[jj / 2] = ffma2(pack_f32x2(vbuf[j & 1][jj], vbuf[j & 1][jj + 1]), pack_f32x2(sc.x, sc.y), acc2[jj / 2]);
                            acc2[jj / 2 + 1] = ffma2(pack_f32x2(vbuf[j & 1][jj + 2], vbuf[j & 1][jj + 3]), pack_f32x2(sc.z, sc.w), acc2[jj / 2 + 1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < MT / 2; ++j) unpack_f32x2(acc2[j], acc[2 * j], acc[2 * j + 1]);
        } else {
            if (nkb > 0) {
                if (mbar_wait(bar_accf0, 0, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F)) {
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < MT / 16; ++c) tmem_ld16(tmem_base + tmem_lane + c * 16, &acc[c * 16]);
                    tmem_ld_wait();
                    float tscale = 1.0f;
                    if (p.scale_a) tscale *= __ldg(p.scale_a);
                    if (p.scale_b) tscale *= __ldg(p.scale_b);
#pragma unroll
                    for (int j = 0; j < MT; ++j) acc[j] *= tscale;
                } else {
                    ok = false;
                }
            }
        }

        if (ok && n_row < p.n) {
            if (p.splits > 1) {
                float* dst = p.partial + ((static_cast<size_t>(split) * p.batch + b) * p.m) * p.n + n_row;
#pragma unroll
                for (int j = 0; j < MT; ++j)
                    if (j < p.m) dst[static_cast<size_t>(j) * p.n] = acc[j];
            } else if (p.out_dtype == OUT_BF16) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + static_cast<size_t>(b) * p.c_batch + n_row;
#pragma unroll
                for (int j = 0; j < MT; ++j)
                    if (j < p.m) dst[static_cast<size_t>(j) * p.ldc] = __float2bfloat16_rn(acc[j]);
            } else {
                float* dst = reinterpret_cast<float*>(p.c) + static_cast<size_t>(b) * p.c_batch + n_row;
#pragma unroll
                for (int j = 0; j < MT; ++j)
                    if (j < p.m) dst[static_cast<size_t>(j) * p.ldc] = acc[j];
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
    }
}

// Sums the split-K partials [splits][rows] -> C (fixed order, so the result is deterministic).
__global__ void decode_splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ c, int splits,
                                            long long per_split, int m, int n, long long ldc, long long c_batch,
                                            int out_dtype) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= per_split) return;
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s += partial[k * per_split + i];
    const long long mn = static_cast<long long>(m) * n;
    const long long b = i / mn;
    const long long r = i - b * mn;
    const long long row = r / n, col = r - row * n;
    const long long o = b * c_batch + row * ldc + col;
    if (out_dtype == OUT_BF16) reinterpret_cast<__nv_bfloat16*>(c)[o] = __float2bfloat16_rn(s);
    else reinterpret_cast<float*>(c)[o] = s;
}

}  // namespace b200
