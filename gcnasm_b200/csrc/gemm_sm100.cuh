// A8W8 FP8 (E4M3) NT GEMM for sm_100a: C[M,N] = A[M,K] . B[N,K]^T with fp32 accumulation.
//
// Replaces the device kernels of the reference (gemm_a8w8_kernel, opus_gemm/gemm_a8w8_8wave.cc:261-563;
// gemm_a8w8_blockscale_kernel + scale_c_tile, block_scale_gemm/gemm_a8w8_blockscale_kernel_template.hpp:24-39,
// 203-591; flatmm_kernel for M above the skinny range, opus_fmm/flatmm_a8w8_gfx950.cc:243-548).
//
// One persistent CTA per SM, 12 warps:
//   warp 0      TMA producer   (one elected lane)  global -> shared ring, mbarrier complete_tx
//   warp 1      UMMA issuer    (one elected lane)  tcgen05.mma kind::f8f6f4 / kind::mxf8f6f4, TMEM alloc
//   warps 2-3   idle (they exist so that register re-allocation can work on whole warpgroups)
//   warps 4-11  epilogue: TMEM -> registers -> scale -> global
// TMEM holds two accumulator buffers of BN columns.  Per-tensor / unscaled / MX modes accumulate a
// whole tile in one buffer while the epilogue drains the other.  Block-scale mode gives every
// 128-wide K group a FRESH buffer (the reference does the same with a fresh MFMA accumulator,
// kernel_template.hpp:317,334) and the epilogue warps fold it into register accumulators with
// acc += partial * (sfa[g][row] * sfb[nblk][g]) -- the analogue of scale_c_tile.
#pragma once

#include "sm100_ptx.cuh"

namespace b200 {

// MODE_ACC16: the accumulate-mode pipeline on bf16 operands (every K quantity counted in bytes by the launcher)
enum : int { MODE_ACC = 0, MODE_BLOCK = 1, MODE_MX = 2, MODE_ACC16 = 3 };
enum : int { BL_NK = 0, BL_FLAT = 1 };
enum : int { OUT_F32 = 0, OUT_BF16 = 1 };

struct GemmParams {
    CUtensorMap tmap_a;          // u8 [batch][M][K], box 128 x 128, 128-byte swizzle
    CUtensorMap tmap_b;          // u8 [batch][N][K] (same box) or the flat 4-D view
    CUtensorMap tmap_sfa;        // pair kernels, MX: scale atoms as u8 [atoms*2][256], box 256 x 2
    CUtensorMap tmap_sfb;        // pair kernels, MX: box 256 x 2*atoms
    CUtensorMap tmap_c;          // pair kernels, block-scale, bf16 out: C [batch][M][N], box 64 x 32, 128-byte swizzle
    void* c;
    const float* sfa;            // block: fp32 [K/128][M];   MX: E8M0 atoms (uint8, see sf_relayout)
    const float* sfb;            // block: fp32 [N/128][K/128]; MX: E8M0 atoms
    const float* scale_a;        // per-tensor device scalars (may be null -> 1)
    const float* scale_b;
    long long ldc, c_batch;
    long long sfa_stride, sfb_stride, sfa_batch, sfb_batch;
    int m, n, k, batch;
    int tiles_m, tiles_n, tiles_total, kblocks;
    int out_dtype;
    int c_tma;                   // block-scale pair kernels: finished tiles leave through TMA bulk stores
    int inputs_ready;            // pair kernels: operands do not depend on the previous kernel (see b200_gemm_flags)
    int b_shared;                // pair kernels: every batch multiplies by the same B (B is read at batch coordinate 0)
    int batch_epoch;             // pair kernels: value a batch's ready word must have reached (with batch_ready)
    const int* batch_ready;      // pair kernels: one ready word per batch, or null
    // pair kernels, block-scale, 256 x 256 tiles, row-major B: the tiles from tail_first on (the last, partly filled
    // round of the persistent schedule) are each computed as tail_split (2 or 4) column parts of 256 / tail_split
    // columns by as many CTA pairs -- narrower MMAs over the full K, so every output element is summed exactly as in a
    // whole tile.  tmap_b_tail is B with a box of 128 / tail_split rows.  tail_split == 0: whole tiles only.
    CUtensorMap tmap_b_tail;
    int tail_first, tail_split;
    int* status;
};

// Work unit u of a pair kernel -> its tile and column part (part < 0: the whole tile).
__device__ __forceinline__ void unit_coords(const GemmParams& p, int u, int& t, int& part) {
    if (p.tail_split == 0 || u < p.tail_first) {
        t = u;
        part = -1;
    } else {
        const int r = u - p.tail_first;
        t = p.tail_first + r / p.tail_split;
        part = r - (t - p.tail_first) * p.tail_split;
    }
}

template <int BN_, int MODE_, int BLAYOUT_>
struct GemmCfg {
    static constexpr bool AB16 = MODE_ == MODE_ACC16;               // bf16 operands: same bytes, kind::f16 MMAs
    static constexpr int BM = 128, BN = BN_, BK = 128, MODE = AB16 ? MODE_ACC : MODE_, BLAYOUT = BLAYOUT_;
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = BN * BK;
    static constexpr int SFA_BYTES = (MODE == MODE_MX) ? 512 : 0;
    static constexpr int SFB_ATOMS = (BN + 127) / 128;
    static constexpr int SFB_BYTES = (MODE == MODE_MX) ? SFB_ATOMS * 512 : 0;
    static constexpr int STAGE_BYTES = ((A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + 1023) / 1024) * 1024;
    static constexpr int SMEM_BUDGET = 225 * 1024;
    static constexpr int STAGES_RAW = (SMEM_BUDGET - 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*barriers*/ + 1024 /*alignment slack*/;
    static constexpr int ACC_COLS = 2 * BN;
    static constexpr int SF_COLS = (MODE == MODE_MX) ? 4 + 4 * SFB_ATOMS : 0;
    static constexpr int TMEM_COLS = (ACC_COLS + SF_COLS) <= 32 ? 32 : (ACC_COLS + SF_COLS) <= 64 ? 64
                                   : (ACC_COLS + SF_COLS) <= 128 ? 128 : (ACC_COLS + SF_COLS) <= 256 ? 256 : 512;
    static constexpr int NCH = BN / 2;              // columns owned by one epilogue thread
    static constexpr int THREADS = 384;
    static_assert(ACC_COLS + SF_COLS <= 512, "TMEM overflow");
    static_assert(BN % 32 == 0 && BN <= 256, "BN must be a multiple of 32, at most 256");
    static_assert(STAGES >= 3, "ring too shallow");
};

// tile index -> (batch, m tile, n tile): groups of 8 M tiles walk N, so that the tiles resident at
// one time share few A row panels and few B column panels in L2.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int t, int& b, int& mi, int& ni) {
    const int per_batch = p.tiles_m * p.tiles_n;
    b = t / per_batch;
    int r = t - b * per_batch;
    constexpr int GM = 8;
    const int group_sz = GM * p.tiles_n;
    const int grp = r / group_sz;
    const int first_m = grp * GM;
    const int rows = (p.tiles_m - first_m) < GM ? (p.tiles_m - first_m) : GM;
    const int in_grp = r - grp * group_sz;
    mi = first_m + in_grp % rows;
    ni = in_grp / rows;
}

// Store `cnt` consecutive output columns of one row (16-byte vectors when aligned and in range).
template <int CNT>
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, void* crow, int col0, const float* v,
                                                bool vec_ok) {
    if (p.out_dtype == OUT_BF16) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(crow) + col0;
        if (vec_ok && col0 + CNT <= p.n) {
#pragma unroll
            for (int j = 0; j < CNT; j += 8) {
                uint4 w;
                w.x = pack_bf16x2(v[j + 0], v[j + 1]);
                w.y = pack_bf16x2(v[j + 2], v[j + 3]);
                w.z = pack_bf16x2(v[j + 4], v[j + 5]);
                w.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < CNT; ++j)
                if (col0 + j < p.n) dst[j] = __float2bfloat16_rn(v[j]);
        }
    } else {
        float* dst = reinterpret_cast<float*>(crow) + col0;
        if (vec_ok && col0 + CNT <= p.n) {
#pragma unroll
            for (int j = 0; j < CNT; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < CNT; ++j)
                if (col0 + j < p.n) dst[j] = v[j];
        }
    }
}

// Coalesced store of one warp's 32-row x CNT-column chunk.  Every lane holds CNT consecutive columns of ITS row
// (the TMEM load layout), so a direct store would touch 32 different rows per instruction.  The chunk is written
// to a warp-private shared-memory buffer (row pitch 80 B: 16-byte accesses stay conflict-free) and read back
// transposed, so that one store instruction covers whole 32- or 64-byte row segments.
// `row0` is the output row of lane 0; `stage` is this warp's 2560-byte buffer; CNT * element size is 32 or 64.
static constexpr int kOutStagePitch = 80;
static constexpr int kOutStageBytesPerWarp = 32 * kOutStagePitch;
template <int CNT>
__device__ __forceinline__ void store_chunk_coalesced(const GemmParams& p, uint8_t* cbatch, uint8_t* stage, int row0,
                                                      int col0, const float* v, int lane, bool vec_ok) {
    const bool bf16 = p.out_dtype == OUT_BF16;
    const int esz = bf16 ? 2 : 4;
    if (!(vec_ok && col0 + CNT <= p.n)) {
        // ragged edge or unaligned output: per-lane path
        const int row = row0 + lane;
        if (row < p.m) store_row_chunk<CNT>(p, cbatch + static_cast<size_t>(row) * p.ldc * esz, col0, v, false);
        return;
    }
    uint8_t* mine = stage + lane * kOutStagePitch;
    int row_bytes;
    if (bf16) {
        row_bytes = CNT * 2;
#pragma unroll
        for (int j = 0; j < CNT; j += 8) {
            uint4 w;
            w.x = pack_bf16x2(v[j + 0], v[j + 1]);
            w.y = pack_bf16x2(v[j + 2], v[j + 3]);
            w.z = pack_bf16x2(v[j + 4], v[j + 5]);
            w.w = pack_bf16x2(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(mine + j * 2) = w;
        }
    } else {
        row_bytes = CNT * 4;
#pragma unroll
        for (int j = 0; j < CNT; j += 4)
            *reinterpret_cast<float4*>(mine + j * 4) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
    __syncwarp();
    const int chunks = row_bytes >> 4;                  // 16-byte pieces per row: 2, 4 or 8
    const int rows_per_pass = 32 / chunks;
    const int c = lane % chunks, r_in = lane / chunks;
    for (int r = r_in; r < 32; r += rows_per_pass) {
        const uint4 w = *reinterpret_cast<const uint4*>(stage + r * kOutStagePitch + c * 16);
        const int row = row0 + r;
        if (row < p.m)
            *reinterpret_cast<uint4*>(cbatch + (static_cast<size_t>(row) * p.ldc + col0) * esz + c * 16) = w;
    }
    __syncwarp();
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1) gemm_a8w8_sm100_kernel(const __grid_constant__ GemmParams p) {
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES, MODE = Cfg::MODE;
    constexpr int NCH = Cfg::NCH;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // barrier block sits after the ring
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
    const uint32_t bar_full0 = smem_base + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_empty0 = bar_full0 + STAGES * 8;
    const uint32_t bar_accf0 = bar_empty0 + STAGES * 8;
    const uint32_t bar_acce0 = bar_accf0 + 2 * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full0 + s * 8, 1);
            mbar_init(bar_empty0 + s * 8, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_accf0 + s * 8, 1);
            mbar_init(bar_acce0 + s * 8, 8);     // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(tmem_slot), Cfg::TMEM_COLS);
        tmem_relinquish<1>();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&p.tmap_a);
        prefetch_tmap(&p.tmap_b);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int groups = (MODE == MODE_BLOCK) ? p.kblocks : 1;          // accumulator phases per tile
    const int kb_per_group = (MODE == MODE_BLOCK) ? 1 : p.kblocks;

    if (warp < 4) {
        setmaxnreg_dec<40>();
        if (warp == 0 && lane == 0) {
            // ------------------------------ TMA producer ------------------------------
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.tiles_total && ok; t += gridDim.x) {
                int b, mi, ni;
                tile_coords(p, t, b, mi, ni);
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(bar_empty0 + s * 8, ph ^ 1, abort_flag, p.status, KSTAT_TIMEOUT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    const uint32_t full = bar_full0 + s * 8;
                    mbar_arrive_expect_tx(full, Cfg::A_BYTES + Cfg::B_BYTES + Cfg::SFA_BYTES + Cfg::SFB_BYTES);
                    tma_load_3d(sa, &p.tmap_a, full, kb * BK, mi * BM, b);
                    if constexpr (Cfg::BLAYOUT == BL_NK)
                        tma_load_3d(sb, &p.tmap_b, full, kb * BK, ni * BN, b);
                    else
                        tma_load_4d(sb, &p.tmap_b, full, 0, ni * (BN / 16), kb * (BK / 16), b);
                    if constexpr (MODE == MODE_MX) {
                        // scale-factor atoms: [batch][K/128][rows/128][512 B]
                        const uint8_t* sfa = reinterpret_cast<const uint8_t*>(p.sfa) + b * p.sfa_batch +
                                             (static_cast<long long>(kb) * p.sfa_stride + mi) * 512;
                        const uint8_t* sfb = reinterpret_cast<const uint8_t*>(p.sfb) + b * p.sfb_batch +
                                             (static_cast<long long>(kb) * p.sfb_stride + ni * Cfg::SFB_ATOMS) * 512;
                        bulk_load(sb + Cfg::B_BYTES, sfa, 512, full);
                        bulk_load(sb + Cfg::B_BYTES + 512, sfb, Cfg::SFB_BYTES, full);
                    }
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ------------------------------ UMMA issuer -------------------------------
            uint32_t it = 0, phase = 0;
            bool ok = true;
            constexpr uint32_t idesc = make_idesc_f8(BM, BN);
            for (int t = blockIdx.x; t < p.tiles_total && ok; t += gridDim.x) {
                for (int g = 0; g < groups && ok; ++g, ++phase) {
                    const uint32_t as = phase & 1;
                    const uint32_t aph = (phase >> 1) & 1;
                    if (!mbar_wait(bar_acce0 + as * 8, aph ^ 1, abort_flag, p.status, KSTAT_TIMEOUT_ACC_E)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t tacc = tmem_base + as * BN;
                    for (int kb = 0; kb < kb_per_group; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!mbar_wait(bar_full0 + s * 8, ph, abort_flag, p.status, KSTAT_TIMEOUT_FULL)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
                        const uint32_t sb = sa + Cfg::A_BYTES;
                        if constexpr (MODE == MODE_MX) {
                            const uint32_t tsf = tmem_base + Cfg::ACC_COLS;
                            tmem_cp_sf<1>(tsf, make_smem_desc(sb + Cfg::B_BYTES, 0, 128, kSwizzleNone));
#pragma unroll
                            for (int a = 0; a < Cfg::SFB_ATOMS; ++a)
                                tmem_cp_sf<1>(tsf + 4 + 4 * a,
                                              make_smem_desc(sb + Cfg::B_BYTES + 512 + 512 * a, 0, 128, kSwizzleNone));
                        }
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k) {
                            const uint64_t da = make_smem_desc(sa + k * 32, 16, 1024, kSwizzle128B);
                            uint64_t db;
                            if constexpr (Cfg::BLAYOUT == BL_NK) {
                                db = make_smem_desc(sb + k * 32, 16, 1024, kSwizzle128B);
                            } else {
                                constexpr uint32_t LBO = (BN / 16) * 256;
                                db = make_smem_desc(sb + k * 2 * LBO, LBO, 128, kSwizzleNone);
                            }
                            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
                            if constexpr (MODE == MODE_MX) {
                                const uint32_t tsf = tmem_base + Cfg::ACC_COLS;
                                umma_mxf8<1>(tacc, da, db, make_idesc_mxf8(BM, BN, k, k), accum, tsf, tsf + 4);
                            } else {
                                if constexpr (Cfg::AB16) umma_f16<1>(tacc, da, db, make_idesc_bf16(BM, BN), accum);
                                else umma_f8<1>(tacc, da, db, idesc, accum);
                            }
                        }
                        umma_commit<1>(bar_empty0 + s * 8);      // stage free once these MMAs retire
                    }
                    if (ok) umma_commit<1>(bar_accf0 + as * 8);  // accumulator phase complete
                }
            }
        }
    } else {
        // ---------------------------------- epilogue ----------------------------------
        setmaxnreg_inc<232>();
        const int ew = warp - 4;
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may touch
        const int half = ew >> 2;                  // which BN/2 column range
        const int row_in_tile = quad * 32 + lane;
        const uint32_t tmem_lane = static_cast<uint32_t>(quad * 32) << 16;
        const size_t esz = (p.out_dtype == OUT_BF16) ? 2 : 4;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && ((p.ldc * esz) % 16 == 0) &&
                            ((p.c_batch * esz) % 16 == 0);
        float tscale = 1.0f;
        if constexpr (MODE == MODE_ACC) {
            if (p.scale_a) tscale *= __ldg(p.scale_a);
            if (p.scale_b) tscale *= __ldg(p.scale_b);
        }
        uint32_t phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.tiles_total && ok; t += gridDim.x) {
            int b, mi, ni;
            tile_coords(p, t, b, mi, ni);
            const int row = mi * BM + row_in_tile;
            const int col_base = ni * BN + half * NCH;
            uint8_t* crow = reinterpret_cast<uint8_t*>(p.c) +
                            (static_cast<size_t>(b) * p.c_batch + static_cast<size_t>(row) * p.ldc) * esz;

            if constexpr (MODE == MODE_BLOCK) {
                float acc[NCH];
#pragma unroll
                for (int j = 0; j < NCH; ++j) acc[j] = 0.0f;
                const float* sfa_p = p.sfa + b * p.sfa_batch + (row < p.m ? row : 0);
                const float* sfb_p = p.sfb + b * p.sfb_batch + static_cast<long long>(col_base / 128) * p.sfb_stride;
                const bool col_ok = col_base < p.n;
                float sa_next = __ldg(sfa_p);
                float sb_next = col_ok ? __ldg(sfb_p) : 0.0f;
                for (int g = 0; g < groups; ++g, ++phase) {
                    const float sc = sa_next * sb_next;
                    if (g + 1 < groups) {
                        sa_next = __ldg(sfa_p + static_cast<long long>(g + 1) * p.sfa_stride);
                        sb_next = col_ok ? __ldg(sfb_p + g + 1) : 0.0f;
                    }
                    const uint32_t as = phase & 1;
                    const uint32_t aph = (phase >> 1) & 1;
                    if (!mbar_wait(bar_accf0 + as * 8, aph, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + tmem_lane + as * BN + half * NCH;
                    float v[2][32];
                    tmem_ld32(taddr, v[0]);
#pragma unroll
                    for (int c = 0; c < NCH / 32; ++c) {
                        tmem_ld_wait();
                        if (c + 1 < NCH / 32) tmem_ld32(taddr + (c + 1) * 32, v[(c + 1) & 1]);
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(v[c & 1][j], sc, acc[c * 32 + j]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acce0 + as * 8);
                }
                if (ok && row < p.m) {
#pragma unroll
                    for (int c = 0; c < NCH / 32; ++c) store_row_chunk<32>(p, crow, col_base + c * 32, &acc[c * 32], vec_ok);
                }
            } else {
                const uint32_t as = phase & 1;
                const uint32_t aph = (phase >> 1) & 1;
                if (!mbar_wait(bar_accf0 + as * 8, aph, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + tmem_lane + as * BN + half * NCH;
                float v[2][32];
                tmem_ld32(taddr, v[0]);
#pragma unroll
                for (int c = 0; c < NCH / 32; ++c) {
                    tmem_ld_wait();
                    if (c + 1 < NCH / 32) tmem_ld32(taddr + (c + 1) * 32, v[(c + 1) & 1]);
                    if (c + 1 == NCH / 32) {
                        // every column of this warp is in registers: hand the buffer back early
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_acce0 + as * 8);
                    }
                    if (MODE == MODE_ACC) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[c & 1][j] *= tscale;
                    }
                    if (row < p.m) store_row_chunk<32>(p, crow, col_base + c * 32, v[c & 1], vec_ok);
                }
                ++phase;
            }
        }
    }

    // ---------------------------------- teardown ----------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace b200
