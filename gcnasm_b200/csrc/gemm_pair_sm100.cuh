// A8W8 FP8 (E4M3) NT GEMM for sm_100a on CTA PAIRS: two CTAs on neighbouring SMs (a 2-CTA cluster)
// compute one 256 x BN output tile with tcgen05.mma.cta_group::2.
//
// Why pairs: the tensor pipe retires a 128x256x128 block in about 512 clocks, and a single CTA has to
// pull 48 KB (A 16 KB + B 32 KB) out of L2 for it -- more than the L2->SM path sustains.  In a pair each CTA
// loads its own 128 A rows and only HALF of the B rows (BN/2); the hardware reads both halves of B
// from the two CTAs' shared memories.  Per CTA that is 16 + 16 KB per block instead of 48 KB.  No load is
// ever shared between CTAs by multicast; each CTA issues plain TMA loads for its own bytes.
//
// Roles per CTA (12 warps, same split as the single-CTA kernel): warp 0 TMA producer, warp 1 UMMA issuer
// (only the pair's leader, cluster rank 0, issues MMAs; it also frees ring stages in BOTH CTAs), warps
// 4-11 epilogue.  Block-scale mode keeps the reference's structure (a fresh accumulator per 128-wide K
// group, gemm_a8w8_blockscale_kernel_template.hpp:317,334; scale_c_tile :24-39): partials ping-pong
// between two TMEM buffers and are folded into register accumulators with packed fp32 FMAs.
#pragma once

#include <type_traits>

#include "gemm_sm100.cuh"

namespace b200 {

// Eight epilogue warps per CTA: two per scheduler, 32 rows x BN/2 columns each.  (A 16-warp variant with 16-column
// TMEM loads and 112 registers computed the same results at 1475 against 2010 TFLOP/s on 8192^3 block-scale.)
template <int BN_, int MODE_, int BLAYOUT_>
struct PairCfg {
    static constexpr bool AB16 = MODE_ == MODE_ACC16;               // bf16 operands: same bytes, kind::f16 MMAs
    static constexpr int BM = 128, BN = BN_, BK = 128, MODE = AB16 ? MODE_ACC : MODE_, BLAYOUT = BLAYOUT_;
    static constexpr int EPI_WARPS = 8, NSPLIT = EPI_WARPS / 4;     // column parts per row quadrant
    static constexpr int BH = BN / 2;                               // B rows loaded by each CTA
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = BH * BK;
    static constexpr int SFB_ATOMS = (BN + 127) / 128;
    static constexpr int SFA_BYTES = (MODE == MODE_MX) ? 512 : 0;
    static constexpr int SFB_BYTES = (MODE == MODE_MX) ? SFB_ATOMS * 512 : 0;
    static constexpr int STAGE_BYTES = ((A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + 1023) / 1024) * 1024;
    // 227 KB per CTA: ring stages, 1 KB of barriers, 1 KB of alignment slack, store staging
    // block-scale: the whole finished bf16 tile of this CTA (128 x BN) is parked in shared memory and leaves
    // through TMA bulk stores, so that the epilogue warps never wait for the memory system
    static constexpr int NCH_ = BN / NSPLIT;
    static constexpr bool TILE_TMA = (MODE == MODE_BLOCK) && (NCH_ % 64 == 0);
    static constexpr int TILE_STAGE_BYTES = TILE_TMA ? 128 * BN * 2 : 0;
    // per-warp staging of the plain-store epilogue; with a tile staging area it lives inside that area (a launch
    // uses one of the two store paths)
    static constexpr int OUT_STAGE_BYTES = TILE_TMA ? 0 : EPI_WARPS * kOutStageBytesPerWarp;
    static_assert(!TILE_TMA || 32 * NCH_ * 2 >= kOutStageBytesPerWarp, "per-warp tile area holds the plain-store staging");
    static constexpr int STAGES_RAW = (227 * 1024 - 2048 - OUT_STAGE_BYTES - TILE_STAGE_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + OUT_STAGE_BYTES + TILE_STAGE_BYTES + 1024;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static constexpr int SF_COLS = (MODE == MODE_MX) ? 4 + 4 * SFB_ATOMS : 0;
    static constexpr int ACC_STAGES = (2 * BN + SF_COLS <= 512) ? 2 : 1;
    static constexpr int ACC_COLS = ACC_STAGES * BN;
    static constexpr int TMEM_COLS = (ACC_COLS + SF_COLS) <= 128 ? 128 : (ACC_COLS + SF_COLS) <= 256 ? 256 : 512;
    static constexpr int NCH = BN / NSPLIT;                         // columns owned by one epilogue thread
    static constexpr int THREADS = 128 + 32 * EPI_WARPS;
    // setmaxnreg only redistributes the registers the CTA got at launch (THREADS x the per-thread count the
    // launch bound allows, a multiple of 8); an increase beyond that pool blocks forever
    static constexpr int ROLE_REGS = 40, EPI_REGS = 232;
    static constexpr int LAUNCH_REGS = (65536 / THREADS) / 8 * 8;
    static_assert(128 * ROLE_REGS + 32 * EPI_WARPS * EPI_REGS <= THREADS * LAUNCH_REGS, "setmaxnreg pool");
    static constexpr int LW = 32;                                   // columns per TMEM load in block-scale mode
    static_assert(BN % 32 == 0 && BN <= 256 && BN >= 64, "pair tile N: multiple of 32 in [64, 256]");
    static_assert(MODE != MODE_BLOCK || ACC_STAGES == 2, "block-scale needs two partial buffers");
    static_assert(MODE != MODE_MX || BN % 128 == 0, "MX scale atoms cover 128 columns");
    static_assert(ACC_COLS + SF_COLS <= 512, "TMEM overflow");
};

// Waits.  The single-thread roles poll (mbarrier.test_wait plus a short sleep), the epilogue warps use the
// suspending try_wait.  Every wait uses the default CTA-scope acquire even when the arrivals come from the
// partner CTA: a cluster-scope acquire was measured at ~430 clocks per wait, and each hand-off here is ordered
// through the async proxy (TMA complete_tx, tcgen05.commit) or tcgen05.fence, not through generic memory.
#define B200_PROD_WAIT mbar_wait_poll<false, 64>
#define B200_MMA_WAIT mbar_wait_poll<false, 20>
// One non-suspending look at the barrier before the suspending wait: an epilogue warp that runs behind finds the phase
// already complete (measured: 0.7 % on 256 x 256 tiles, 4 % on the 224- and 192-column tiles).
__device__ __forceinline__ bool mbar_probe(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
#define B200_EPI_WAIT(bar, ph, af, st, code) (mbar_probe(bar, ph) || mbar_wait<false, 0>(bar, ph, af, st, code))
// UMMA issuer threads in block-scale mode (warps 1..kBlockIssuers of the leader CTA); at most the number of
// TMEM buffers, because an issuer has to observe every phase of the barriers it waits on.
static constexpr int kBlockIssuers = 2;
// The TMA producer thread sits on the scheduler that hosts no issuer (warps 1..2 issue, warp w runs on scheduler w % 4):
// measured against warp 0, 1.5-2 % on the 4096 x 7168 x 2048 and 16384 x 7168 x 8192 problems, nothing on 8192^3.
static constexpr int kProducerWarp = 3;

// Building with -DB200_TRACE records clock64() stamps of the hand-offs of the first CTA pair into g_trace
// (read back with b200_trace_read); it is how the latencies quoted in the comments here were measured.
#ifdef B200_TRACE
// [cta][epilogue warp][phase < 128][8 slots], then the MMA issuer's [phase < 128][8 slots].  Epilogue slots per K group:
// 7 loop top, 6 accumulator-full barrier passed, 0 first loads issued, 3 first wait::ld done, 4 last load landed,
// 1 buffer handed back, 5 / 2 the FMAs of the hand-back chunk / of the last chunk have completed (these two read the
// clock behind a data dependency on the accumulator; a plain clock read does not order against arithmetic)
// then [phase < 128]: when a polling observer (warp 0 of the leader) saw the group's accumulator-full barrier flip
__device__ long long g_trace[2 * 8 * 128 * 8 + 128 * 8 + 128];
#define B200_TRACE_EPI(slot)                                                                     \
    do {                                                                                         \
        if (pair_id == 0 && lane == 0 && phase < 128)                                            \
            g_trace[((static_cast<int>(cta) * 8 + ew) * 128 + phase) * 8 + (slot)] = clock64();   \
    } while (0)
#define B200_TRACE_EPI_DEP(slot, val)                                                            \
    do {                                                                                         \
        long long t_;                                                                            \
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_) : "l"(val));                            \
        if (pair_id == 0 && lane == 0 && phase < 128)                                            \
            g_trace[((static_cast<int>(cta) * 8 + ew) * 128 + phase) * 8 + (slot)] = t_;         \
    } while (0)
#define B200_TRACE_MMA(slot)                                                                     \
    do {                                                                                         \
        if (pair_id == 0 && phase < 128) g_trace[2 * 8 * 128 * 8 + phase * 8 + (slot)] = clock64(); \
    } while (0)
// the producers' stamps share the issuer rows: slots 6 and 7 of row it (leader CTA only)
#define B200_TRACE_PROD(slot)                                                                    \
    do {                                                                                         \
        if (pair_id == 0 && cta == 0 && warp == kProducerWarp && it < 128) g_trace[2 * 8 * 128 * 8 + it * 8 + 6 + (slot)] = clock64(); \
    } while (0)
#else
#define B200_TRACE_EPI(slot)
#define B200_TRACE_EPI_DEP(slot, val)
#define B200_TRACE_MMA(slot)
#define B200_TRACE_PROD(slot)
#endif

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::THREADS, 1)
gemm_a8w8_pair_sm100_kernel(const __grid_constant__ GemmParams p) {
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, BH = Cfg::BH, STAGES = Cfg::STAGES, MODE = Cfg::MODE;
    constexpr int NCH = Cfg::NCH, ACC_STAGES = Cfg::ACC_STAGES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
    const uint32_t bar_full0 = smem_base + STAGES * Cfg::STAGE_BYTES;   // used in the leader only
    const uint32_t bar_empty0 = bar_full0 + STAGES * 8;                 // one set per CTA
    const uint32_t bar_accf0 = bar_empty0 + STAGES * 8;                 // one set per CTA
    const uint32_t bar_acce0 = bar_accf0 + 2 * 8;                       // used in the leader only
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();          // 0 = leader
    const uint32_t peer = cta ^ 1u;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    // Programmatic dependent launch: the next kernel on the stream may be scheduled as soon as every CTA of this
    // one has passed this point and an SM is free.  What THIS kernel may do before its own predecessor has
    // completed is decided by pdl_wait() below.
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full0 + s * 8, 1);          // leader's arrive.expect_tx; bytes from both CTAs
            mbar_init(bar_empty0 + s * 8, 1);         // one tcgen05.commit per use
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_accf0 + s * 8, 1);          // one tcgen05.commit per use
            mbar_init(bar_acce0 + s * 8, 2 * Cfg::EPI_WARPS);   // every epilogue warp of the two CTAs
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
    // both CTAs' barriers must exist before either CTA signals the other
    cluster_arrive();
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // cta_group::2 MMAs write the same TMEM address in both CTAs: the two allocations must agree
    const bool tmem_ok = ld_shared_cluster_u32(mapa_shared(smem_u32(tmem_slot), peer)) == tmem_base;
    if (!tmem_ok && threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, KSTAT_TMEM_MISMATCH);

    const int groups = (MODE == MODE_BLOCK) ? p.kblocks : 1;
    const int kb_per_group = (MODE == MODE_BLOCK) ? 1 : p.kblocks;
    // work units: whole tiles, then (block-scale, when the launcher set it up) the column parts of the tail tiles
    constexpr bool kTail = (MODE == MODE_BLOCK) && BN == 256 && Cfg::BLAYOUT == BL_NK;
    const int units_total = (kTail && p.tail_split) ? p.tail_first + (p.tiles_total - p.tail_first) * p.tail_split
                                                    : p.tiles_total;
    // Unless the caller vouched for the operands, nothing is read or written before the previous kernel is complete.
    // With inputs_ready only the writes to C wait (in the epilogue, before the first tile is stored).
    if (!p.inputs_ready) pdl_wait();

    if (!tmem_ok) {
        // fall through to the teardown
    } else if (warp < 4) {
        setmaxnreg_dec<Cfg::ROLE_REGS>();
        if (warp == kProducerWarp && lane == 0) {
            // ------------------------------ TMA producer (both CTAs) ------------------------------
            uint32_t it = 0;
            bool ok = true;
            int ready_b = -1;                         // last batch whose ready word has been seen
            const uint32_t leader_full0 = mapa_shared(bar_full0, 0);
            for (int u = pair_id; u < units_total && ok; u += num_pairs) {
                int t = u, part = -1;
                if constexpr (kTail) unit_coords(p, u, t, part);
                int b, mi, ni;
                tile_coords(p, t, b, mi, ni);
                if (p.batch_ready && b != ready_b) {
                    // this batch's activation slab may still be on its way (a copy or collective on another stream)
                    if (!wait_ready_word(p.batch_ready + b, p.batch_epoch, abort_flag, p.status)) break;
                    ready_b = b;
                }
                const int bq = p.b_shared ? 0 : b;    // batch coordinate of the weights
                const int row_a = mi * (2 * BM) + static_cast<int>(cta) * BM;
                // a column part of a tail tile takes BH / tail_split rows of B per CTA, through the narrower box
                const int sub_rows = (kTail && part >= 0) ? BH / p.tail_split : BH;
                const int row_b = ni * BN + ((kTail && part >= 0) ? part * 2 * sub_rows : 0) + static_cast<int>(cta) * sub_rows;
                const CUtensorMap* tmap_b_u = (kTail && part >= 0) ? &p.tmap_b_tail : &p.tmap_b;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!B200_PROD_WAIT(bar_empty0 + s * 8, ph ^ 1, abort_flag, p.status, KSTAT_TIMEOUT_EMPTY)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    B200_TRACE_PROD(0);
                    if (cta == 0)
                        mbar_arrive_expect_tx(bar_full0 + s * 8,
                                              2 * (Cfg::A_BYTES + sub_rows * BK + Cfg::SFA_BYTES + Cfg::SFB_BYTES));
                    const uint32_t full = leader_full0 + s * 8;
                    tma_load_3d_pair(sa, &p.tmap_a, full, kb * BK, row_a, b);
                    if constexpr (Cfg::BLAYOUT == BL_NK)
                        tma_load_3d_pair(sb, tmap_b_u, full, kb * BK, row_b, bq);
                    else
                        tma_load_4d_pair(sb, &p.tmap_b, full, 0, row_b / 16, kb * (BK / 16), bq);
                    B200_TRACE_PROD(1);
                    if constexpr (MODE == MODE_MX) {
                        // scale atoms [batch][K/128][rows/128][512 B], addressed as rows of 256 bytes
                        const long long atom_a = b * (p.sfa_batch >> 9) + static_cast<long long>(kb) * p.sfa_stride + (mi * 2 + cta);
                        const long long atom_b = b * (p.sfb_batch >> 9) + static_cast<long long>(kb) * p.sfb_stride + ni * Cfg::SFB_ATOMS;
                        tma_load_2d_pair(sb + Cfg::B_BYTES, &p.tmap_sfa, full, 0, static_cast<int>(atom_a * 2));
                        tma_load_2d_pair(sb + Cfg::B_BYTES + 512, &p.tmap_sfb, full, 0, static_cast<int>(atom_b * 2));
                    }
                }
            }
        } else if (warp >= 1 && warp <= ((MODE == MODE_BLOCK) ? kBlockIssuers : 1) && lane == 0 && cta == 0) {
            // ------------------------------ UMMA issuer (leader only) ------------------------------
            // Block-scale mode runs several issuer threads (warps 1..kBlockIssuers, one per scheduler) that take the
            // K groups round-robin.  An issuer is effectively tied up until its own MMAs and commits have gone
            // through the tensor queue, so a single issuer cannot start group g+1 while group g executes; with
            // several, the next group is already queued.  Order on a TMEM buffer is kept by its drained-buffer
            // barrier, order on a ring stage by its full barrier.
            constexpr uint32_t kIssuers = (MODE == MODE_BLOCK) ? kBlockIssuers : 1;
            const uint32_t my_slot = static_cast<uint32_t>(warp - 1);
            uint32_t it = 0, phase = 0;
            bool ok = true;
            constexpr uint32_t idesc = make_idesc_f8(2 * BM, BN);
            for (int u = pair_id; u < units_total && ok; u += num_pairs) {
                // A column part of a tail tile: the same K loop with a narrower instruction, and tail_split K groups per
                // accumulator hand-off -- their partial sums lie side by side in the 256-column buffer (4 x 64 or 2 x 128).
                const bool tail_u = kTail && p.tail_split && u >= p.tail_first;
                const uint32_t idesc_u = tail_u ? make_idesc_f8(2 * BM, BN / p.tail_split) : idesc;
                const int gp = tail_u ? p.tail_split : 1;
                const uint32_t nsub = tail_u ? static_cast<uint32_t>(BN / p.tail_split) : 0u;
                for (int g = 0; g < groups && ok; g += gp, ++phase) {
                    const int cnt = (groups - g) < gp ? (groups - g) : gp;
                    if (kIssuers > 1 && (phase % kIssuers) != my_slot) {
                        it += cnt * kb_per_group;     // another issuer's hand-off
                        continue;
                    }
                    const uint32_t as = phase % ACC_STAGES;
                    const uint32_t aph = (phase / ACC_STAGES) & 1;
                    for (int j = 0; j < cnt && ok; ++j) {
                    const uint32_t tacc = tmem_base + as * BN + j * nsub;
                    for (int kb = 0; kb < kb_per_group; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        // operands first (they were prefetched long ago), then the accumulator buffer: the
                        // second wait is the latency-critical one and the MMAs follow it immediately
                        if (!B200_MMA_WAIT(bar_full0 + s * 8, ph, abort_flag, p.status, KSTAT_TIMEOUT_FULL)) {
                            ok = false;
                            break;
                        }
                        if (kb == 0 && j == 0) {
                            B200_TRACE_MMA(0);
                            if (!B200_MMA_WAIT(bar_acce0 + as * 8, aph ^ 1, abort_flag, p.status, KSTAT_TIMEOUT_ACC_E)) {
                                ok = false;
                                break;
                            }
                            B200_TRACE_MMA(1);
                        }
                        B200_TRACE_MMA(2);
                        tc_fence_after();
                        const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
                        const uint32_t sb = sa + Cfg::A_BYTES;
                        if constexpr (MODE == MODE_MX) {
                            const uint32_t tsf = tmem_base + Cfg::ACC_COLS;
                            tmem_cp_sf<2>(tsf, make_smem_desc(sb + Cfg::B_BYTES, 0, 128, kSwizzleNone));
#pragma unroll
                            for (int a = 0; a < Cfg::SFB_ATOMS; ++a)
                                tmem_cp_sf<2>(tsf + 4 + 4 * a,
                                              make_smem_desc(sb + Cfg::B_BYTES + 512 + 512 * a, 0, 128, kSwizzleNone));
                        }
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k) {
                            const uint64_t da = make_smem_desc(sa + k * 32, 16, 1024, kSwizzle128B);
                            uint64_t db;
                            if constexpr (Cfg::BLAYOUT == BL_NK) {
                                db = make_smem_desc(sb + k * 32, 16, 1024, kSwizzle128B);
                            } else {
                                constexpr uint32_t LBO = (BH / 16) * 256;
                                db = make_smem_desc(sb + k * 2 * LBO, LBO, 128, kSwizzleNone);
                            }
                            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
                            if constexpr (MODE == MODE_MX) {
                                const uint32_t tsf = tmem_base + Cfg::ACC_COLS;
                                umma_mxf8<2>(tacc, da, db, make_idesc_mxf8(2 * BM, BN, k, k), accum, tsf, tsf + 4);
                            } else {
                                if constexpr (Cfg::AB16) umma_f16<2>(tacc, da, db, make_idesc_bf16(2 * BM, BN), accum);
                                else umma_f8<2>(tacc, da, db, idesc_u, accum);
                            }
                        }
                        B200_TRACE_MMA(4);
                        umma_commit_pair(bar_empty0 + s * 8);       // frees stage s in both CTAs
                        B200_TRACE_MMA(5);
                    }
                    }
                    if (ok) umma_commit_pair(bar_accf0 + as * 8);   // wakes the epilogues of both CTAs
                    B200_TRACE_MMA(3);
                }
            }
        }
#ifdef B200_TRACE
        else if (MODE == MODE_BLOCK && warp == 0 && lane == 0 && cta == 0 && pair_id == 0) {
            uint32_t phase = 0;
            bool ok = true;
            for (int u = pair_id; u < units_total && ok && phase < 128; u += num_pairs)
                for (int g = 0; g < groups && ok && phase < 128; ++g, ++phase) {
                    ok = mbar_wait_poll<false, 32>(bar_accf0 + (phase & 1) * 8, (phase >> 1) & 1, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F);
                    g_trace[2 * 8 * 128 * 8 + 128 * 8 + phase] = clock64();
                }
        }
#endif
    } else {
        // ---------------------------------- epilogue (both CTAs) ----------------------------------
        setmaxnreg_inc<Cfg::EPI_REGS>();
        const int ew = warp - 4;
        const int quad = warp & 3;
        const int half = ew >> 2;
        const int row_in_tile = static_cast<int>(cta) * BM + quad * 32 + lane;
        const uint32_t tmem_lane = static_cast<uint32_t>(quad * 32) << 16;
        const size_t esz = (p.out_dtype == OUT_BF16) ? 2 : 4;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && ((p.ldc * esz) % 16 == 0) &&
                            ((p.c_batch * esz) % 16 == 0);
        const uint32_t leader_acce0 = mapa_shared(bar_acce0, 0);
        bool stores_pending = false;
        bool c_ordered = !p.inputs_ready;           // writes to C must follow the previous kernel (see pdl_wait above)
        float tscale = 1.0f;
        if constexpr (MODE == MODE_ACC) {
            if (p.scale_a) tscale *= __ldg(p.scale_a);
            if (p.scale_b) tscale *= __ldg(p.scale_b);
        }
        uint32_t phase = 0;
        bool ok = true;
        // One column part of a tail tile: NC 32-column chunks per thread and K group (the part is 64 * NC columns wide;
        // the half-0 warps take its first 32 * NC columns, the half-1 warps the rest).  The MMA issuer puts GP = 4 / NC
        // K groups side by side into one 256-column buffer per hand-off, so a hand-off brings four chunks per thread,
        // all loaded at once, each scaled with its own group's scales into the same accumulators.  The result leaves
        // through the per-warp staging buffer.
        auto tail_unit = [&](auto nc_tag, const int b, const int mi, const int ni, const int part) -> bool {
            constexpr int NC = decltype(nc_tag)::value;
            constexpr int CW = NC * 32, GP = 4 / NC;
            unsigned long long acc_t[CW / 2];
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) acc_t[j] = 0ull;
            const int row = mi * (2 * BM) + row_in_tile;
            const int col_first = ni * BN + part * (2 * CW) + half * CW;
            const bool col_ok = col_first < p.n;
            const float* sfa_p = p.sfa + b * p.sfa_batch + (row < p.m ? row : 0);
            const float* sfb_p = p.sfb + b * p.sfb_batch + static_cast<long long>(col_first >> 7) * p.sfb_stride;
            const uint32_t taddr0 = tmem_base + tmem_lane + half * CW;
            float sa_c[GP], sb_c[GP];
            auto load_scales = [&](const int g0) {
#pragma unroll
                for (int j = 0; j < GP; ++j) {
                    const int g = (g0 + j < groups) ? g0 + j : groups - 1;
                    sa_c[j] = __ldg(sfa_p + static_cast<long long>(g) * p.sfa_stride);
                    sb_c[j] = col_ok ? __ldg(sfb_p + g) : 0.0f;
                }
            };
            load_scales(0);
            for (int g0 = 0; g0 < groups; g0 += GP, ++phase) {
                const int cnt = (groups - g0) < GP ? (groups - g0) : GP;
                const uint32_t as = phase & 1;
                const uint32_t aph = (phase >> 1) & 1;
                if (!B200_EPI_WAIT(bar_accf0 + as * 8, aph, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F)) return false;
                tc_fence_after();
                unsigned long long sc2[GP];
#pragma unroll
                for (int j = 0; j < GP; ++j) {
                    const float sc = sa_c[j] * sb_c[j];
                    sc2[j] = pack_f32x2(sc, sc);
                }
                // the four chunks q = j * NC + c of this hand-off in two rounds of two (two 32-column register buffers,
                // as in the whole-tile loop); the buffer goes back once the second round has landed
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float v[2][32];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // (loaded whether or not group j exists in this hand-off: a conditional load would keep the
                        // buffer's old contents alive; what it brings for a missing group is never used)
                        const int q = 2 * r + h, j = q / NC, c = q % NC;
                        tmem_ld<32>(taddr0 + as * BN + j * (2 * CW) + c * 32, v[h]);
                    }
                    tmem_ld_wait();
                    if (r == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(leader_acce0 + as * 8);
                        if (g0 + GP < groups) load_scales(g0 + GP);
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int q = 2 * r + h, j = q / NC, c = q % NC;
                        if (j < cnt) {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                acc_t[c * 16 + i] = ffma2(pack_f32x2(v[h][2 * i], v[h][2 * i + 1]), sc2[j], acc_t[c * 16 + i]);
                        }
                    }
                }
            }
            if (!c_ordered) {
                pdl_wait();
                c_ordered = true;
            }
            if (stores_pending) {
                // the staging buffer lies inside the area the previous tile's bulk stores are reading
                if (lane == 0) bulk_wait_read_all();
                __syncwarp();
                stores_pending = false;
            }
            const int row0 = row - lane;
            uint8_t* cbatch = reinterpret_cast<uint8_t*>(p.c) + static_cast<size_t>(b) * p.c_batch * esz;
            uint8_t* out_stage = smem_gen + STAGES * Cfg::STAGE_BYTES + 1024 +
                                 (Cfg::TILE_TMA ? ew * (32 * NCH * 2) : ew * kOutStageBytesPerWarp);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float o[32];
#pragma unroll
                for (int j = 0; j < 16; ++j) unpack_f32x2(acc_t[c * 16 + j], o[2 * j], o[2 * j + 1]);
                if (p.out_dtype == OUT_BF16) {
                    store_chunk_coalesced<32>(p, cbatch, out_stage, row0, col_first + c * 32, o, lane, vec_ok);
                } else {
                    store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_first + c * 32, o, lane, vec_ok);
                    store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_first + c * 32 + 16, o + 16, lane, vec_ok);
                }
            }
            return true;
        };
        for (int u = pair_id; u < units_total && ok; u += num_pairs) {
            int t = u, part = -1;
            if constexpr (kTail) unit_coords(p, u, t, part);
            int b, mi, ni;
            tile_coords(p, t, b, mi, ni);
            // (first unit of this pair in batch b; recomputed from u so that no state stays live across the K loop.  The
            // unit before, u - num_pairs, is always a whole tile: the column parts are the last round.)
            if (MODE == MODE_BLOCK && p.batch_ready &&
                (u < num_pairs || (u - num_pairs) / (p.tiles_m * p.tiles_n) != b)) {
                // the A scales of this batch travel with its slab: they are read below, possibly long before the
                // producer's first load of the tile, so the epilogue warps look at the ready word themselves
                int seen = 1;
                if (lane == 0) seen = wait_ready_word(p.batch_ready + b, p.batch_epoch, abort_flag, p.status) ? 1 : 0;
                seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
                if (!seen) {
                    ok = false;
                    break;
                }
            }
            const int row = mi * (2 * BM) + row_in_tile;

            if constexpr (MODE == MODE_BLOCK) {
                if constexpr (kTail) {
                    if (part >= 0) {
                        const bool fine = (p.tail_split == 4) ? tail_unit(std::integral_constant<int, 1>{}, b, mi, ni, part)
                                                              : tail_unit(std::integral_constant<int, 2>{}, b, mi, ni, part);
                        if (!fine) {
                            ok = false;
                            break;
                        }
                        continue;
                    }
                }
                unsigned long long acc[NCH / 2];
#pragma unroll
                for (int j = 0; j < NCH / 2; ++j) acc[j] = 0ull;
                // this thread's NCH columns touch at most two 128-wide scale blocks of B
                // (with BN = 256 every thread's 128 columns are exactly one block: no second scale)
                constexpr bool kStraddle = (BN % 256) != 0;
                const int col_first = ni * BN + half * NCH;
                const int blk0 = col_first >> 7;
                const int split = kStraddle ? ((blk0 + 1) << 7) - col_first : NCH;   // columns before the block boundary
                const bool has1 = kStraddle && split < NCH && ((blk0 + 1) << 7) < p.n;
                const bool col_ok = col_first < p.n;
                const float* sfa_p = p.sfa + b * p.sfa_batch + (row < p.m ? row : 0);
                const float* sfb_p = p.sfb + b * p.sfb_batch + static_cast<long long>(blk0) * p.sfb_stride;
                const uint32_t taddr0 = tmem_base + tmem_lane + half * NCH;       // this thread's lane and first column
                float sa_cur = __ldg(sfa_p);
                float sb0_cur = col_ok ? __ldg(sfb_p) : 0.0f;
                float sb1_cur = has1 ? __ldg(sfb_p + p.sfb_stride) : 0.0f;
                // 32-column loads into NB register buffers, all in flight at the start; a 16-column tail when
                // NCH % 32 != 0.  The TMEM buffer goes back to the MMA issuer as soon as the last load has landed,
                // before the last FMAs; the next group's scales are fetched after that arrive (an arrive waits for
                // the thread's outstanding loads).
                constexpr int LW = Cfg::LW;
                constexpr int CFULL = NCH / LW, TAIL = NCH % LW;
                constexpr int NLD = CFULL + (TAIL ? 1 : 0);          // loads per group
                static_assert(TAIL == 0 || (LW == 32 && TAIL == 16), "tail load is 16 columns");
                // register buffers for the loads: with NCH <= 96 the accumulators leave room for every load of a group
                constexpr int NB = (NCH <= 96 && NLD <= 3) ? NLD : 2;
                constexpr int REL = ((NLD - 1) / NB) * NB;           // the wait at this chunk covers the final load
                for (int g = 0; g < groups; ++g, ++phase) {
                    const uint32_t as = phase & 1;
                    const uint32_t aph = (phase >> 1) & 1;
                    B200_TRACE_EPI(7);
                    if (!B200_EPI_WAIT(bar_accf0 + as * 8, aph, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F)) {
                        ok = false;
                        break;
                    }
                    B200_TRACE_EPI(6);
                    tc_fence_after();
                    const uint32_t taddr = taddr0 + as * BN;
                    B200_TRACE_EPI(0);
                    float v[NB][LW];
                    auto load_chunk = [&](const int c) {
                        if (c < CFULL) tmem_ld<LW>(taddr + c * LW, v[c % NB]);
                        else tmem_ld16(taddr + c * LW, v[c % NB]);
                    };
#pragma unroll
                    for (int c = 0; c < NB && c < NLD; ++c) load_chunk(c);
                    // (only now: the scales were requested during the previous group and may still be on their way; the
                    // multiply that waits for them must not stand between the barrier and the tensor-memory loads)
                    const float s0 = sa_cur * sb0_cur, s1 = kStraddle ? sa_cur * sb1_cur : s0;
                    const unsigned long long sc0 = pack_f32x2(s0, s0), sc1 = kStraddle ? pack_f32x2(s1, s1) : sc0;
                    // tcgen05.wait::ld waits for every load in flight, so it is executed only before the first chunk
                    // of each round of NB: the other chunks of the round landed with it, and a wait there would
                    // stall on the refill load issued a moment earlier
                    auto fma_chunk = [&](const int c) {
                        const unsigned long long scA = (!kStraddle || c * LW < split) ? sc0 : sc1;
                        const unsigned long long scB = (!kStraddle || c * LW + 16 < split) ? sc0 : sc1;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            acc[c * (LW / 2) + j] = ffma2(pack_f32x2(v[c % NB][2 * j], v[c % NB][2 * j + 1]), scA, acc[c * (LW / 2) + j]);
                        if constexpr (LW == 32) {
                            if (c < CFULL) {
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    acc[c * 16 + 8 + j] = ffma2(pack_f32x2(v[c % NB][16 + 2 * j], v[c % NB][16 + 2 * j + 1]), scB, acc[c * 16 + 8 + j]);
                            }
                        }
                    };
#pragma unroll
                    for (int c = 0; c < NLD; ++c) {
                        if (c % NB == 0) {
                            tmem_ld_wait();                              // chunks c .. c+NB-1 have landed
                            if (c == 0) B200_TRACE_EPI(3);
                        }
                        if (c == REL) {
                            // every load has landed: hand the TMEM buffer back, then fetch the next scales
                            B200_TRACE_EPI(4);
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive_cluster(leader_acce0 + as * 8);
                            B200_TRACE_EPI(1);
                            if (g + 1 < groups) {
                                sa_cur = __ldg(sfa_p + static_cast<long long>(g + 1) * p.sfa_stride);
                                sb0_cur = col_ok ? __ldg(sfb_p + g + 1) : 0.0f;
                                if (kStraddle) sb1_cur = has1 ? __ldg(sfb_p + p.sfb_stride + g + 1) : 0.0f;
                            }
                        }
                        fma_chunk(c);
#ifdef B200_TRACE
                        if (c == REL) B200_TRACE_EPI_DEP(5, acc[(c + 1) * (LW / 2) - 1]);
                        if (c == NLD - 1) B200_TRACE_EPI_DEP(2, acc[NCH / 2 - 1]);
#endif
                        // refill the buffer just drained; the load runs behind the next chunk's FMAs
                        if (c + NB < NLD) load_chunk(c + NB);
                    }
                }
                if (!ok) break;
                if (!c_ordered) {
                    pdl_wait();
                    c_ordered = true;
                }
                // Everything the store phase needs is derived again from the tile index here, behind an opaque copy of
                // it: nothing of it then has to stay in a register across the K loop, where the accumulators and the two
                // load buffers leave none to spare.
                int t_s = u, ew_s = ew;                                // (a whole tile here: its unit index is its tile index)
                uint32_t sb_s = smem_base;
                asm volatile("" : "+r"(t_s), "+r"(ew_s), "+r"(sb_s));
                uint8_t* smem_gen_s = smem_raw + (sb_s - smem_u32(smem_raw));
                int b_s, mi_s, ni_s;
                tile_coords(p, t_s, b_s, mi_s, ni_s);
                const int half_s = ew_s >> 2;
                const int row0 = mi_s * (2 * BM) + static_cast<int>(cta) * BM + (ew_s & 3) * 32;   // output row of lane 0
                const int col_base = ni_s * BN + half_s * NCH;
                const int b = b_s;
                uint8_t* cbatch = reinterpret_cast<uint8_t*>(p.c) + static_cast<size_t>(b_s) * p.c_batch * esz;
                uint8_t* out_stage = smem_gen_s + STAGES * Cfg::STAGE_BYTES + 1024 +
                                     (Cfg::TILE_TMA ? ew_s * (32 * NCH * 2) : ew_s * kOutStageBytesPerWarp);
                // this warp's part of the tile staging area: NCH/64 boxes of 32 rows x 128 bytes (1024-byte aligned)
                const uint32_t tile_stage = sb_s + STAGES * Cfg::STAGE_BYTES + 1024 +
                                            Cfg::OUT_STAGE_BYTES + ew_s * (32 * NCH * 2);
                uint8_t* tile_stage_gen = smem_gen_s + (tile_stage - sb_s);
                if (ok && Cfg::TILE_TMA && p.c_tma) {
                    // bf16 tile -> shared memory in the 128-byte-swizzled layout of the TMA box (16-byte piece c of
                    // row r sits at piece c ^ (r & 7): conflict-free for the row-per-lane register layout), then
                    // one bulk store per 64-column box.  The stores run behind the next tile's work.
                    if (stores_pending) {
                        if (lane == 0) bulk_wait_read_all();      // the previous tile's stores have read the buffer
                        __syncwarp();
                    }
#pragma unroll
                    for (int q = 0; q < NCH / 8; ++q) {                  // 8 columns = 16 bytes per piece
                        float o[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) unpack_f32x2(acc[q * 4 + j], o[2 * j], o[2 * j + 1]);
                        uint4 w;
                        w.x = pack_bf16x2(o[0], o[1]);
                        w.y = pack_bf16x2(o[2], o[3]);
                        w.z = pack_bf16x2(o[4], o[5]);
                        w.w = pack_bf16x2(o[6], o[7]);
                        const int box = q >> 3, piece = q & 7;
                        *reinterpret_cast<uint4*>(tile_stage_gen + box * 4096 + lane * 128 + ((piece ^ (lane & 7)) << 4)) = w;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
#pragma unroll
                        for (int box = 0; box < NCH / 64; ++box)
                            tma_store_3d(&p.tmap_c, tile_stage + box * 4096, col_base + box * 64, row0, b);
                        bulk_commit_group();
                    }
                    stores_pending = true;
#ifdef B200_TRACE
                    --phase;
                    B200_TRACE_EPI(7);     // end of the store phase, filed under the tile's last group
                    ++phase;
#endif
                } else if (ok) {
                    // 64-byte row segments: 32 columns of bf16 or 16 columns of fp32 per pass
                    if (p.out_dtype == OUT_BF16) {
#pragma unroll
                        for (int c = 0; c + 1 < NCH / 16; c += 2) {
                            float o[32];
#pragma unroll
                            for (int j = 0; j < 16; ++j) unpack_f32x2(acc[c * 8 + j], o[2 * j], o[2 * j + 1]);
                            store_chunk_coalesced<32>(p, cbatch, out_stage, row0, col_base + c * 16, o, lane, vec_ok);
                        }
                        if ((NCH / 16) & 1) {
                            constexpr int c = NCH / 16 - 1;
                            float o[16];
#pragma unroll
                            for (int j = 0; j < 8; ++j) unpack_f32x2(acc[c * 8 + j], o[2 * j], o[2 * j + 1]);
                            store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_base + c * 16, o, lane, vec_ok);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < NCH / 16; ++c) {
                            float o[16];
#pragma unroll
                            for (int j = 0; j < 8; ++j) unpack_f32x2(acc[c * 8 + j], o[2 * j], o[2 * j + 1]);
                            store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_base + c * 16, o, lane, vec_ok);
                        }
                    }
                }
            } else {
                const int row0 = row - lane;                       // output row of this warp's lane 0
                const int col_base = ni * BN + half * NCH;
                uint8_t* cbatch = reinterpret_cast<uint8_t*>(p.c) + static_cast<size_t>(b) * p.c_batch * esz;
                uint8_t* out_stage = smem_gen + STAGES * Cfg::STAGE_BYTES + 1024 + ew * kOutStageBytesPerWarp;
                const uint32_t as = phase % ACC_STAGES;
                const uint32_t aph = (phase / ACC_STAGES) & 1;
                if (!B200_EPI_WAIT(bar_accf0 + as * 8, aph, abort_flag, p.status, KSTAT_TIMEOUT_ACC_F)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (!c_ordered) {
                    pdl_wait();
                    c_ordered = true;
                }
                const uint32_t taddr = tmem_base + tmem_lane + as * BN + half * NCH;
                constexpr int CW = (NCH % 32 == 0) ? 32 : 16;      // columns per TMEM load
                constexpr int NC = NCH / CW;
                if constexpr (ACC_STAGES == 1) {
                    // A single accumulator buffer (MX, 256 columns + scale columns fill TMEM): pull this thread's
                    // whole row slice into registers at once and give the buffer back before converting and
                    // storing, so the next tile's MMAs run under the stores.
                    float v[NCH];
#pragma unroll
                    for (int c = 0; c < NC; ++c) tmem_ld<CW>(taddr + c * CW, &v[c * CW]);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(leader_acce0 + as * 8);
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        if (MODE == MODE_ACC) {
#pragma unroll
                            for (int j = 0; j < CW; ++j) v[c * CW + j] *= tscale;
                        }
                        if (p.out_dtype == OUT_BF16 || CW == 16) {
                            store_chunk_coalesced<CW>(p, cbatch, out_stage, row0, col_base + c * CW, &v[c * CW], lane, vec_ok);
                        } else {
                            store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_base + c * CW, &v[c * CW], lane, vec_ok);
                            store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_base + c * CW + 16, &v[c * CW + 16], lane, vec_ok);
                        }
                    }
                } else {
                    float v[2][CW];
                    tmem_ld<CW>(taddr, v[0]);
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        tmem_ld_wait();
                        if (c + 1 < NC) tmem_ld<CW>(taddr + (c + 1) * CW, v[(c + 1) & 1]);
                        if (c + 1 == NC) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive_cluster(leader_acce0 + as * 8);
                        }
                        if (MODE == MODE_ACC) {
#pragma unroll
                            for (int j = 0; j < CW; ++j) v[c & 1][j] *= tscale;
                        }
                        if (p.out_dtype == OUT_BF16 || CW == 16) {
                            store_chunk_coalesced<CW>(p, cbatch, out_stage, row0, col_base + c * CW, v[c & 1], lane, vec_ok);
                        } else {
                            store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_base + c * CW, v[c & 1], lane, vec_ok);
                            store_chunk_coalesced<16>(p, cbatch, out_stage, row0, col_base + c * CW + 16, v[c & 1] + 16, lane, vec_ok);
                        }
                    }
                }
                ++phase;
            }
        }
    }

    // ---------------------------------- teardown ----------------------------------
    // (a CTA must not exit while its bulk stores still read its shared memory)
    if (warp >= 4 && lane == 0) bulk_wait_all();
    tc_fence_before();
    __syncthreads();
    // neither CTA may leave while its partner can still read its shared memory or signal its barriers
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace b200
