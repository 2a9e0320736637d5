// Host side of libb200gemm.so: argument validation, tile-config selection, TMA tensor-map
// construction and kernel launches behind the C ABI declared in include/b200gemm.h.
//
// Tile-config selection replaces the reference's compile-time traits structs
// (opus_gemm/gemm_a8w8_8wave.cc:36-96, block_scale_gemm/gemm_a8w8_blockscale_common.h:28-84,
// opus_fmm/flatmm_a8w8_gfx950.cc:36-104) with a run-time choice from a small static table.
#include "../../include/b200gemm.h"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "aux_kernels.cuh"
#include "decode_sm100.cuh"
#include "gemm_pair_sm100.cuh"
#include "gemm_sm100.cuh"
#include "weight_file.h"

namespace {

using namespace b200;

std::atomic<uint64_t> g_launches{0};
thread_local int g_last_cuda = 0;

__device__ int g_status_word;

#define CU_TRY(expr)                                   \
    do {                                               \
        cudaError_t e_ = (expr);                       \
        if (e_ != cudaSuccess) {                       \
            g_last_cuda = static_cast<int>(e_);        \
            return B200_ERR_CUDA;                      \
        }                                              \
    } while (0)

// ---- per-device state ------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
struct DeviceState {
    bool init = false;
    int sm_count = 0;
    int cc_major = 0;
    int* status_ptr = nullptr;
    // cached buffers of b200_gemm_a8w8_host
    void* buf[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t cap[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // b200_gemm_a8w8_host: second stream for the copy-back of finished row slabs, one event per slab
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t slab_done[16] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                 nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t copies_done = nullptr;
    cudaStream_t peek_stream = nullptr;   // b200_peek_status: reads the status word without waiting for other streams
    std::mutex host_entry_mu;             // b200_gemm_a8w8_host: one caller at a time per device (shared staging buffers)
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
typedef CUresult (*StreamWriteValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
StreamWriteValue32Fn g_write_value32 = nullptr;     // null when the driver does not offer stream memory operations
StreamWriteValue32Fn g_wait_value32 = nullptr;      // cuStreamWaitValue32 has the same signature


int device_state(DeviceState** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        g_last_cuda = static_cast<int>(e);
        return B200_ERR_NO_DEVICE;
    }
    if (dev < 0 || dev >= kMaxDevices) return B200_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = g_dev[dev];
    if (!s.init) {
        cudaDeviceProp prop;
        CU_TRY(cudaGetDeviceProperties(&prop, dev));
        s.sm_count = prop.multiProcessorCount;
        // B200GEMM_MAX_SMS caps the SMs the persistent GEMM grids occupy, so that a collective running on another
        // stream (the activation broadcast of the N-sharded mode) finds free SMs and overlaps with the GEMM
        if (const char* cap = std::getenv("B200GEMM_MAX_SMS")) {
            const int v = std::atoi(cap);
            if (v >= 2 && v < s.sm_count) s.sm_count = v;
        }
        s.cc_major = prop.major;
        if (prop.major != 10) return B200_ERR_NO_DEVICE;
        void* sym = nullptr;
        CU_TRY(cudaGetSymbolAddress(&sym, g_status_word));
        s.status_ptr = static_cast<int*>(sym);
        CU_TRY(cudaMemset(s.status_ptr, 0, sizeof(int)));
        if (!g_encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            CU_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
            if (q != cudaDriverEntryPointSuccess || !fn) return B200_ERR_NO_DEVICE;
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
            void* wv = nullptr;
            if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &wv, cudaEnableDefault, &q) == cudaSuccess &&
                q == cudaDriverEntryPointSuccess && wv)
                g_write_value32 = reinterpret_cast<StreamWriteValue32Fn>(wv);
            else
                cudaGetLastError();
            wv = nullptr;
            if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &wv, cudaEnableDefault, &q) == cudaSuccess &&
                q == cudaDriverEntryPointSuccess && wv)
                g_wait_value32 = reinterpret_cast<StreamWriteValue32Fn>(wv);
            else
                cudaGetLastError();
        }
        s.init = true;
    }
    *out = &s;
    return B200_OK;
}

// u8 tensor map of rank `rank`; dims/strides innermost first, strides[i] = byte stride of dim i+1
// Encoding a tensor map costs a driver call; serving loops present the same few buffers over and over, so
// the most recent encodings are kept (keyed by every encode parameter; a map holds no device-specific state
// beyond the address it was encoded for).
struct TmapKey {
    const void* base;
    uint64_t dims[5], strides[4];
    uint32_t box[5];
    int rank, swz, dtype;
};
struct TmapEntry {
    TmapKey key;
    CUtensorMap map;
    bool used;
};
constexpr int kTmapCache = 64;
TmapEntry g_tmaps[kTmapCache];
int g_tmap_next = 0;
std::mutex g_tmap_mu;

int make_tmap(CUtensorMap* tm, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
              const uint32_t* box, CUtensorMapSwizzle swz, CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_UINT8) {
    TmapKey key;
    std::memset(&key, 0, sizeof(key));
    key.base = base;
    key.rank = rank;
    key.swz = static_cast<int>(swz);
    key.dtype = static_cast<int>(dtype);
    for (int i = 0; i < rank; ++i) {
        key.dims[i] = dims[i];
        key.box[i] = box[i];
    }
    for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
    {
        std::lock_guard<std::mutex> lk(g_tmap_mu);
        for (int i = 0; i < kTmapCache; ++i)
            if (g_tmaps[i].used && std::memcmp(&g_tmaps[i].key, &key, sizeof(key)) == 0) {
                *tm = g_tmaps[i].map;
                return B200_OK;
            }
    }
    cuuint64_t gd[5], gs[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) {
        gd[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) gs[i] = strides[i];
    CUresult r = g_encode(tm, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gd,
                          gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda = 100000 + static_cast<int>(r);
        return B200_ERR_CUDA;
    }
    {
        std::lock_guard<std::mutex> lk(g_tmap_mu);
        TmapEntry& e = g_tmaps[g_tmap_next];
        g_tmap_next = (g_tmap_next + 1) % kTmapCache;
        e.key = key;
        e.map = *tm;
        e.used = true;
    }
    return B200_OK;
}

// row-major u8 [batch][rows][K] with a 128-byte-swizzled box of 128 (K) x box_rows
int make_rowmajor_tmap(CUtensorMap* tm, const void* base, int64_t rows, int64_t k, int64_t ld, int64_t batch,
                       int64_t batch_stride, uint32_t box_rows) {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(rows), static_cast<uint64_t>(batch)};
    const uint64_t strides[2] = {static_cast<uint64_t>(ld),
                                 static_cast<uint64_t>(batch > 1 ? batch_stride : ld * rows)};
    const uint32_t box[3] = {128, box_rows, 1};
    return make_tmap(tm, base, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// flat image [N/16][K/16][256 B] viewed as (256 B, slab, k-chunk, batch): a box {256, rows/16, 8, 1}
// lands in shared memory as [k-chunk][slab][256 B]
int make_flat_tmap(CUtensorMap* tm, const void* base, int64_t n, int64_t k, int64_t batch, int64_t batch_stride,
                   uint32_t box_rows) {
    const uint64_t dims[4] = {256, static_cast<uint64_t>(n / 16), static_cast<uint64_t>(k / 16),
                              static_cast<uint64_t>(batch)};
    const uint64_t strides[3] = {static_cast<uint64_t>(k * 16), 256,
                                 static_cast<uint64_t>(batch > 1 ? batch_stride : n * k)};
    const uint32_t box[4] = {256, box_rows / 16, 8, 1};
    return make_tmap(tm, base, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// ---- validation and config selection -----------------------------------------------------------
struct Plan {
    int tile;        // b200_tile_hint value actually used
    int mt;          // decode token block
    int splits;      // decode K splits
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ab16: `a` is the byte view of a bf16 problem (K and the A/B strides counted in bytes)
int validate(const b200_gemm_args* a, int sm_count, Plan* plan, bool ab16 = false) {
    if (!a || !a->ptr_a || !a->ptr_b || !a->ptr_c) return B200_ERR_BAD_ARG;
    if (a->m <= 0 || a->n <= 0 || a->k <= 0 || a->batch <= 0) return B200_ERR_BAD_ARG;
    if (a->scale_mode < 0 || a->scale_mode > 3 || a->b_layout < 0 || a->b_layout > 1 || a->out_dtype < 0 ||
        a->out_dtype > 1 || a->tile_hint < 0 || a->tile_hint > 8)
        return B200_ERR_BAD_ARG;
    if (ab16 && (a->scale_mode == B200_SCALE_BLOCK || a->scale_mode == B200_SCALE_MX)) return B200_ERR_UNSUPPORTED;
    if (a->m > 0x7FFFFFFF || a->n > 0x7FFFFFFF || a->k > 0x7FFFFFFF || a->batch > 65535) return B200_ERR_TOO_LARGE;
    if (a->stride_a < a->k || a->stride_c < a->n) return B200_ERR_BAD_ARG;
    // TMA: 16-byte aligned bases and row pitches
    if (!aligned16(a->ptr_a) || !aligned16(a->ptr_b)) return B200_ERR_UNSUPPORTED;
    if (a->stride_a % 16 != 0 || a->k % 16 != 0) return B200_ERR_UNSUPPORTED;
    if (a->batch > 1 && (a->stride_a_batch % 16 != 0 || a->stride_b_batch % 16 != 0)) return B200_ERR_UNSUPPORTED;
    if (a->b_layout == B200_B_NK_ROWMAJOR) {
        if (a->stride_b < a->k) return B200_ERR_BAD_ARG;
        if (a->stride_b % 16 != 0) return B200_ERR_UNSUPPORTED;
    } else {
        if (a->n % 16 != 0 || a->k % 128 != 0) return B200_ERR_UNSUPPORTED;   // flat needs whole 16x16 blocks
    }
    if (a->scale_mode == B200_SCALE_BLOCK) {
        if (!a->ptr_sfa || !a->ptr_sfb) return B200_ERR_BAD_ARG;
        // GROUP_M/N/K = 1/128/128 check of gemm_a8w8_blockscale_host.cc:183
        if (a->n % 128 != 0 || a->k % 128 != 0) return B200_ERR_UNSUPPORTED;
        if (a->stride_sfa < a->m || a->stride_sfb < a->k / 128) return B200_ERR_BAD_ARG;
    }
    if (a->scale_mode == B200_SCALE_MX) {
        if (!a->ptr_sfa || !a->ptr_sfb) return B200_ERR_BAD_ARG;
        if (a->k % 128 != 0) return B200_ERR_UNSUPPORTED;
        if (!aligned16(a->ptr_sfa) || !aligned16(a->ptr_sfb)) return B200_ERR_UNSUPPORTED;
        if (a->batch > 1 && (a->stride_sfa_batch % 16 != 0 || a->stride_sfb_batch % 16 != 0)) return B200_ERR_UNSUPPORTED;
    }

    // slabs that are still arriving, and one B for every batch: the 2-CTA tile kernels only
    const bool batch_ready = (a->flags & B200_GEMM_BATCH_READY) != 0;
    const bool b_shared = a->batch > 1 && a->stride_b_batch == 0;
    const bool pair_only = batch_ready || b_shared;
    if (batch_ready && !a->ptr_batch_ready) return B200_ERR_BAD_ARG;
    if (batch_ready && (ab16 || a->scale_mode == B200_SCALE_MX)) return B200_ERR_UNSUPPORTED;
    if (b_shared && a->scale_mode == B200_SCALE_BLOCK && a->stride_sfb_batch != 0) return B200_ERR_BAD_ARG;
    if (pair_only && a->m <= 128) return B200_ERR_UNSUPPORTED;

    Plan pl{B200_TILE_128x128, 0, 1};
    const int64_t kblocks = (a->k + 127) / 128;
    const bool decode_ok = !pair_only && !ab16 && a->m <= 64 && a->scale_mode != B200_SCALE_MX && (a->n % 16 == 0);
    int hint = a->tile_hint;
    if (hint == B200_TILE_DECODE && !decode_ok) return B200_ERR_UNSUPPORTED;
    if (hint == B200_TILE_128x64) return B200_ERR_UNSUPPORTED;
    const bool mx = a->scale_mode == B200_SCALE_MX;
    // MX pair kernels address the scale atoms through a tensor map: batch strides in whole atoms
    const bool mx_pair_ok = !mx || a->batch == 1 || (a->stride_sfa_batch % 512 == 0 && a->stride_sfb_batch % 512 == 0);
    if (hint == B200_TILE_AUTO) {
        if (decode_ok) {
            hint = B200_TILE_DECODE;
        } else {
            // cost of a persistent schedule: rounds x time per tile (proportional to the tile's N)
            const int pairs = sm_count / 2;
            const int64_t tm2 = (a->m + 255) / 256, tm1 = (a->m + 127) / 128;
            int64_t best = -1;
            auto consider = [&](int tile, int bn, bool pair) {
                const int64_t tiles = (pair ? tm2 : tm1) * ((a->n + bn - 1) / bn) * a->batch;
                const int64_t units = pair ? pairs : sm_count;
                const int64_t rounds = (tiles + units - 1) / units;
                // weight = relative time per output column: pairs with wide tiles feed the tensor pipe best,
                // narrow and single-CTA tiles re-read more of A/B per flop from L2
                // (block-scale tiles that straddle the 128-column scale blocks pay for the second scale)
                int64_t w = pair ? (bn >= 192 ? 10 : 13) : (bn >= 256 ? 14 : 18);
                if (a->scale_mode == B200_SCALE_BLOCK && bn % 128 != 0) w += 2;
                const int64_t cost = rounds * bn * w;
                if (best < 0 || cost < best) {
                    best = cost;
                    hint = tile;
                }
            };
            if (mx) {
                if (mx_pair_ok && a->m > 128) consider(B200_TILE_PAIR_256x256, 256, true);
                if (!pair_only) consider(B200_TILE_128x128, 128, false);
            } else {
                if (a->m > 128) {
                    consider(B200_TILE_PAIR_256x256, 256, true);
                }
                if (a->m > 128 && !ab16) {
                    consider(B200_TILE_PAIR_256x224, 224, true);
                    consider(B200_TILE_PAIR_256x192, 192, true);
                    consider(B200_TILE_PAIR_256x128, 128, true);
                }
                if (!pair_only) {
                    consider(B200_TILE_128x256, 256, false);
                    consider(B200_TILE_128x128, 128, false);
                }
            }
        }
    }
    if (pair_only && !(hint == B200_TILE_PAIR_256x256 || hint == B200_TILE_PAIR_256x224 || hint == B200_TILE_PAIR_256x192 ||
                       hint == B200_TILE_PAIR_256x128))
        return B200_ERR_UNSUPPORTED;
    if (mx && !(hint == B200_TILE_128x128 || (hint == B200_TILE_PAIR_256x256 && mx_pair_ok))) return B200_ERR_UNSUPPORTED;
    // bf16 operands: pair 256x256 and the two single-CTA tiles are built
    if (ab16 && !(hint == B200_TILE_128x128 || hint == B200_TILE_128x256 || hint == B200_TILE_PAIR_256x256)) return B200_ERR_UNSUPPORTED;
    pl.tile = hint;
    if (hint == B200_TILE_DECODE) {
        pl.mt = a->m <= 16 ? 16 : (a->m <= 32 ? 32 : 64);
        // K splits: fill the machine when there are fewer weight panels than SMs, and keep the
        // per-CTA scale staging within its shared-memory budget
        const int64_t tiles = ((a->n + 127) / 128) * a->batch;
        int splits = 1;
        while (tiles * splits * 2 <= sm_count && splits * 2 <= kblocks && splits < 16) splits *= 2;
        if (a->scale_mode == B200_SCALE_BLOCK) {
            const int64_t cap = decode_sf_bytes(pl.mt) / 4;
            while (((kblocks + splits - 1) / splits) * (pl.mt + 1) > cap) {
                splits *= 2;
                if (splits > kblocks) return B200_ERR_TOO_LARGE;
            }
        }
        pl.splits = splits;
    }
    if (plan) *plan = pl;
    return B200_OK;
}

// (one call per kernel and device: the attribute sticks, and a launch should cost no more host time than it
// has to.  Keyed by the function address -- every instantiation has the same pointer TYPE.)
struct SmemAttrDone {
    const void* fn;
    int dev;
};
SmemAttrDone g_smem_done[256];
int g_smem_done_count = 0;
std::mutex g_smem_mu;

template <class Kernel>
int set_smem(Kernel kernel, int bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B200_ERR_NO_DEVICE;
    const void* fn = reinterpret_cast<const void*>(kernel);
    std::lock_guard<std::mutex> lk(g_smem_mu);
    for (int i = 0; i < g_smem_done_count; ++i)
        if (g_smem_done[i].fn == fn && g_smem_done[i].dev == dev) return B200_OK;
    CU_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (g_smem_done_count < 256) g_smem_done[g_smem_done_count++] = SmemAttrDone{fn, dev};
    return B200_OK;
}

template <int BN, int MODE, int BL>
int launch_gemm(const GemmParams& p, int grid, cudaStream_t st) {
    using Cfg = GemmCfg<BN, MODE, BL>;
    auto kernel = gemm_a8w8_sm100_kernel<Cfg>;
    int rc = set_smem(kernel, Cfg::SMEM_BYTES);
    if (rc) return rc;
    kernel<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, st>>>(p);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}

template <int MT, int MODE, int BL>
int launch_decode(const DecodeParams& p, int grid, cudaStream_t st) {
    using Cfg = DecodeCfg<MT, MODE, BL>;
    auto kernel = decode_a8w8_sm100_kernel<Cfg>;
    int rc = set_smem(kernel, Cfg::SMEM_BYTES);
    if (rc) return rc;
    // programmatic serialization: a following decode launch may begin (and request its first weight tiles)
    // while this one drains; the kernel waits for its predecessor before it touches tokens, scales or C
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    std::memset(&attr, 0, sizeof(attr));
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    CU_TRY(cudaLaunchKernelEx(&cfg, kernel, p));
    g_launches.fetch_add(1);
    return B200_OK;
}

// number of CTA pairs that can be resident at once (GPCs with an odd SM count strand one SM)
template <class Kernel>
int max_pairs(Kernel kernel, int threads, int smem, int sm_count) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = sm_count / 2;
    }
    return n < sm_count / 2 ? n : sm_count / 2;
}

// CTA pairs of this kernel that are resident at once on the current device (0 on failure)
template <int BN, int MODE, int BL>
int pair_capacity(int sm_count) {
    using Cfg = PairCfg<BN, MODE, BL>;
    auto kernel = gemm_a8w8_pair_sm100_kernel<Cfg>;
    if (set_smem(kernel, Cfg::SMEM_BYTES)) return 0;
    static int pairs_cached[kMaxDevices] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return 0;
    if (pairs_cached[dev] == 0) pairs_cached[dev] = max_pairs(kernel, Cfg::THREADS, Cfg::SMEM_BYTES, sm_count);
    return pairs_cached[dev];
}

// The last round of a persistent schedule is rarely full: 448 tiles on 74 CTA pairs leave 4 tiles for a seventh round, and 70
// pairs idle while those are computed.  Block-scale GEMMs on 256 x 256 tiles (row-major B) therefore compute the
// tiles of a partial last round as 4 (or 2) column parts each, one part per pair, when there are pairs enough: the
// same K loop with 64- (128-) column MMAs, so every element is summed in exactly the order of a whole tile and
// nothing meets in memory.  Sets p.tail_first / p.tail_split; B200GEMM_TAIL_SPLIT=0 in the environment (read once)
// switches it off.
thread_local int t_last_tail[2] = {0, 0};      // the calling thread's last pair launch (b200_last_tail_split)
void plan_tail(GemmParams& p, int capacity) {
    static const bool off = [] {
        const char* e = std::getenv("B200GEMM_TAIL_SPLIT");
        return e && *e == '0';
    }();
    p.tail_first = p.tiles_total;
    p.tail_split = 0;
    if (off || capacity <= 0 || p.kblocks < 4) return;
    const int full = (p.tiles_total / capacity) * capacity;
    const int rem = p.tiles_total - full;
    // (a problem of less than one round is left alone: measured, four times as many pairs on quarter tiles gain nothing there)
    if (rem == 0 || full == 0) return;
    const int split = rem * 4 <= capacity ? 4 : (rem * 2 <= capacity ? 2 : 0);
    if (!split) return;
    p.tail_first = full;
    p.tail_split = split;
    t_last_tail[0] = full;
    t_last_tail[1] = split;
}

template <int BN, int MODE, int BL>
int launch_pair(const GemmParams& p, int sm_count, cudaStream_t st) {
    using Cfg = PairCfg<BN, MODE, BL>;
    auto kernel = gemm_a8w8_pair_sm100_kernel<Cfg>;
    if (!p.tail_split) t_last_tail[0] = t_last_tail[1] = 0;
    const int capacity = pair_capacity<BN, MODE, BL>(sm_count);
    if (capacity <= 0) return B200_ERR_CUDA;
    int pairs = p.tiles_total < capacity ? p.tiles_total : capacity;
    if (p.tail_split) pairs = capacity;              // (plan_tail: whole rounds, then one round of parts)
    // programmatic serialization: this launch may begin while its predecessor drains; the kernel decides what it
    // does before the predecessor is complete (b200_gemm_flags)
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
    cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    std::memset(&attr, 0, sizeof(attr));
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    // A launch that waits for ready words starts in plain stream order, after its predecessor has COMPLETED.  With
    // programmatic serialization its first CTAs would be placed on whatever SMs the predecessor leaves free -- the very
    // SMs a capped grid (B200GEMM_MAX_SMS) sets aside for the collective that delivers the slabs -- and spin there on
    // words that collective can then never write.
    cfg.numAttrs = p.batch_ready ? 0 : 1;
    CU_TRY(cudaLaunchKernelEx(&cfg, kernel, p));
    g_launches.fetch_add(1);
    return B200_OK;
}

template <int BN>
int launch_pair_modes(const b200_gemm_args* a, const GemmParams& p, int sm_count, cudaStream_t st) {
    const bool flat = a->b_layout == B200_B_FLAT_16x16;
    switch (a->scale_mode) {
        case B200_SCALE_BLOCK:
            return flat ? launch_pair<BN, MODE_BLOCK, BL_FLAT>(p, sm_count, st) : launch_pair<BN, MODE_BLOCK, BL_NK>(p, sm_count, st);
        case B200_SCALE_MX:
            if constexpr (BN == 256)
                return flat ? launch_pair<BN, MODE_MX, BL_FLAT>(p, sm_count, st) : launch_pair<BN, MODE_MX, BL_NK>(p, sm_count, st);
            else
                return B200_ERR_UNSUPPORTED;
        default:
            return flat ? launch_pair<BN, MODE_ACC, BL_FLAT>(p, sm_count, st) : launch_pair<BN, MODE_ACC, BL_NK>(p, sm_count, st);
    }
}

template <int MODE, int BL>
int launch_decode_mt(int mt, const DecodeParams& p, int grid, cudaStream_t st) {
    switch (mt) {
        case 16: return launch_decode<16, MODE, BL>(p, grid, st);
        case 32: return launch_decode<32, MODE, BL>(p, grid, st);
        default: return launch_decode<64, MODE, BL>(p, grid, st);
    }
}

// Split-K workspaces of the skinny-M path.  One per (device, stream): launches on different streams never share
// partials.  A workspace that has been handed to a launch is never freed or moved before b200_release() -- a
// launch still in flight, or a CUDA graph that captured one, keeps using the pointer it was given -- so a stream
// that needs more gets an additional, larger one and the old one merely stops being handed out.
struct Scratch {
    int dev;
    cudaStream_t stream;
    float* ptr;
    size_t cap;          // bytes
    bool current;        // the one handed out for (dev, stream); older, smaller ones stay allocated until release
};
constexpr int kMaxScratch = 256;
Scratch g_scratch[kMaxScratch];
int g_scratch_count = 0;

int scratch_for(int dev, cudaStream_t st, size_t need, float** out) {
    std::lock_guard<std::mutex> lk(g_mu);
    Scratch* cur = nullptr;
    for (int i = 0; i < g_scratch_count; ++i)
        if (g_scratch[i].current && g_scratch[i].dev == dev && g_scratch[i].stream == st) cur = &g_scratch[i];
    if (cur && cur->cap >= need) {
        *out = cur->ptr;
        return B200_OK;
    }
    if (g_scratch_count == kMaxScratch) return B200_ERR_TOO_LARGE;      // too many (stream, size) generations
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        return B200_ERR_UNSUPPORTED;                                      // no allocation inside a capture
    float* ptr = nullptr;
    CU_TRY(cudaMalloc(&ptr, need));
    if (cur) cur->current = false;
    g_scratch[g_scratch_count++] = Scratch{dev, st, ptr, need, true};
    *out = ptr;
    return B200_OK;
}

// ---- allocation-free decode variant -------------------------------------------------------------------
// Split-K scratch that lives in the library image instead of in cudaMalloc'd memory: every GPU that loads the
// library holds these bytes until the process exits.  In host code the NAME of the array is only a host-side
// handle, not a device address; the address each device uses comes from cudaGetSymbolAddress, asked once
// per device with that device current.
constexpr size_t kStaticScratchFloats = 256 * 1024;                   // 1 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
float* g_static_scratch_ptr[kMaxDevices] = {nullptr};

int static_scratch(size_t need_floats, float** out) {
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return B200_ERR_NO_DEVICE;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_static_scratch_ptr[dev]) {
            void* sym = nullptr;
            CU_TRY(cudaGetSymbolAddress(&sym, g_static_scratch));     // this device's copy of the array
            g_static_scratch_ptr[dev] = static_cast<float*>(sym);
        }
        *out = g_static_scratch_ptr[dev];
    }
    return need_floats > kStaticScratchFloats ? B200_ERR_TOO_LARGE : B200_OK;
}

// use_static: the split-K partials go to the fixed array above (b200_gemm_a8w8_decode_static) instead of a
// cudaMalloc'd per-stream workspace.  Every element of the partials that the reduction reads is written by the
// launch first, so neither kind of workspace is ever cleared.
int run_decode(const b200_gemm_args* a, const Plan& pl, DeviceState* ds, cudaStream_t st, bool use_static = false) {
    DecodeParams p;
    std::memset(&p, 0, sizeof(p));
    const size_t need_floats = pl.splits > 1 ? static_cast<size_t>(pl.splits) * a->batch * a->m * a->n : 0;
    if (use_static) {
        float* scratch = nullptr;
        int rc0 = static_scratch(need_floats, &scratch);
        if (rc0) return rc0;
        p.partial = pl.splits > 1 ? scratch : nullptr;
    } else if (pl.splits > 1) {
        int dev = 0;
        CU_TRY(cudaGetDevice(&dev));
        int rc0 = scratch_for(dev, st, need_floats * sizeof(float), &p.partial);
        if (rc0) return rc0;
    }
    int rc;
    if (a->b_layout == B200_B_NK_ROWMAJOR)
        rc = make_rowmajor_tmap(&p.tmap_w, a->ptr_b, a->n, a->k, a->stride_b, a->batch, a->stride_b_batch, 128);
    else
        rc = make_flat_tmap(&p.tmap_w, a->ptr_b, a->n, a->k, a->batch, a->stride_b_batch, 128);
    if (rc) return rc;
    rc = make_rowmajor_tmap(&p.tmap_x, a->ptr_a, a->m, a->k, a->stride_a, a->batch, a->stride_a_batch, pl.mt);
    if (rc) return rc;
    p.c = a->ptr_c;
    p.sfa = static_cast<const float*>(a->ptr_sfa);
    p.sfb = static_cast<const float*>(a->ptr_sfb);
    p.scale_a = a->scale_mode == B200_SCALE_TENSOR ? a->ptr_scale_a : nullptr;
    p.scale_b = a->scale_mode == B200_SCALE_TENSOR ? a->ptr_scale_b : nullptr;
    p.ldc = a->stride_c;
    p.c_batch = a->stride_c_batch;
    p.sfa_stride = a->stride_sfa;
    p.sfb_stride = a->stride_sfb;
    p.sfa_batch = a->stride_sfa_batch;
    p.sfb_batch = a->stride_sfb_batch;
    p.m = static_cast<int>(a->m);
    p.n = static_cast<int>(a->n);
    p.k = static_cast<int>(a->k);
    p.batch = static_cast<int>(a->batch);
    p.tiles_n = static_cast<int>((a->n + 127) / 128);
    p.kblocks = static_cast<int>((a->k + 127) / 128);
    p.splits = pl.splits;
    p.kb_per_split = (p.kblocks + pl.splits - 1) / pl.splits;
    p.out_dtype = a->out_dtype;
    p.inputs_ready = (a->flags & B200_GEMM_INPUTS_READY) ? 1 : 0;
    p.status = ds->status_ptr;
    const int grid = p.tiles_n * p.batch * pl.splits;
    const bool block = a->scale_mode == B200_SCALE_BLOCK;
    if (a->b_layout == B200_B_NK_ROWMAJOR)
        rc = block ? launch_decode_mt<MODE_BLOCK, BL_NK>(pl.mt, p, grid, st) : launch_decode_mt<MODE_ACC, BL_NK>(pl.mt, p, grid, st);
    else
        rc = block ? launch_decode_mt<MODE_BLOCK, BL_FLAT>(pl.mt, p, grid, st) : launch_decode_mt<MODE_ACC, BL_FLAT>(pl.mt, p, grid, st);
    if (rc) return rc;
    if (pl.splits > 1) {
        const long long per_split = static_cast<long long>(a->batch) * a->m * a->n;
        const int threads = 256;
        const unsigned blocks = static_cast<unsigned>((per_split + threads - 1) / threads);
        decode_splitk_reduce_kernel<<<blocks, threads, 0, st>>>(p.partial, a->ptr_c, pl.splits, per_split, p.m, p.n,
                                                               p.ldc, p.c_batch, p.out_dtype);
        CU_TRY(cudaGetLastError());
        g_launches.fetch_add(1);
    }
    return B200_OK;
}

int run_gemm(const b200_gemm_args* a, const Plan& pl, DeviceState* ds, cudaStream_t st, bool ab16 = false) {
    int BN = 128;
    bool pair = false;
    switch (pl.tile) {
        case B200_TILE_128x256: BN = 256; break;
        case B200_TILE_PAIR_256x256: BN = 256; pair = true; break;
        case B200_TILE_PAIR_256x224: BN = 224; pair = true; break;
        case B200_TILE_PAIR_256x192: BN = 192; pair = true; break;
        case B200_TILE_PAIR_256x128: BN = 128; pair = true; break;
        default: BN = 128; break;
    }
    const int BMT = pair ? 256 : 128;                 // output rows per tile
    const int BROWS = pair ? BN / 2 : BN;             // B rows one CTA loads
    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    int rc = make_rowmajor_tmap(&p.tmap_a, a->ptr_a, a->m, a->k, a->stride_a, a->batch, a->stride_a_batch, 128);
    if (rc) return rc;
    const bool b_shared = a->batch > 1 && a->stride_b_batch == 0;      // one B for every batch (validate(): pair tiles)
    const int64_t b_batches = b_shared ? 1 : a->batch;
    if (a->b_layout == B200_B_NK_ROWMAJOR)
        rc = make_rowmajor_tmap(&p.tmap_b, a->ptr_b, a->n, a->k, a->stride_b, b_batches, a->stride_b_batch, BROWS);
    else
        rc = make_flat_tmap(&p.tmap_b, a->ptr_b, a->n, a->k, b_batches, a->stride_b_batch, BROWS);
    if (rc) return rc;
    if (pair && a->scale_mode == B200_SCALE_MX) {
        // scale atoms as rows of 256 bytes; one atom = 2 rows
        const uint64_t bytes_a = a->batch > 1 ? static_cast<uint64_t>(a->stride_sfa_batch) * a->batch : b200_mx_sf_bytes(a->m, a->k);
        const uint64_t bytes_b = a->batch > 1 ? static_cast<uint64_t>(a->stride_sfb_batch) * a->batch : b200_mx_sf_bytes(a->n, a->k);
        const uint64_t da[2] = {256, bytes_a / 256}, db[2] = {256, bytes_b / 256};
        const uint64_t str[1] = {256};
        const uint32_t box_a[2] = {256, 2}, box_b[2] = {256, static_cast<uint32_t>(2 * ((BN + 127) / 128))};
        if ((rc = make_tmap(&p.tmap_sfa, a->ptr_sfa, 2, da, str, box_a, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
        if ((rc = make_tmap(&p.tmap_sfb, a->ptr_sfb, 2, db, str, box_b, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    }
    if (pair && a->scale_mode == B200_SCALE_BLOCK && a->out_dtype == B200_OUT_BF16 && aligned16(a->ptr_c) &&
        a->stride_c % 8 == 0 && (a->batch == 1 || a->stride_c_batch % 8 == 0)) {
        // bf16 C [batch][M][N] for the epilogue's bulk stores: 64-column x 32-row boxes, clipped at the edges
        const uint64_t d[3] = {static_cast<uint64_t>(a->n), static_cast<uint64_t>(a->m), static_cast<uint64_t>(a->batch)};
        const uint64_t st[2] = {static_cast<uint64_t>(a->stride_c) * 2,
                                static_cast<uint64_t>(a->batch > 1 ? a->stride_c_batch : a->stride_c * a->m) * 2};
        const uint32_t bx[3] = {64, 32, 1};
        if ((rc = make_tmap(&p.tmap_c, a->ptr_c, 3, d, st, bx, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16))) return rc;
        p.c_tma = 1;
    }
    p.c = a->ptr_c;
    p.sfa = static_cast<const float*>(a->ptr_sfa);
    p.sfb = static_cast<const float*>(a->ptr_sfb);
    p.scale_a = a->scale_mode == B200_SCALE_TENSOR ? a->ptr_scale_a : nullptr;
    p.scale_b = a->scale_mode == B200_SCALE_TENSOR ? a->ptr_scale_b : nullptr;
    p.ldc = a->stride_c;
    p.c_batch = a->stride_c_batch;
    p.m = static_cast<int>(a->m);
    p.n = static_cast<int>(a->n);
    p.k = static_cast<int>(a->k);
    p.batch = static_cast<int>(a->batch);
    p.tiles_m = static_cast<int>((a->m + BMT - 1) / BMT);
    p.tiles_n = static_cast<int>((a->n + BN - 1) / BN);
    const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batch;
    if (total > 0x7FFFFFFF) return B200_ERR_TOO_LARGE;
    p.tiles_total = static_cast<int>(total);
    p.kblocks = static_cast<int>((a->k + 127) / 128);
    p.out_dtype = a->out_dtype;
    p.inputs_ready = (a->flags & (B200_GEMM_INPUTS_READY | B200_GEMM_BATCH_READY)) ? 1 : 0;
    p.b_shared = b_shared ? 1 : 0;
    if (a->flags & B200_GEMM_BATCH_READY) {
        p.batch_ready = reinterpret_cast<const int*>(a->ptr_batch_ready);
        p.batch_epoch = a->batch_epoch;
    }
    p.status = ds->status_ptr;
    if (a->scale_mode == B200_SCALE_MX) {
        // atoms [K/128][rows/128][512 B]: strides in atoms, batch strides in bytes
        p.sfa_stride = (a->m + 127) / 128;
        p.sfb_stride = (a->n + 127) / 128;
        p.sfa_batch = a->stride_sfa_batch;
        p.sfb_batch = a->stride_sfb_batch;
    } else {
        p.sfa_stride = a->stride_sfa;
        p.sfb_stride = a->stride_sfb;
        p.sfa_batch = a->stride_sfa_batch;
        p.sfb_batch = a->stride_sfb_batch;
    }
    if (pair && BN == 256 && !ab16 && a->scale_mode == B200_SCALE_BLOCK && a->b_layout == B200_B_NK_ROWMAJOR) {
        plan_tail(p, pair_capacity<256, MODE_BLOCK, BL_NK>(ds->sm_count));
        if (p.tail_split) {
            rc = make_rowmajor_tmap(&p.tmap_b_tail, a->ptr_b, a->n, a->k, a->stride_b, b_batches, a->stride_b_batch,
                                    static_cast<uint32_t>(BROWS / p.tail_split));
            if (rc) return rc;
        }
    }
    if (ab16) {
        const bool flat16 = a->b_layout == B200_B_FLAT_16x16;
        if (pair) return flat16 ? launch_pair<256, MODE_ACC16, BL_FLAT>(p, ds->sm_count, st) : launch_pair<256, MODE_ACC16, BL_NK>(p, ds->sm_count, st);
        const int grid16 = p.tiles_total < ds->sm_count ? p.tiles_total : ds->sm_count;
        if (BN == 256) return flat16 ? launch_gemm<256, MODE_ACC16, BL_FLAT>(p, grid16, st) : launch_gemm<256, MODE_ACC16, BL_NK>(p, grid16, st);
        return flat16 ? launch_gemm<128, MODE_ACC16, BL_FLAT>(p, grid16, st) : launch_gemm<128, MODE_ACC16, BL_NK>(p, grid16, st);
    }
    if (pair) {
        switch (BN) {
            case 256: return launch_pair_modes<256>(a, p, ds->sm_count, st);
            case 224: return launch_pair_modes<224>(a, p, ds->sm_count, st);
            case 192: return launch_pair_modes<192>(a, p, ds->sm_count, st);
            default: return launch_pair_modes<128>(a, p, ds->sm_count, st);
        }
    }
    const int grid = p.tiles_total < ds->sm_count ? p.tiles_total : ds->sm_count;
    const bool flat = a->b_layout == B200_B_FLAT_16x16;
    switch (a->scale_mode) {
        case B200_SCALE_BLOCK:
            if (BN == 256) return flat ? launch_gemm<256, MODE_BLOCK, BL_FLAT>(p, grid, st) : launch_gemm<256, MODE_BLOCK, BL_NK>(p, grid, st);
            return flat ? launch_gemm<128, MODE_BLOCK, BL_FLAT>(p, grid, st) : launch_gemm<128, MODE_BLOCK, BL_NK>(p, grid, st);
        case B200_SCALE_MX:
            return flat ? launch_gemm<128, MODE_MX, BL_FLAT>(p, grid, st) : launch_gemm<128, MODE_MX, BL_NK>(p, grid, st);
        default:
            if (BN == 256) return flat ? launch_gemm<256, MODE_ACC, BL_FLAT>(p, grid, st) : launch_gemm<256, MODE_ACC, BL_NK>(p, grid, st);
            return flat ? launch_gemm<128, MODE_ACC, BL_FLAT>(p, grid, st) : launch_gemm<128, MODE_ACC, BL_NK>(p, grid, st);
    }
}

// ---- host generators ----------------------------------------------------------------------------
inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
inline uint64_t stream_key(uint64_t seed, uint32_t tensor_id) {
    return mix64(seed ^ (static_cast<uint64_t>(tensor_id) << 32) ^ 0xA8F8A8F8ull);
}
inline uint64_t draw64(uint64_t key, uint64_t idx) { return mix64(key + idx * 0xD1342543DE82EF95ull); }

int ensure(DeviceState* ds, int slot, size_t bytes) {
    if (ds->cap[slot] >= bytes) return B200_OK;
    if (ds->buf[slot]) CU_TRY(cudaFree(ds->buf[slot]));
    ds->buf[slot] = nullptr;
    ds->cap[slot] = 0;
    const size_t want = bytes + (bytes >> 3) + 256;
    CU_TRY(cudaMalloc(&ds->buf[slot], want));
    ds->cap[slot] = want;
    return B200_OK;
}

}  // namespace

// =================================================================================================
extern "C" {

int b200_gemm_check(const b200_gemm_args* args, int32_t* chosen_tile) {
    Plan pl;
    int sms = 148;
    int rc = validate(args, sms, &pl);
    if (rc == B200_OK && chosen_tile) *chosen_tile = pl.tile;
    return rc;
}

int b200_gemm_a8w8(const b200_gemm_args* args, void* cuda_stream) {
    Plan pl;
    int rc = validate(args, 148, &pl);
    if (rc) return rc;
    DeviceState* ds = nullptr;
    rc = device_state(&ds);
    if (rc) return rc;
    rc = validate(args, ds->sm_count, &pl);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (pl.tile == B200_TILE_DECODE) return run_decode(args, pl, ds, st);
    return run_gemm(args, pl, ds, st);
}

// bf16 operands: the same pipeline on the byte view of the problem (a bf16 row of K elements is a row of 2K bytes;
// tile bytes, swizzle and descriptor steps are those of the 8-bit path), with kind::f16 MMAs
static int byte_view16(const b200_gemm_args* a, b200_gemm_args* v) {
    if (!a) return B200_ERR_BAD_ARG;
    if (a->k > 0x3FFFFFFF) return B200_ERR_TOO_LARGE;
    *v = *a;
    v->k = a->k * 2;
    v->stride_a = a->stride_a * 2;
    v->stride_b = a->stride_b * 2;
    v->stride_a_batch = a->stride_a_batch * 2;
    v->stride_b_batch = a->stride_b_batch * 2;
    return B200_OK;
}
int b200_gemm_a16w16_check(const b200_gemm_args* args, int32_t* chosen_tile) {
    b200_gemm_args v;
    int rc = byte_view16(args, &v);
    if (rc) return rc;
    Plan pl;
    rc = validate(&v, 148, &pl, true);
    if (rc == B200_OK && chosen_tile) *chosen_tile = pl.tile;
    return rc;
}
int b200_gemm_a16w16(const b200_gemm_args* args, void* cuda_stream) {
    b200_gemm_args v;
    int rc = byte_view16(args, &v);
    if (rc) return rc;
    Plan pl;
    rc = validate(&v, 148, &pl, true);
    if (rc) return rc;
    DeviceState* ds = nullptr;
    rc = device_state(&ds);
    if (rc) return rc;
    rc = validate(&v, ds->sm_count, &pl, true);
    if (rc) return rc;
    return run_gemm(&v, pl, ds, static_cast<cudaStream_t>(cuda_stream), true);
}

int b200_gemm_a8w8_decode_static(const b200_gemm_args* args, void* cuda_stream) {
    Plan pl;
    int rc = validate(args, 148, &pl);
    if (rc) return rc;
    DeviceState* ds = nullptr;
    rc = device_state(&ds);
    if (rc) return rc;
    rc = validate(args, ds->sm_count, &pl);
    if (rc) return rc;
    if (pl.tile != B200_TILE_DECODE) return B200_ERR_UNSUPPORTED;      // only the skinny-M kernel has this variant
    return run_decode(args, pl, ds, static_cast<cudaStream_t>(cuda_stream), true);
}

int b200_gemm_a8w8_simple(const b200_gemm_args* a, void* cuda_stream) {
    if (!a || !a->ptr_a || !a->ptr_b || !a->ptr_c) return B200_ERR_BAD_ARG;
    if (a->m <= 0 || a->n <= 0 || a->k <= 0 || a->batch <= 0 || a->m > 65535 * 1LL * 65535 || a->batch > 65535) return B200_ERR_BAD_ARG;
    if (a->m > 65535) return B200_ERR_TOO_LARGE;
    if ((a->scale_mode == B200_SCALE_BLOCK || a->scale_mode == B200_SCALE_MX) && (!a->ptr_sfa || !a->ptr_sfb)) return B200_ERR_BAD_ARG;
    SimpleParams p;
    p.a = static_cast<const uint8_t*>(a->ptr_a);
    p.b = static_cast<const uint8_t*>(a->ptr_b);
    p.c = a->ptr_c;
    p.sfa = a->ptr_sfa;
    p.sfb = a->ptr_sfb;
    p.scale_a = a->ptr_scale_a;
    p.scale_b = a->ptr_scale_b;
    p.m = a->m; p.n = a->n; p.k = a->k; p.batch = a->batch;
    p.lda = a->stride_a; p.ldb = a->stride_b; p.ldc = a->stride_c;
    p.a_batch = a->stride_a_batch; p.b_batch = a->stride_b_batch; p.c_batch = a->stride_c_batch;
    if (a->scale_mode == B200_SCALE_MX) {
        p.sfa_stride = (a->m + 127) / 128;
        p.sfb_stride = (a->n + 127) / 128;
    } else {
        p.sfa_stride = a->stride_sfa;
        p.sfb_stride = a->stride_sfb;
    }
    p.sfa_batch = a->stride_sfa_batch; p.sfb_batch = a->stride_sfb_batch;
    p.scale_mode = a->scale_mode; p.b_layout = a->b_layout; p.out_dtype = a->out_dtype;
    dim3 grid(static_cast<unsigned>((a->n + 127) / 128), static_cast<unsigned>(a->m), static_cast<unsigned>(a->batch));
    gemm_simple_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(p);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}

// End of the synchronous host-buffer entry: wait for the stream, then look at the status word, so that a launch
// that gave up (an expired wait, a pair whose CTAs disagreed on their tensor-memory address) is an error HERE and
// not a silently wrong C.  The word is left for b200_last_status() to report and clear.
static int host_entry_finish(DeviceState* ds, cudaStream_t st) {
    CU_TRY(cudaStreamSynchronize(st));
    int v = 0;
    CU_TRY(cudaMemcpy(&v, ds->status_ptr, sizeof(int), cudaMemcpyDeviceToHost));
    return v == 0 ? B200_OK : B200_ERR_DEVICE_TIMEOUT;
}

// a * b for non-negative operands, or -1 when the product does not fit in 2^46 bytes (64 TiB: far above any device)
static int64_t mul_checked(int64_t a, int64_t b) {
    if (a < 0 || b < 0) return -1;
    if (a == 0 || b == 0) return 0;
    if (a > (int64_t(1) << 46) / b) return -1;
    return a * b;
}

int b200_gemm_a8w8_host(const b200_gemm_args* h, void* cuda_stream) {
    Plan pl;
    if (!h || !h->ptr_a || !h->ptr_b || !h->ptr_c) return B200_ERR_BAD_ARG;
    if (h->flags & B200_GEMM_BATCH_READY) return B200_ERR_UNSUPPORTED;       // ready words are device memory
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    // validate before anything is allocated, copied or queued: the same checks as the device entry, run on a copy
    // whose operand pointers are stand-ins with the alignment the library's own buffers will have
    {
        b200_gemm_args probe = *h;
        probe.ptr_a = probe.ptr_b = probe.ptr_c = reinterpret_cast<void*>(uintptr_t(256));
        if (h->scale_mode == B200_SCALE_BLOCK || h->scale_mode == B200_SCALE_MX) {
            if (!h->ptr_sfa || !h->ptr_sfb) return B200_ERR_BAD_ARG;
            probe.ptr_sfa = probe.ptr_sfb = reinterpret_cast<void*>(uintptr_t(256));
        }
        if ((rc = validate(&probe, ds->sm_count, &pl))) return rc;
        if (h->b_layout == B200_B_NK_ROWMAJOR && h->stride_b < h->k) return B200_ERR_BAD_ARG;
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int64_t esz = h->out_dtype == B200_OUT_BF16 ? 2 : 4;
    const int64_t a_sz = h->batch > 1 ? mul_checked(h->stride_a_batch, h->batch) : mul_checked(h->stride_a, h->m);
    const int64_t b_sz = h->batch > 1 ? mul_checked(h->stride_b_batch, h->batch)
                                      : (h->b_layout == B200_B_FLAT_16x16 ? mul_checked(h->n, h->k) : mul_checked(h->stride_b, h->n));
    const int64_t c_sz = mul_checked(h->batch > 1 ? mul_checked(h->stride_c_batch, h->batch) : mul_checked(h->stride_c, h->m), esz);
    int64_t sfa_sz = 0, sfb_sz = 0;
    if (h->scale_mode == B200_SCALE_BLOCK) {
        sfa_sz = mul_checked(h->batch > 1 ? mul_checked(h->stride_sfa_batch, h->batch) : mul_checked(h->stride_sfa, h->k / 128), 4);
        sfb_sz = mul_checked(h->batch > 1 ? mul_checked(h->stride_sfb_batch, h->batch) : mul_checked(h->stride_sfb, h->n / 128), 4);
    } else if (h->scale_mode == B200_SCALE_MX) {
        sfa_sz = h->batch > 1 ? mul_checked(h->stride_sfa_batch, h->batch) : static_cast<int64_t>(b200_mx_sf_bytes(h->m, h->k));
        sfb_sz = h->batch > 1 ? mul_checked(h->stride_sfb_batch, h->batch) : static_cast<int64_t>(b200_mx_sf_bytes(h->n, h->k));
    }
    if (a_sz <= 0 || b_sz <= 0 || c_sz <= 0 || sfa_sz < 0 || sfb_sz < 0) return B200_ERR_BAD_ARG;   // zero, negative or overflowing
    const size_t a_bytes = static_cast<size_t>(a_sz), b_bytes = static_cast<size_t>(b_sz), c_bytes = static_cast<size_t>(c_sz);
    const size_t sfa_bytes = static_cast<size_t>(sfa_sz), sfb_bytes = static_cast<size_t>(sfb_sz);
    // the staging buffers, the copy stream and its events are per device: one caller at a time
    std::lock_guard<std::mutex> entry(ds->host_entry_mu);
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if ((rc = ensure(ds, 0, a_bytes)) || (rc = ensure(ds, 1, b_bytes)) || (rc = ensure(ds, 2, c_bytes)) ||
            (rc = ensure(ds, 3, sfa_bytes + 16)) || (rc = ensure(ds, 4, sfb_bytes + 16)) || (rc = ensure(ds, 5, 64)))
            return rc;
    }
    b200_gemm_args d = *h;
    d.ptr_a = ds->buf[0];
    d.ptr_b = ds->buf[1];
    d.ptr_c = ds->buf[2];
    rc = validate(&d, ds->sm_count, &pl);
    if (rc) return rc;
    CU_TRY(cudaMemcpyAsync(ds->buf[1], h->ptr_b, b_bytes, cudaMemcpyHostToDevice, st));
    if (sfa_bytes) {
        CU_TRY(cudaMemcpyAsync(ds->buf[3], h->ptr_sfa, sfa_bytes, cudaMemcpyHostToDevice, st));
        CU_TRY(cudaMemcpyAsync(ds->buf[4], h->ptr_sfb, sfb_bytes, cudaMemcpyHostToDevice, st));
        d.ptr_sfa = ds->buf[3];
        d.ptr_sfb = ds->buf[4];
    }
    if (h->scale_mode == B200_SCALE_TENSOR) {
        float* sc = static_cast<float*>(ds->buf[5]);
        if (h->ptr_scale_a) {
            CU_TRY(cudaMemcpyAsync(sc, h->ptr_scale_a, 4, cudaMemcpyHostToDevice, st));
            d.ptr_scale_a = sc;
        }
        if (h->ptr_scale_b) {
            CU_TRY(cudaMemcpyAsync(sc + 1, h->ptr_scale_b, 4, cudaMemcpyHostToDevice, st));
            d.ptr_scale_b = sc + 1;
        }
    }
    // Large single-batch problems run as row slabs: the copy-back of slab i (the largest transfer of the call)
    // proceeds on a second stream while slab i+1 is uploaded and computed, so the two PCIe directions overlap.
    // (MX scale atoms are indexed by the full M, so MX problems take the single-shot path.)
    const int64_t slab_rows = ((h->m + 7) / 8 + 255) / 256 * 256;
    const bool slabs = h->batch == 1 && h->m >= 2048 && h->scale_mode != B200_SCALE_MX && (h->m + slab_rows - 1) / slab_rows <= 16;
    if (!slabs) {
        CU_TRY(cudaMemcpyAsync(ds->buf[0], h->ptr_a, a_bytes, cudaMemcpyHostToDevice, st));
        rc = b200_gemm_a8w8(&d, st);
        if (rc) return rc;
        CU_TRY(cudaMemcpyAsync(h->ptr_c, ds->buf[2], c_bytes, cudaMemcpyDeviceToHost, st));
        return host_entry_finish(ds, st);
    }
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!ds->copy_stream) {
            CU_TRY(cudaStreamCreateWithFlags(&ds->copy_stream, cudaStreamNonBlocking));
            for (auto& e : ds->slab_done) CU_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            CU_TRY(cudaEventCreateWithFlags(&ds->copies_done, cudaEventDisableTiming));
        }
    }
    int slab = 0;
    for (int64_t r0 = 0; r0 < h->m; r0 += slab_rows, ++slab) {
        const int64_t rows = (h->m - r0) < slab_rows ? (h->m - r0) : slab_rows;
        b200_gemm_args s = d;
        s.m = rows;
        s.ptr_a = static_cast<const uint8_t*>(d.ptr_a) + r0 * h->stride_a;
        s.ptr_c = static_cast<uint8_t*>(d.ptr_c) + static_cast<size_t>(r0) * h->stride_c * esz;
        if (h->scale_mode == B200_SCALE_BLOCK) s.ptr_sfa = static_cast<const float*>(d.ptr_sfa) + r0;   // [K/128][M]: same pitch
        CU_TRY(cudaMemcpyAsync(const_cast<void*>(s.ptr_a), static_cast<const uint8_t*>(h->ptr_a) + r0 * h->stride_a,
                               static_cast<size_t>(rows * h->stride_a), cudaMemcpyHostToDevice, st));
        rc = b200_gemm_a8w8(&s, st);
        if (rc) return rc;
        CU_TRY(cudaEventRecord(ds->slab_done[slab], st));
        CU_TRY(cudaStreamWaitEvent(ds->copy_stream, ds->slab_done[slab], 0));
        CU_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(h->ptr_c) + static_cast<size_t>(r0) * h->stride_c * esz, s.ptr_c,
                               static_cast<size_t>(rows * h->stride_c) * esz, cudaMemcpyDeviceToHost, ds->copy_stream));
    }
    CU_TRY(cudaEventRecord(ds->copies_done, ds->copy_stream));
    CU_TRY(cudaStreamWaitEvent(st, ds->copies_done, 0));
    return host_entry_finish(ds, st);
}

// ---- layout ----------------------------------------------------------------------------------------
static int shuffle_common(const void* src, void* dst, int64_t n, int64_t k, int32_t kn, bool to_flat, void* stream) {
    if (!src || !dst || n <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (n % 16 != 0 || k % 16 != 0) return B200_ERR_UNSUPPORTED;
    if (!aligned16(src) || !aligned16(dst)) return B200_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (kn) {
        dim3 grid(static_cast<unsigned>((n + 255) / 256), static_cast<unsigned>((k + 63) / 64));
        if (grid.y > 65535) return B200_ERR_TOO_LARGE;
        if (to_flat) shuffle_kn_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), n, k);
        else shuffle_kn_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), n, k);
    } else {
        dim3 grid(static_cast<unsigned>((k / 16 + 15) / 16), static_cast<unsigned>(n / 16));
        if (grid.y > 65535) return B200_ERR_TOO_LARGE;
        if (to_flat) shuffle_nk_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), n, k);
        else shuffle_nk_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), n, k);
    }
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
int b200_shuffle_b(const void* src, void* dst, int64_t n, int64_t k, int32_t src_is_kn, void* stream) {
    return shuffle_common(src, dst, n, k, src_is_kn, true, stream);
}
int b200_unshuffle_b(const void* flat, void* dst, int64_t n, int64_t k, int32_t dst_is_kn, void* stream) {
    return shuffle_common(flat, dst, n, k, dst_is_kn, false, stream);
}

static int shuffle16_common(const void* src, void* dst, int64_t n, int64_t k, int32_t kn, bool to_flat, void* stream) {
    if (!src || !dst || n <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (n % 16 != 0 || k % 8 != 0) return B200_ERR_UNSUPPORTED;
    if (!kn) return shuffle_common(src, dst, n, 2 * k, 0, to_flat, stream);      // [N][K] bf16 = [N][2K] bytes
    if (!aligned16(src) || !aligned16(dst)) return B200_ERR_UNSUPPORTED;
    dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((k + 63) / 64));
    if (grid.y > 65535) return B200_ERR_TOO_LARGE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (to_flat) shuffle_kn16_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), n, k);
    else shuffle_kn16_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), n, k);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
int b200_shuffle_b_bf16(const void* src, void* dst, int64_t n, int64_t k, int32_t src_is_kn, void* stream) {
    return shuffle16_common(src, dst, n, k, src_is_kn, true, stream);
}
int b200_unshuffle_b_bf16(const void* flat, void* dst, int64_t n, int64_t k, int32_t dst_is_kn, void* stream) {
    return shuffle16_common(flat, dst, n, k, dst_is_kn, false, stream);
}

// ---- quantisers ------------------------------------------------------------------------------------
static unsigned grid_for(int64_t work_items, int threads) {
    int64_t blocks = (work_items + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}
int b200_cast_e4m3(const float* x, void* q, int64_t count, void* stream) {
    if (!x || !q || count <= 0) return B200_ERR_BAD_ARG;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 3)) return B200_ERR_UNSUPPORTED;
    cast_e4m3_kernel<<<grid_for(count / 4 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<uint8_t*>(q), count);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
size_t b200_quantize_tensor_workspace(void) { return 256; }
int b200_quantize_tensor(const float* x, void* q, float* scale, int64_t count, void* workspace, void* stream) {
    if (!x || !q || !scale || !workspace || count <= 0) return B200_ERR_BAD_ARG;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(workspace) & 3)) return B200_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int* amax = static_cast<unsigned int*>(workspace);
    CU_TRY(cudaMemsetAsync(amax, 0, sizeof(unsigned int), st));
    amax_kernel<<<grid_for(count / 4 + 1, 256), 256, 0, st>>>(x, count, amax);
    CU_TRY(cudaGetLastError());
    quant_tensor_kernel<<<grid_for(count / 4 + 1, 256), 256, 0, st>>>(x, static_cast<uint8_t*>(q), scale, count, amax);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(2);
    return B200_OK;
}
int b200_quantize_1x128(const float* x, void* q, float* sfa, int64_t m, int64_t k, void* stream) {
    if (!x || !q || !sfa || m <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (k % 128 != 0 || !aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 3)) return B200_ERR_UNSUPPORTED;
    const int64_t warps = m * (k / 128);
    const int64_t blocks = (warps + 7) / 8;
    if (blocks > 0x7FFFFFFF) return B200_ERR_TOO_LARGE;
    quant_1x128_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<uint8_t*>(q), sfa, m, k);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
// persistent grid of the probe kernels: two 1024-thread blocks per SM, fewer for small buffers
static unsigned membw_grid(int sm_count, unsigned long long n16) {
    const unsigned long long want = (n16 + 1023) / 1024;
    const unsigned long long cap = static_cast<unsigned long long>(sm_count) * 2;
    return static_cast<unsigned>(want < cap ? (want ? want : 1) : cap);
}
int b200_membw_read(const void* src, size_t bytes, uint32_t* word_sum, void* stream) {
    if (!src || !word_sum || bytes == 0) return B200_ERR_BAD_ARG;
    if (bytes % 16 != 0 || !aligned16(src)) return B200_ERR_UNSUPPORTED;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    const unsigned long long n16 = bytes / 16;
    membw_read_kernel<<<membw_grid(ds->sm_count, n16), 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), n16, word_sum);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
int b200_membw_copy(const void* src, void* dst, size_t bytes, void* stream) {
    if (!src || !dst || bytes == 0) return B200_ERR_BAD_ARG;
    if (bytes % 16 != 0 || !aligned16(src) || !aligned16(dst)) return B200_ERR_UNSUPPORTED;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    const unsigned long long n16 = bytes / 16;
    membw_copy_kernel<<<membw_grid(ds->sm_count, n16), 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), n16);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
int b200_quantize_act_bf16_1x128(const void* x_bf16, int64_t ldx, void* q, int64_t ldq, float* sfa, int64_t stride_sfa,
                                 int64_t m, int64_t k, void* stream) {
    if (!x_bf16 || !q || !sfa || m <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (ldx < k || ldq < k || stride_sfa < m) return B200_ERR_BAD_ARG;
    // 16-byte loads of eight bf16 and 8-byte stores of eight e4m3: pitches and bases must keep that alignment
    if (k % 128 != 0 || ldx % 8 != 0 || ldq % 8 != 0 || (reinterpret_cast<uintptr_t>(x_bf16) & 15) ||
        (reinterpret_cast<uintptr_t>(q) & 7))
        return B200_ERR_UNSUPPORTED;
    const int64_t gx = (k / 128 + 15) / 16, gy = (m + 31) / 32;
    if (gy > 65535) {
        // rows beyond the grid's y range: run in slabs of 65535 x 32 rows
        int rc = B200_OK;
        const int64_t slab = 65535LL * 32;
        for (int64_t r = 0; r < m && rc == B200_OK; r += slab) {
            const int64_t mm = (m - r) < slab ? (m - r) : slab;
            rc = b200_quantize_act_bf16_1x128(static_cast<const uint16_t*>(x_bf16) + r * ldx, ldx, static_cast<uint8_t*>(q) + r * ldq,
                                              ldq, sfa + r, stride_sfa, mm, k, stream);
        }
        return rc;
    }
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    act_quant_bf16_1x128_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x_bf16), ldx, static_cast<uint8_t*>(q), ldq, sfa, stride_sfa, m, k);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
int b200_quantize_act_bf16_mx32(const void* x_bf16, int64_t ldx, void* q, int64_t ldq, void* sf_atoms, int64_t rows, int64_t k,
                                void* stream) {
    if (!x_bf16 || !q || !sf_atoms || rows <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (ldx < k || ldq < k) return B200_ERR_BAD_ARG;
    if (k % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0 || (reinterpret_cast<uintptr_t>(x_bf16) & 7) ||
        (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(sf_atoms) & 3))
        return B200_ERR_UNSUPPORTED;
    const int64_t gx = (k / 128 + 7) / 8, gy = ((rows + 127) / 128) * 4;
    if (gy > 65535) return B200_ERR_TOO_LARGE;          // more than 2,097,120 rows
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    act_quant_bf16_mx32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x_bf16), ldx, static_cast<uint8_t*>(q), ldq, static_cast<uint32_t*>(sf_atoms), rows, k);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
int b200_quantize_128x128(const float* x, void* q, float* sfb, int64_t n, int64_t k, void* stream) {
    if (!x || !q || !sfb || n <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (n % 128 != 0 || k % 128 != 0 || !aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 3)) return B200_ERR_UNSUPPORTED;
    dim3 grid(static_cast<unsigned>(k / 128), static_cast<unsigned>(n / 128));
    if (grid.y > 65535) return B200_ERR_TOO_LARGE;
    quant_128x128_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<uint8_t*>(q), sfb, n, k);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
int b200_quantize_mx32(const float* x, void* q, void* sf, int64_t rows, int64_t k, void* stream) {
    if (!x || !q || !sf || rows <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (k % 32 != 0 || !aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 3)) return B200_ERR_UNSUPPORTED;
    const int64_t threads = rows * (k / 32) * 8;
    const int64_t blocks = (threads + 255) / 256;
    if (blocks > 0x7FFFFFFF) return B200_ERR_TOO_LARGE;
    quant_mx32_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), rows, k);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}
size_t b200_mx_sf_bytes(int64_t rows, int64_t k) {
    if (rows <= 0 || k <= 0) return 0;
    return static_cast<size_t>((k + 127) / 128) * static_cast<size_t>((rows + 127) / 128) * 512;
}
int b200_mx_sf_relayout(const void* sf_logical, void* sf_atoms, int64_t rows, int64_t k, void* stream) {
    if (!sf_logical || !sf_atoms || rows <= 0 || k <= 0) return B200_ERR_BAD_ARG;
    if (k % 128 != 0 || (reinterpret_cast<uintptr_t>(sf_logical) & 3) || !aligned16(sf_atoms)) return B200_ERR_UNSUPPORTED;
    const int64_t words = (k / 128) * ((rows + 127) / 128) * 128;
    const int64_t blocks = (words + 255) / 256;
    if (blocks > 0x7FFFFFFF) return B200_ERR_TOO_LARGE;
    mx_sf_relayout_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(sf_logical), static_cast<uint32_t*>(sf_atoms), rows, k);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return B200_OK;
}

// ---- seeded inputs ---------------------------------------------------------------------------------
void b200_fill_uniform(float* out, size_t count, uint64_t seed, uint32_t tensor_id, float lo, float hi) {
    const uint64_t key = stream_key(seed, tensor_id);
    const float span = hi - lo;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < static_cast<long long>(count); ++i) {
        const uint32_t r = static_cast<uint32_t>(draw64(key, static_cast<uint64_t>(i)) >> 40);
        const float u = static_cast<float>(r) * (1.0f / 16777216.0f);
        volatile float prod = span * u;      // keep the multiply and the add separately rounded
        out[i] = lo + prod;
    }
}
void b200_fill_normal(float* out, size_t count, uint64_t seed, uint32_t tensor_id) {
    const uint64_t key = stream_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < static_cast<long long>(count); ++i) {
        const uint64_t d = draw64(key, static_cast<uint64_t>(i));
        const uint32_t r1 = static_cast<uint32_t>(d >> 40);
        const uint32_t r2 = static_cast<uint32_t>(d >> 8) & 0xFFFFFFu;
        const double u1 = (static_cast<double>(r1) + 1.0) * (1.0 / 16777216.0);
        const double u2 = static_cast<double>(r2) * (1.0 / 16777216.0);
        out[i] = static_cast<float>(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
    }
}

// ---- status ------------------------------------------------------------------------------------------
int b200_last_status(void) {
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    CU_TRY(cudaDeviceSynchronize());
    int v = 0;
    CU_TRY(cudaMemcpy(&v, ds->status_ptr, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) CU_TRY(cudaMemset(ds->status_ptr, 0, sizeof(int)));
    return v;
}
int b200_peek_status(void) {
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    {
        // (created on first use, not with the per-device state: the allocation-free entry point must not create anything)
        std::lock_guard<std::mutex> lk(g_mu);
        if (!ds->peek_stream) CU_TRY(cudaStreamCreateWithFlags(&ds->peek_stream, cudaStreamNonBlocking));
    }
    int v = 0;
    CU_TRY(cudaMemcpyAsync(&v, ds->status_ptr, sizeof(int), cudaMemcpyDeviceToHost, ds->peek_stream));
    CU_TRY(cudaStreamSynchronize(ds->peek_stream));
    return v;
}
int b200_flag_write(int32_t* flag, int32_t value, void* cuda_stream) {
    if (!flag || (reinterpret_cast<uintptr_t>(flag) & 3)) return B200_ERR_BAD_ARG;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (g_write_value32) {
        const CUresult r = g_write_value32(reinterpret_cast<CUstream>(st), reinterpret_cast<CUdeviceptr>(flag),
                                           static_cast<cuuint32_t>(value), 0 /* CU_STREAM_WRITE_VALUE_DEFAULT */);
        if (r == CUDA_SUCCESS) return B200_OK;
        g_last_cuda = 100000 + static_cast<int>(r);
        return B200_ERR_CUDA;
    }
    // A driver without stream memory operations: a one-thread kernel could do the write, but it would need an SM,
    // and the consumer of these words is a persistent GEMM that may hold every SM while it waits for them.
    return B200_ERR_UNSUPPORTED;
}
int b200_flag_wait(const int32_t* flag, int32_t value, void* cuda_stream) {
    if (!flag || (reinterpret_cast<uintptr_t>(flag) & 3)) return B200_ERR_BAD_ARG;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    if (!g_wait_value32) return B200_ERR_UNSUPPORTED;
    const CUresult r = g_wait_value32(reinterpret_cast<CUstream>(cuda_stream), reinterpret_cast<CUdeviceptr>(flag),
                                      static_cast<cuuint32_t>(value), 0x0 /* CU_STREAM_WAIT_VALUE_GEQ */);
    if (r == CUDA_SUCCESS) return B200_OK;
    g_last_cuda = 100000 + static_cast<int>(r);
    return B200_ERR_CUDA;
}
int b200_stream_copy(void* dst, const void* src, size_t bytes, void* cuda_stream) {
    if (!dst || !src || bytes == 0) return B200_ERR_BAD_ARG;
    CU_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(cuda_stream)));
    return B200_OK;
}
int b200_ipc_alloc(size_t bytes, void** dev_ptr, void* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    if (!dev_ptr || !handle64 || bytes == 0) return B200_ERR_BAD_ARG;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    void* p = nullptr;
    CU_TRY(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        g_last_cuda = static_cast<int>(e);
        cudaFree(p);
        return B200_ERR_CUDA;
    }
    std::memcpy(handle64, &h, sizeof(h));
    *dev_ptr = p;
    return B200_OK;
}
int b200_ipc_open(const void* handle64, void** dev_ptr) {
    if (!handle64 || !dev_ptr) return B200_ERR_BAD_ARG;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    CU_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *dev_ptr = p;
    return B200_OK;
}
int b200_ipc_close(void* dev_ptr) {
    if (!dev_ptr) return B200_ERR_BAD_ARG;
    CU_TRY(cudaIpcCloseMemHandle(dev_ptr));
    return B200_OK;
}
int b200_ipc_free(void* dev_ptr) {
    if (!dev_ptr) return B200_ERR_BAD_ARG;
    CU_TRY(cudaFree(dev_ptr));
    return B200_OK;
}
size_t b200_slab_bytes(int64_t slab_rows, int64_t k) {
    if (slab_rows <= 0 || k <= 0 || k % 128 != 0 || slab_rows % 4 != 0) return 0;
    return static_cast<size_t>(slab_rows) * static_cast<size_t>(k) + 4 * static_cast<size_t>(k / 128) * static_cast<size_t>(slab_rows);
}
int b200_slab_upload(const void* host_a, const float* host_sfa, void* dev_slabs, int64_t m, int64_t k, int64_t slab_rows,
                     int64_t slab, void* cuda_stream) {
    if (!host_a || !host_sfa || !dev_slabs || m <= 0 || slab < 0) return B200_ERR_BAD_ARG;
    const size_t bytes = b200_slab_bytes(slab_rows, k);
    if (bytes == 0) return B200_ERR_UNSUPPORTED;
    if (m % slab_rows != 0 || (slab + 1) * slab_rows > m) return B200_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    uint8_t* dst = static_cast<uint8_t*>(dev_slabs) + static_cast<size_t>(slab) * bytes;
    const size_t a_bytes = static_cast<size_t>(slab_rows) * static_cast<size_t>(k);
    CU_TRY(cudaMemcpyAsync(dst, static_cast<const uint8_t*>(host_a) + static_cast<size_t>(slab) * a_bytes, a_bytes,
                           cudaMemcpyHostToDevice, st));
    // the slab's columns of every K group: K/128 rows of slab_rows floats, source pitch M floats
    CU_TRY(cudaMemcpy2DAsync(dst + a_bytes, static_cast<size_t>(slab_rows) * 4, host_sfa + slab * slab_rows,
                             static_cast<size_t>(m) * 4, static_cast<size_t>(slab_rows) * 4, static_cast<size_t>(k / 128),
                             cudaMemcpyHostToDevice, st));
    return B200_OK;
}
int b200_selftest_bounded_wait(int64_t budget_us, int32_t polling, void* cuda_stream) {
    if (budget_us < 100 || budget_us > 100000) return B200_ERR_BAD_ARG;          // 0.1 ms .. 100 ms
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if ((rc = ensure(ds, 6, 64))) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    int* returned = static_cast<int*>(ds->buf[6]);
    CU_TRY(cudaMemsetAsync(returned, 0, sizeof(int), st));
    selftest_bounded_wait_kernel<<<1, 64, 0, st>>>(ds->status_ptr, static_cast<unsigned long long>(budget_us) * 1000ull,
                                                   polling, returned);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(st));
    int n = 0;
    CU_TRY(cudaMemcpy(&n, returned, sizeof(int), cudaMemcpyDeviceToHost));
    return n == 2 ? B200_OK : B200_ERR_DEVICE_TIMEOUT;       // both waits must have returned "gave up"
}
int b200_last_cuda_error(void) { return g_last_cuda; }
int b200_weight_file_write(const char* path, int32_t b_layout, int32_t scale_mode, int64_t n, int64_t k, const void* data,
                           const void* scales) {
    return b200::weight_file_write(path, b_layout, scale_mode, n, k, data, scales);
}
int b200_weight_file_stat(const char* path, b200_weight_desc* out) { return b200::weight_file_stat(path, out); }
int b200_weight_file_read(const char* path, void* data, size_t data_capacity, void* scales, size_t scale_capacity) {
    return b200::weight_file_read(path, data, data_capacity, scales, scale_capacity);
}
const char* b200_strerror(int code) {
    switch (code) {
        case B200_OK: return "ok";
        case B200_ERR_BAD_ARG: return "bad argument";
        case B200_ERR_UNSUPPORTED: return "unsupported shape, stride or alignment";
        case B200_ERR_CUDA: return "CUDA call failed";
        case B200_ERR_DEVICE_TIMEOUT: return "bounded device wait expired";
        case B200_ERR_NO_DEVICE: return "no sm_100 device";
        case B200_ERR_TOO_LARGE: return "request exceeds an internal capacity";
        case B200_ERR_IO: return "weight file i/o failed";
        case B200_ERR_CORRUPT: return "weight file checksum mismatch";
        default: return "unknown";
    }
}
int b200_sm_count(void) {
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    return rc ? rc : ds->sm_count;
}
int b200_release(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = g_dev[dev];
    for (int i = 0; i < 8; ++i) {
        if (s.buf[i]) cudaFree(s.buf[i]);
        s.buf[i] = nullptr;
        s.cap[i] = 0;
    }
    {
        int kept = 0;
        for (int i = 0; i < g_scratch_count; ++i) {
            if (g_scratch[i].dev == dev) cudaFree(g_scratch[i].ptr);
            else g_scratch[kept++] = g_scratch[i];
        }
        g_scratch_count = kept;
    }
    if (s.copy_stream) {
        cudaStreamDestroy(s.copy_stream);
        s.copy_stream = nullptr;
        for (auto& e : s.slab_done) {
            cudaEventDestroy(e);
            e = nullptr;
        }
        cudaEventDestroy(s.copies_done);
        s.copies_done = nullptr;
    }
    return B200_OK;
}
const char* b200_version(void) { return "b200gemm 0.1 (sm_100a)"; }
#ifdef B200_TRACE
int b200_trace_read(long long* host, int count) {
    CU_TRY(cudaDeviceSynchronize());
    CU_TRY(cudaMemcpyFromSymbol(host, b200::g_trace, sizeof(long long) * count));
    return 0;
}
#endif
uint64_t b200_launch_count(void) { return g_launches.load(); }
int b200_last_tail_split(int32_t* first_tile, int32_t* parts) {
    if (first_tile) *first_tile = t_last_tail[0];
    if (parts) *parts = t_last_tail[1];
    return t_last_tail[1] > 0 ? 1 : 0;
}

}  // extern "C"
