/*
 * b200gemm -- C ABI of the sm_100a A8W8 FP8 (OCP E4M3) GEMM library (libb200gemm.so).
 *
 * The reference (carlushuang/gcnasm) has no plugin or FFI layer: each example's main() fills a
 * POD `kargs` struct and launches `kernel<Traits><<<grid, block>>>(kargs)` on the default
 * stream.  The entry points below sit exactly at that seam; each comment names the reference
 * launch site or host function it replaces.  All pointers are plain device (or, where stated,
 * host) addresses; no C++ or framework types cross this boundary.  Every function returns 0 on
 * success or a negative B200_ERR_* code; nothing here falls back to the CPU.
 */
#ifndef B200GEMM_H
#define B200GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums ----------------------------------------------------------------------------- */
enum b200_scale_mode {
    B200_SCALE_NONE   = 0, /* C = A.B^T, the reference's gemm_a8w8_8wave / flatmm_a8w8 semantics        */
    B200_SCALE_TENSOR = 1, /* C = (A.B^T) * scale_a * scale_b, one fp32 per tensor (device scalars)      */
    B200_SCALE_BLOCK  = 2, /* A: 1x128 groups, SFA fp32 [K/128][M]; B: 128x128 blocks, SFB [N/128][K/128] */
    B200_SCALE_MX     = 3  /* MXFP8: one E8M0 byte per 1x32 block of A and of B (see b200_mx_sf_relayout) */
};
enum b200_b_layout {
    B200_B_NK_ROWMAJOR = 0, /* B[N][K], K contiguous (gemm_a8w8_8wave.cc, block_scale_gemm)              */
    B200_B_FLAT_16x16  = 1  /* shuffle_b output [N/16][K/16][16][16] (opus_fmm/flatmm_a8w8_gfx950.cc)     */
};
enum b200_out_dtype { B200_OUT_F32 = 0, B200_OUT_BF16 = 1 };
enum b200_tile_hint {
    B200_TILE_AUTO = 0, B200_TILE_128x128 = 1, B200_TILE_128x256 = 2, B200_TILE_DECODE = 3,
    B200_TILE_PAIR_256x256 = 4, B200_TILE_128x64 = 5 /* reserved */, B200_TILE_PAIR_256x128 = 6,
    B200_TILE_PAIR_256x224 = 7, B200_TILE_PAIR_256x192 = 8   /* PAIR_*: two CTAs share a 256-row tile */
};
enum b200_error {
    B200_OK = 0,
    B200_ERR_BAD_ARG = -1,       /* null pointer, non-positive size, unknown enum                         */
    B200_ERR_UNSUPPORTED = -2,   /* shape/stride/alignment the kernels do not cover (see b200_gemm_check)  */
    B200_ERR_CUDA = -3,          /* a CUDA runtime/driver call failed; b200_last_cuda_error() has the code */
    B200_ERR_DEVICE_TIMEOUT = -4,/* a bounded device-side wait expired (b200_last_status)                  */
    B200_ERR_NO_DEVICE = -5,     /* no sm_100 device / driver entry point unavailable                      */
    B200_ERR_TOO_LARGE = -6,     /* request exceeds a fixed internal capacity or a caller's buffer          */
    B200_ERR_IO = -7,            /* weight file: cannot open / short read or write / truncated             */
    B200_ERR_CORRUPT = -8        /* weight file: checksum mismatch                                         */
};

/* ---- GEMM arguments ---------------------------------------------------------------------- */
/* Superset of the three reference kargs structs, with 64-bit strides:
 *   opus_gemm_kargs            opus_gemm/gemm_a8w8_8wave.cc:99-113
 *   opus_gemm_kargs (+scales)  opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_common.h:4-25
 *   opus_fmm_kargs             opus_fmm/flatmm_a8w8_gfx950.cc:107-122 (ptr_bias is unused there and dropped)
 * Strides are in ELEMENTS, as in the reference.  A is [batch][M][K] e4m3, B is [batch][N][K] e4m3
 * (or its flat image), C is [batch][M][N] fp32 or bf16.                                                 */
typedef struct b200_gemm_args {
    const void* ptr_a;
    const void* ptr_b;
    void*       ptr_c;
    int64_t m, n, k, batch;
    int64_t stride_a, stride_b, stride_c;                    /* row strides; stride_b ignored for flat B   */
    int64_t stride_a_batch, stride_b_batch, stride_c_batch;
    const void* ptr_sfa;          /* BLOCK: fp32 [K/128][M] (M contiguous).  MX: relayouted E8M0 bytes     */
    const void* ptr_sfb;          /* BLOCK: fp32 [N/128][K/128].             MX: relayouted E8M0 bytes     */
    int64_t stride_sfa;           /* BLOCK: elements between K groups of SFA (= M in the reference)        */
    int64_t stride_sfb;           /* BLOCK: elements between N blocks of SFB (= K/128 in the reference)    */
    int64_t stride_sfa_batch, stride_sfb_batch;
    const float* ptr_scale_a;     /* TENSOR: device fp32 scalars; null means 1.0                           */
    const float* ptr_scale_b;
    int32_t scale_mode;           /* b200_scale_mode  */
    int32_t b_layout;             /* b200_b_layout    */
    int32_t out_dtype;            /* b200_out_dtype   */
    int32_t tile_hint;            /* b200_tile_hint   */
    int32_t flags;                /* b200_gemm_flags, 0 for the reference's behaviour */
    int32_t batch_epoch;          /* B200_GEMM_BATCH_READY: the value a batch's ready word must have reached   */
    const int32_t* ptr_batch_ready; /* B200_GEMM_BATCH_READY: device int32 [batch]; null otherwise              */
} b200_gemm_args;

/* Launches on one stream are chained with programmatic dependent launch: a GEMM's prologue (barrier set-up, TMEM
 * allocation) runs while the previous kernel drains, and by default everything else waits for the previous kernel
 * to complete.
 * B200_GEMM_INPUTS_READY is the caller's promise that A, B and the scales of THIS call are not written by work
 * still in flight on the stream (for instance consecutive GEMMs of independent requests, or weights and
 * activations prepared earlier).  The 2-CTA tile kernels then start loading and multiplying at once -- on the SMs
 * the previous launch no longer uses, e.g. during its last, partly filled wave of tiles -- and only their writes to
 * C wait for the previous kernel.  The skinny-M kernel requests its first ring of WEIGHT tiles before it waits for
 * the previous kernel only when this flag is set (without it a weight written by the previous kernel -- a shuffle,
 * a quantiser, a copy -- is read only after that kernel has completed).  The single-CTA tile kernels ignore it.
 * B200_GEMM_BATCH_READY turns `batch` into a sequence of activation slabs that may still be arriving while the
 * kernel runs: before anything of batch b's A or SFA is read, the kernel waits until ptr_batch_ready[b] >=
 * batch_epoch (a bounded wait: after about 2 s the launch gives up and b200_last_status() reports 8).  Whoever delivers
 * the slab -- a copy or a collective on another stream, a peer GPU -- writes the word after the slab's last byte,
 * e.g. with b200_flag_write on the delivering stream.  B, SFB and C are not covered: B must be resident, and C is
 * ordered like any other launch.  Words only grow (use a step counter as epoch), so nothing is ever cleared.
 * Such a launch starts in plain stream order, after its predecessor has completed (no programmatic early start: its
 * first CTAs would otherwise occupy the SMs a capped grid leaves to the collective that delivers the slabs, and
 * wait there for words that collective could then never write).
 * Only the 2-CTA tile kernels implement it: M > 128 per batch and scale mode NONE, TENSOR or BLOCK, else
 * B200_ERR_UNSUPPORTED.
 * A batched problem may share one B: stride_b_batch == 0 (and stride_sfb_batch == 0) makes every batch multiply
 * by the same weights (2-CTA tile kernels and b200_gemm_a8w8_simple).                                            */
enum b200_gemm_flags { B200_GEMM_INPUTS_READY = 1, B200_GEMM_BATCH_READY = 2 };

/* Replaces the launches `gemm_a8w8_kernel<Traits><<<grid,block>>>(kargs)` (gemm_a8w8_8wave.cc:738),
 * `gemm_a8w8_blockscale_kernel<GemmTraits><<<grid,block>>>(kargs)` (gemm_a8w8_blockscale_host.cc:257)
 * and `flatmm_kernel<Traits><<<grid,block>>>(kargs)` (flatmm_a8w8_gfx950.cc:780).  Asynchronous on
 * `cuda_stream` (a cudaStream_t, 0 = default stream); buffers are caller-owned device memory.           */
int b200_gemm_a8w8(const b200_gemm_args* args, void* cuda_stream);
/* Rules of the skinny-M path (M <= 64) of b200_gemm_a8w8.  When a problem has fewer 128-row weight panels than the
 * GPU has SMs the kernel splits K and needs an fp32 workspace.  The library keeps one workspace per (device,
 * stream) -- launches on different streams never share one -- allocates it with cudaMalloc on first use or when a
 * larger one is needed, and never frees or moves a workspace that a launch has been given (b200_release frees them
 * all).  So: make the first split-K call of a stream, at the largest size it will see, before capturing that stream
 * into a CUDA graph (an allocation cannot happen inside a capture, and a captured launch keeps the pointer it was
 * given); and do not call b200_release while captured graphs that contain these launches are still replayed.      */

/* Tail of a block-scale GEMM.  The kernels are persistent: CTA pairs take tiles round by round, and the last round is
 * rarely full (448 tiles of 256 x 256 on 74 pairs: a seventh round of 4 tiles, 70 pairs idle meanwhile).  With row-major B
 * and 256 x 256 tiles the tiles of a partial last round that follows at least one whole round are each computed as 4
 * (or 2) column parts by as many pairs, when there are pairs enough for all parts: narrower MMAs over the full K, every element summed in the order of a
 * whole tile -- results do not depend on whether a tile was split.  B200GEMM_TAIL_SPLIT=0 in the environment (read
 * once) switches this off.  b200_last_tail_split reports what the calling thread's last pair-kernel launch did:
 * returns 1 and the first split tile and the parts per tile, or 0.                                              */
int b200_last_tail_split(int32_t* first_tile, int32_t* parts);

/* Validates `args` exactly as b200_gemm_a8w8 would, without touching the GPU. Also reports the tile
 * configuration the launcher would pick (a b200_tile_hint value) when `chosen_tile` is not null.        */
int b200_gemm_check(const b200_gemm_args* args, int32_t* chosen_tile);

/* Same contract as b200_gemm_a8w8 but computed by a one-thread-per-output CUDA kernel that mirrors the
 * host gemm_ref loops (gemm_a8w8_8wave.cc:601-612, gemm_a8w8_blockscale_host.cc:66-90): the device-side
 * checker for problem sizes the CPU loops cannot finish.  MX scales are read in the relayouted form.     */
int b200_gemm_a8w8_simple(const b200_gemm_args* args, void* cuda_stream);

/* Not re-entrant per device: the staging buffers, the copy stream and its events are shared, so concurrent callers on
 * one device are serialised by a per-device lock inside the call.  Arguments are validated (and byte sizes checked for
 * overflow) before anything is allocated or queued.  After the final synchronisation the device status word is read:
 * a launch that gave up makes the call return B200_ERR_DEVICE_TIMEOUT instead of delivering a wrong C.
 * Whole reference main() data path with HOST buffers (hipMemcpy H2D -> launch -> hipMemcpy D2H,
 * gemm_a8w8_blockscale_host.cc:212-226,257,262): copies the operands in `args` (host pointers) to
 * device buffers owned by the library, runs the GEMM and copies C back; returns after the copy-back.
 * Device buffers are cached per device and grown on demand; b200_release() frees them.  Single-batch problems
 * with M >= 2048 (not MX) run as row slabs whose copy-back overlaps the next slab's upload and GEMM on a second,
 * library-owned stream; the call still returns only when all of C is on the host.                        */
int b200_gemm_a8w8_host(const b200_gemm_args* host_args, void* cuda_stream);

/* No counterpart in the reference.  Skinny-M (M <= 64) GEMM with the same arguments and the same results as
 * b200_gemm_a8w8, for callers that must not allocate device memory while they run: code inside a serving
 * loop whose memory was carved up ahead of time, a real-time or latency-critical thread where cudaMalloc's
 * device-wide synchronisation is unacceptable, or a host that hands this library a fixed memory budget and
 * forbids it to grow.  b200_gemm_a8w8 may cudaMalloc (and later cudaFree) a split-K workspace when a skinny
 * problem has fewer 128-row weight panels than the GPU has SMs; this entry point never calls cudaMalloc,
 * cudaFree or any allocating routine.  Its split-K workspace is a fixed 1 MiB array inside the library image
 * (every GPU that loads the library holds it until the process exits).
 *   - Limit: splits * batch * M * N fp32 partials must fit in 1 MiB (262,144 floats); otherwise the call
 *     returns B200_ERR_TOO_LARGE and launches nothing.  Shapes the launcher would not send to the skinny-M
 *     kernel (M > 64, MX scales) return B200_ERR_UNSUPPORTED.
 *   - The first call on each device looks up that device's address of the array (and the library's other
 *     per-device set-up); make that first call before starting any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Nothing needs
 *     clearing (each launch writes every partial it later reads), but two calls that overlap on the GPU --
 *     different streams, or the same stream from different threads without ordering -- race on it.            */
int b200_gemm_a8w8_decode_static(const b200_gemm_args* args, void* cuda_stream);

/* ---- a16w16 siblings: bf16 operands -------------------------------------------------------------- */
/* Replaces the launches of opus_gemm/gemm_a16w16_8wave.cc (kernel :252-560, launch in main) and
 * opus_fmm/flatmm_a16w16_gfx950.cc (flat B): C = A * B^T with bf16 A [M][K] and B [N][K] (or the flat image of
 * b200_shuffle_b_bf16), fp32 accumulate, bf16 (what the reference writes) or fp32 output.  Same b200_gemm_args;
 * k and the A/B strides count bf16 ELEMENTS.  scale_mode NONE or TENSOR.  K % 8 == 0 (flat: K % 64 == 0, N % 16 == 0),
 * stride_a, stride_b multiples of 8, 16-byte aligned bases.  Tiles: AUTO, 128x128, 128x256, PAIR_256x256.       */
int b200_gemm_a16w16(const b200_gemm_args* args, void* cuda_stream);
int b200_gemm_a16w16_check(const b200_gemm_args* args, int32_t* chosen_tile);
/* shuffle_b<bf16> of opus_fmm/flatmm_a16w16_gfx950.cc:623-666 (ItemsPerAccess 8): [K][N] (src_is_kn != 0) or
 * [N][K] row-major bf16 -> flat [N/16][K/8][16 n][8 k]; N % 16 == 0, K % 8 == 0.  Byte-exact.                     */
int b200_shuffle_b_bf16(const void* src, void* dst, int64_t n, int64_t k, int32_t src_is_kn, void* cuda_stream);
int b200_unshuffle_b_bf16(const void* flat, void* dst, int64_t n, int64_t k, int32_t dst_is_kn, void* cuda_stream);

/* ---- weight pre-shuffle -------------------------------------------------------------------- */
/* shuffle_b (flatmm_a8w8_gfx950.cc:638-681) on the device: src is [K][N] row-major when src_is_kn != 0
 * (the reference's input) or [N][K] row-major otherwise; dst is [N/16][K/16][16][16].  Bit-exact byte
 * permutation; N % 16 == 0 and K % 16 == 0 required (asserts at :650-651).                              */
int b200_shuffle_b(const void* src, void* dst, int64_t n, int64_t k, int32_t src_is_kn, void* cuda_stream);
/* inverse: flat -> [K][N] (dst_is_kn != 0) or [N][K] */
int b200_unshuffle_b(const void* flat, void* dst, int64_t n, int64_t k, int32_t dst_is_kn, void* cuda_stream);

/* ---- quantisers (device) -------------------------------------------------------------------- */
/* The reference has no quantiser (operands are static_cast<fp8>(uniform float),
 * gemm_a8w8_blockscale_host.cc:32-44); these implement the benchmark configurations' rules:
 * scale = amax/448 (1.0 for an all-zero group), q = e4m3_rne_satfinite(x / scale).                      */
int b200_cast_e4m3(const float* x, void* q, int64_t count, void* cuda_stream);
/* workspace: at least b200_quantize_tensor_workspace() bytes of device scratch */
int b200_quantize_tensor(const float* x, void* q, float* scale, int64_t count, void* workspace, void* cuda_stream);
size_t b200_quantize_tensor_workspace(void);
int b200_quantize_1x128(const float* x, void* q, float* sfa, int64_t m, int64_t k, void* cuda_stream);   /* sfa [K/128][M] */
int b200_quantize_128x128(const float* x, void* q, float* sfb, int64_t n, int64_t k, void* cuda_stream); /* sfb [N/128][K/128] */
/* MX 1x32: e = floor(log2(amax)) - 8, byte = clamp(e + 127, 0, 254), q = e4m3(x * 2^-e); sf is [rows][K/32] */
int b200_quantize_mx32(const float* x, void* q, void* sf, int64_t rows, int64_t k, void* cuda_stream);
/* Fused activation quantisers: bf16 activations -> e4m3 operand + scales in the layout the GEMM reads, one pass
 * (no fp32 staging copy, no separate re-layout).  The reference names the scale layout
 * (block_scale_gemm/README.md:21,28: SFA is [K/128][M], M contiguous) but has no quantiser; same rules as above.
 * ldx/ldq: row pitches in elements (>= k); stride_sfa: pitch between K groups (>= m); k % 128 == 0.
 * 1x128: ldx, ldq multiples of 8, x 16-byte and q 8-byte aligned.  MX: multiples of 4, x 8-byte, q 4-byte.  */
int b200_quantize_act_bf16_1x128(const void* x_bf16, int64_t ldx, void* q, int64_t ldq, float* sfa, int64_t stride_sfa,
                                 int64_t m, int64_t k, void* cuda_stream);
/* MX 1x32 scales written directly as atoms (b200_mx_sf_bytes(rows, k) bytes), padding rows = 127 */
int b200_quantize_act_bf16_mx32(const void* x_bf16, int64_t ldx, void* q, int64_t ldq, void* sf_atoms, int64_t rows,
                                int64_t k, void* cuda_stream);
/* Re-lays logical E8M0 scales [rows][K/32] into the tensor-core atom order the MX GEMM reads:
 * [K/128][ceil(rows/128)][32][4][4] bytes, padded rows = 127 (scale 1.0).  Size: b200_mx_sf_bytes().     */
int b200_mx_sf_relayout(const void* sf_logical, void* sf_atoms, int64_t rows, int64_t k, void* cuda_stream);
size_t b200_mx_sf_bytes(int64_t rows, int64_t k);

/* ---- weight files (host only) ------------------------------------------------------------------ */
/* A pre-quantised, optionally pre-shuffled B operand with its scales on disk, so that a run does not repeat the
 * host-side layout pass the reference performs at every start (opus_fmm/flatmm_a8w8_gfx950.cc:736-742).  The
 * reference has no file format; this one is: 128-byte header below, N*K operand bytes, padding to 64, scales.
 * Little-endian.  checksum = FNV-1a/64 over operand bytes then scale bytes.  8-bit (e4m3) operands only: the header
 * has no element-size field, so the bf16 siblings' weights are not storable.  N and K are limited to 2^31.       */
typedef struct b200_weight_desc {
    char magic[8];            /* "B200WGT1" */
    int32_t version;          /* 1 */
    int32_t b_layout;         /* b200_b_layout of the operand bytes */
    int32_t scale_mode;       /* b200_scale_mode: which scales follow */
    int32_t reserved0;
    int64_t n, k;
    int64_t data_bytes;       /* n * k */
    int64_t scale_bytes;      /* NONE 0; TENSOR 4; BLOCK 4*(n/128)*(k/128); MX b200_mx_sf_bytes(n, k) (atoms) */
    uint64_t checksum;
    uint8_t reserved[64];
} b200_weight_desc;
int b200_weight_file_write(const char* path, int32_t b_layout, int32_t scale_mode, int64_t n, int64_t k, const void* data,
                           const void* scales);
int b200_weight_file_stat(const char* path, b200_weight_desc* out);
/* host buffers; B200_ERR_TOO_LARGE if a capacity is too small, B200_ERR_CORRUPT on a checksum mismatch */
int b200_weight_file_read(const char* path, void* data, size_t data_capacity, void* scales, size_t scale_capacity);

/* ---- HBM bandwidth probe ---------------------------------------------------------------------- */
/* The two streams of the reference's bandwidth_memread/bandwidth_kernel.cu (memread_kernel :67-92,
 * memcpy_kernel :94-118): read-only and read+write over a caller-owned buffer, persistent grid, 16-byte
 * accesses.  bytes % 16 == 0, pointers 16-byte aligned.  The caller times the launches.
 * read: adds the sum (mod 2^32) of all 32-bit words of the buffer to *word_sum (device memory, caller zeroes). */
int b200_membw_read(const void* src, size_t bytes, uint32_t* word_sum, void* cuda_stream);
int b200_membw_copy(const void* src, void* dst, size_t bytes, void* cuda_stream);

/* ---- seeded inputs (host) --------------------------------------------------------------------- */
/* The reference draws inputs from std::random_device (gemm_a8w8_8wave.cc:570-571), which cannot be
 * reproduced; these counter-based generators replace it.  Element i depends only on (seed, tensor_id, i). */
void b200_fill_uniform(float* host_out, size_t count, uint64_t seed, uint32_t tensor_id, float lo, float hi);
void b200_fill_normal(float* host_out, size_t count, uint64_t seed, uint32_t tensor_id);

/* ---- stream-ordered flag write --------------------------------------------------------------------- */
/* Writes `value` to the device word `flag` when everything queued on `cuda_stream` before this call has completed
 * (a stream memory operation: no kernel, no SM).  The producer side of B200_GEMM_BATCH_READY: queue it behind the
 * copy or collective that delivers a slab.  B200_ERR_UNSUPPORTED on a driver without stream memory operations.
 * No counterpart in the reference (its kernels never wait for data).                                             */
int b200_flag_write(int32_t* flag, int32_t value, void* cuda_stream);

/* ---- peer memory: slabs pushed from GPU to GPU by the copy engines ------------------------------------------- */
/* For the N-sharded mode with one process per GPU.  The activation of a call can travel down a chain of GPUs without
 * any kernel: every rank copies a slab it has received into the next rank's buffer with a device-to-device copy (copy
 * engines over NVLink), then writes that rank's ready word; the consumer is the GEMM of B200_GEMM_BATCH_READY.  These
 * entry points are the pieces: memory another process can map, the mapping, a stream-ordered copy, and a stream-
 * ordered wait on a word.  The reference has no counterpart (one GPU, one process).
 * b200_ipc_alloc: cudaMalloc on the current device plus the 64-byte handle (cudaIpcMemHandle_t) another process on
 * the same machine passes to b200_ipc_open, which maps the memory into the caller and enables peer access between
 * the two devices.  b200_ipc_close unmaps, b200_ipc_free frees (only the allocating process, after every peer has
 * closed).  How the handle reaches the peer is the caller's business.                                             */
int b200_ipc_alloc(size_t bytes, void** dev_ptr, void* handle64);
int b200_ipc_open(const void* handle64, void** dev_ptr);
int b200_ipc_close(void* dev_ptr);
int b200_ipc_free(void* dev_ptr);
/* Copy between device buffers (this GPU's or a mapped peer's) in stream order; no kernel is launched. */
int b200_stream_copy(void* dst, const void* src, size_t bytes, void* cuda_stream);
/* Everything queued on `cuda_stream` after this call waits until the device word `flag` (this GPU's memory) holds a
 * value >= `value` (a stream memory operation: no kernel, no SM, no host thread).  The counterpart of b200_flag_write
 * for words that ANOTHER GPU writes.  Nothing bounds this wait: only wait for words whose writer is already queued.  */
int b200_flag_wait(const int32_t* flag, int32_t value, void* cuda_stream);

/* ---- activation slabs ---------------------------------------------------------------------------------- */
/* The layout in which the N-sharded mode moves a block-scale activation between GPUs and feeds it to a batched GEMM
 * (B200_GEMM_BATCH_READY): the M rows are cut into slabs of `slab_rows`, and slab s is ONE contiguous piece
 *     [ slab_rows x K e4m3 bytes | (K/128) x slab_rows fp32 scales ]
 * i.e. a complete (A, SFA) pair in the reference's layouts (block_scale_gemm/README.md:21,28) for its rows, so that a
 * slab travels as a single copy or collective and the GEMM addresses slab s as batch s (stride_a_batch =
 * b200_slab_bytes, ptr_sfa = base + slab_rows * K, stride_sfa = slab_rows, stride_sfa_batch = b200_slab_bytes / 4).
 * No counterpart in the reference (single GPU, operands uploaded whole).  K % 128 == 0, slab_rows % 4 == 0.        */
size_t b200_slab_bytes(int64_t slab_rows, int64_t k);
/* Queues on `cuda_stream` the upload of rows [slab * slab_rows, +slab_rows) of a HOST activation in the reference's
 * layouts -- A [M][K] bytes, SFA fp32 [K/128][M] -- into slab `slab` of a device buffer in the slab layout: one
 * contiguous copy for the bytes, one pitched copy for the scale columns.  Pinned host memory makes it asynchronous.  */
int b200_slab_upload(const void* host_a, const float* host_sfa, void* dev_slabs, int64_t m, int64_t k, int64_t slab_rows,
                     int64_t slab, void* cuda_stream);

/* ---- status / housekeeping --------------------------------------------------------------------- */
/* Device status word of the current device: 0, or the code of the first bounded wait that expired (1-5, 8), of a
 * pair launch whose two CTAs disagreed on their tensor-memory address (6: that launch computed nothing) or of the
 * self-test (7) since the last call, which also clears it.  Synchronises the device.                         */
int b200_last_status(void);
/* The same word without synchronising and without clearing it: what has been recorded by kernels that have
 * already finished.  Cheap enough to poll between steps of a serving loop.                                   */
int b200_peek_status(void);
/* Self-test of the failure path: a one-block kernel waits, with a budget of `budget_us` (100..100000), on a barrier
 * that nothing signals (polling != 0: the test_wait flavour).  Returns B200_OK when both waiting threads gave up;
 * afterwards b200_last_status() reports 7 (the self-test's code) once, and the context stays usable.  No part of
 * the reference corresponds to this (its kernels have no waits that can be bounded).                          */
int b200_selftest_bounded_wait(int64_t budget_us, int32_t polling, void* cuda_stream);
int b200_last_cuda_error(void);
const char* b200_strerror(int code);
int b200_sm_count(void);
int b200_release(void);              /* frees cached device buffers of b200_gemm_a8w8_host              */
const char* b200_version(void);
uint64_t b200_launch_count(void);    /* kernels launched by this library in this process                  */

#ifdef __cplusplus
}
#endif
#endif /* B200GEMM_H */
