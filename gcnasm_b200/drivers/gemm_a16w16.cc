// gemm_a16w16: batched bf16 NT GEMM, C[b,M,N] = A[b,M,K] . B[b,N,K]^T, and with --flat the same product on a
// pre-shuffled weight matrix.  Host driver with the operator surface of opus_gemm/gemm_a16w16_8wave.cc:629-760
// (defaults 256x512x128 batch 8, A ~ U[0,1), B ~ U[-0.5,0.5), bf16 result, absolute threshold 0.5 at :736-739) and of
// opus_fmm/flatmm_a16w16_gfx950.cc (B created as [K,N], shuffled into [N/16][K/8][16][8], only the shuffled copy is
// used by the device, the host check reads the unshuffled matrix, :571-582).  The launches are replaced by
// b200_gemm_a16w16(); the shuffle runs on the device through b200_shuffle_b_bf16 and is compared with a host shuffle.
#include "driver_common.h"

using namespace drv;

static uint16_t f32_to_bf16_bits(float f) {                       // round to nearest even, quiet NaN
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
    return static_cast<uint16_t>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

static void fill_bf16(uint16_t* dst, size_t count, uint64_t seed, uint32_t tid, float lo, float hi) {
    std::vector<float> tmp(count);
    b200_fill_uniform(tmp.data(), count, seed, tid, lo, hi);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < static_cast<long long>(count); ++i) dst[i] = f32_to_bf16_bits(tmp[i]);
}

// gemm_ref of gemm_a16w16_8wave.cc:584-595 (b_kn == false) and of flatmm_a16w16_gfx950.cc:571-582 (b_kn == true)
static void gemm_ref(const uint16_t* a, const uint16_t* b, float* c, int m, int n, int k, bool b_kn) {
#pragma omp parallel for collapse(2)
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (int p = 0; p < k; ++p)
                sum += bf16_bits_to_f32(a[(size_t)i * k + p]) * bf16_bits_to_f32(b_kn ? b[(size_t)p * n + j] : b[(size_t)j * k + p]);
            c[(size_t)i * n + j] = bf16_bits_to_f32(f32_to_bf16_bits(sum));      // static_cast<bf16_t>(sum)
        }
}

static void shuffle_host(const uint16_t* b_kn, uint16_t* out, int n, int k) {
#pragma omp parallel for
    for (int nn = 0; nn < n; ++nn)
        for (int kk = 0; kk < k; ++kk)
            out[(size_t)(nn / 16) * ((size_t)k * 16) + (size_t)(kk / 8) * 128 + (nn % 16) * 8 + (kk % 8)] = b_kn[(size_t)kk * n + nn];
}

int main(int argc, char** argv) {
    bool flat = false, k_given = false;
    for (int i = 1; i < argc; ++i) {
        flat |= std::strcmp(argv[i], "--flat") == 0;
        k_given |= std::strcmp(argv[i], "-k") == 0 || std::strcmp(argv[i], "--k") == 0 || std::strncmp(argv[i], "-k=", 3) == 0;
    }
    Options o = parse(argc, argv, 1);
    if (!k_given) o.k = 128;                                       // gemm_a16w16_8wave.cc:651
    if (o.m <= 0 || o.n <= 0 || o.k <= 0 || o.batch <= 0) {
        std::fprintf(stderr, "Invalid problem size: M,N,K and batch must be positive.\n");
        return 1;
    }
    if (flat && (o.n % 16 != 0 || o.k % 64 != 0)) {
        std::fprintf(stderr, "flat layout needs N %% 16 == 0 and K %% 64 == 0.\n");
        return 1;
    }
    const bool f32out = o.out == "f32" && [&] { for (int i = 1; i < argc; ++i) if (std::strncmp(argv[i], "--out", 5) == 0) return true; return false; }();
    const size_t M = o.m, N = o.n, K = o.k, B = o.batch;
    std::vector<uint16_t> ha(B * M * K), hb(B * N * K);
    fill_bf16(ha.data(), ha.size(), o.seed, 0, 0.0f, 1.0f);
    fill_bf16(hb.data(), hb.size(), o.seed, 1, -0.5f, 0.5f);       // [N,K] per batch, or [K,N] with --flat
    uint16_t* da = dev_upload(ha.data(), ha.size());
    uint16_t* db = dev_upload(hb.data(), hb.size());
    bool shuffle_ok = true;
    if (flat) {
        uint16_t* dflat = nullptr;
        DRV_CUDA(cudaMalloc(&dflat, hb.size() * 2));
        std::printf("Shuffling B matrix for FlatMM layout (batch=%d)...\n", o.batch);
        for (size_t b = 0; b < B; ++b) DRV_B200(b200_shuffle_b_bf16(db + b * N * K, dflat + b * N * K, o.n, o.k, 1, nullptr));
        if (o.verify) {
            std::vector<uint16_t> got(B * N * K), want(N * K);
            DRV_CUDA(cudaMemcpy(got.data(), dflat, got.size() * 2, cudaMemcpyDeviceToHost));
            for (size_t b = 0; b < B; ++b) {
                shuffle_host(hb.data() + b * N * K, want.data(), o.n, o.k);
                shuffle_ok = shuffle_ok && std::memcmp(want.data(), got.data() + b * N * K, N * K * 2) == 0;
            }
            std::printf("[shuffle_b] device vs host: %s\n", shuffle_ok ? "BIT-EXACT" : "MISMATCH");
        }
        cudaFree(db);
        db = dflat;
    }
    void* dc = nullptr;
    DRV_CUDA(cudaMalloc(&dc, B * M * N * (f32out ? 4 : 2)));

    b200_gemm_args args{};
    args.ptr_a = da; args.ptr_b = db; args.ptr_c = dc;
    args.m = o.m; args.n = o.n; args.k = o.k; args.batch = o.batch;
    args.stride_a = o.k; args.stride_b = flat ? o.n : o.k; args.stride_c = o.n;
    args.stride_a_batch = (int64_t)M * K; args.stride_b_batch = (int64_t)N * K; args.stride_c_batch = (int64_t)M * N;
    args.scale_mode = B200_SCALE_NONE;
    args.b_layout = flat ? B200_B_FLAT_16x16 : B200_B_NK_ROWMAJOR;
    args.out_dtype = f32out ? B200_OUT_F32 : B200_OUT_BF16;
    args.tile_hint = o.tile;

    int32_t tile = 0;
    DRV_B200(b200_gemm_a16w16_check(&args, &tile));
    std::printf("Launching %s kernel: M=%d, N=%d, K=%d, batch=%d, tile_config=%d, sms=%d\n", flat ? "FlatMM" : "GEMM", o.m, o.n, o.k,
                o.batch, tile, b200_sm_count());
    DRV_B200(b200_gemm_a16w16(&args, nullptr));
    DRV_CUDA(cudaDeviceSynchronize());
    if (int st = b200_last_status()) {
        std::fprintf(stderr, "device wait expired, status %d\n", st);
        return 1;
    }
    bool all_valid = shuffle_ok;
    if (o.verify) {
        std::vector<float> hc, ref(M * N);
        fetch_c(hc, dc, B * M * N, !f32out);
        for (size_t b = 0; b < B; ++b) {
            gemm_ref(ha.data() + b * M * K, hb.data() + b * N * K, ref.data(), o.m, o.n, o.k, flat);
            double me, mr;
            valid_relative(ref.data(), hc.data() + b * M * N, (long long)(M * N), &me, &mr);
            const bool valid = valid_vector(ref.data(), hc.data() + b * M * N, (long long)(M * N), 5e-1f);      // :736-739
            std::printf("[%s batch %zu/%zu: %dx%dx%d] %s (max_err=%.3g, max_ref=%.3g)\n", flat ? "FlatMM" : "GEMM", b + 1, B, o.m, o.n,
                        o.k, valid ? "VALID" : "FAIL", me, mr);
            all_valid = all_valid && valid;
        }
        std::printf("\n[Overall] %s\n", all_valid ? "ALL BATCHES VALID" : "SOME BATCHES FAILED");
    }
    std::printf("\n");
    // warm-up + timed loop of benchmark_kernel (gemm_a16w16_8wave.cc:598-627: 50 + 100 launches)
    const int warm = o.warmup == 200 ? 50 : o.warmup;
    for (int i = 0; i < warm; ++i) DRV_B200(b200_gemm_a16w16(&args, nullptr));
    cudaEvent_t e0, e1;
    DRV_CUDA(cudaEventCreate(&e0));
    DRV_CUDA(cudaEventCreate(&e1));
    DRV_CUDA(cudaDeviceSynchronize());
    DRV_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < o.iters; ++i) DRV_B200(b200_gemm_a16w16(&args, nullptr));
    DRV_CUDA(cudaEventRecord(e1));
    DRV_CUDA(cudaEventSynchronize(e1));
    float total = 0.0f;
    DRV_CUDA(cudaEventElapsedTime(&total, e0, e1));
    const double ms = total / o.iters;
    std::printf("Kernel Performance: avg_time=%.4f ms, %.2f TFlops\n\n", ms, 2.0 * M * N * K * B / 1e9 / ms);
    if (o.json)
        std::printf("{\"driver\": \"gemm_a16w16\", \"flat\": %s, \"m\": %d, \"n\": %d, \"k\": %d, \"batch\": %d, \"ms\": %.5f, \"tflops\": %.2f, \"valid\": %s}\n",
                    flat ? "true" : "false", o.m, o.n, o.k, o.batch, ms, 2.0 * M * N * K * B / 1e9 / ms, all_valid ? "true" : "false");
    cudaFree(da); cudaFree(db); cudaFree(dc);
    return 0;
}
