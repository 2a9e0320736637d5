// flatmm_a8w8: FP8 GEMM on a pre-shuffled ("flat") weight matrix.  Host driver with the operator surface
// of opus_fmm/flatmm_a8w8_gfx950.cc:683-821: B is created as [K,N], shuffled per batch into
// [N/16][K/16][16][16] (shuffle_b, :638-681), only the shuffled copy goes to the device, the host check
// reads the unshuffled [K,N] matrix (:586-597) with absolute threshold 0.1, benchmark 50 + 100 launches.
// The shuffle runs on the device through b200_shuffle_b and is compared byte for byte with a host
// shuffle; the launch at :780 is replaced by b200_gemm_a8w8().
// Additions: --scale block applies the block-scale semantics of gemm_a8w8_blockscale to the flat layout
// (per-token 1x128 A scales, 128x128 B scales) for decode shapes; --out bf16; --seed; --json.
// --save-weights FILE writes the shuffled operand and its block scales after the shuffle; --load-weights FILE
// starts from such a file instead of generating and shuffling B (batch 1), so that a decode run skips the
// layout pass the reference repeats at every start (:736-742).
#include "driver_common.h"

using namespace drv;

static void unshuffle_b_host(const uint8_t* flat, uint8_t* b_kn, int n, int k) {
#pragma omp parallel for
    for (int nn = 0; nn < n; ++nn)
        for (int kk = 0; kk < k; ++kk)
            b_kn[(size_t)kk * n + nn] = flat[(size_t)(nn / 16) * ((size_t)k * 16) + (size_t)(kk / 16) * 256 + (nn % 16) * 16 + (kk % 16)];
}

static void shuffle_b_host(const uint8_t* b_kn, uint8_t* out, int n, int k) {
#pragma omp parallel for
    for (int nn = 0; nn < n; ++nn)
        for (int kk = 0; kk < k; ++kk)
            out[(size_t)(nn / 16) * ((size_t)k * 16) + (size_t)(kk / 16) * 256 + (nn % 16) * 16 + (kk % 16)] = b_kn[(size_t)kk * n + nn];
}

// gemm_ref of flatmm_a8w8_gfx950.cc:586-597: b[p*ldb + j] on the UNSHUFFLED [K,N] matrix; optional block scales
static void gemm_ref_kn(const uint8_t* a, const uint8_t* b_kn, const float* sfa, const float* sfb, float* c, int m, int n, int k) {
    const float* lut = e4m3_table();
#pragma omp parallel for collapse(2)
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float sum = 0.0f;
            if (!sfa) {
                for (int p = 0; p < k; ++p) sum += lut[a[(size_t)i * k + p]] * lut[b_kn[(size_t)p * n + j]];
            } else {
                for (int g = 0; g < k / 128; ++g) {
                    const float scale = sfa[(size_t)g * m + i] * sfb[(size_t)(j / 128) * (k / 128) + g];
                    for (int p = g * 128; p < (g + 1) * 128; ++p) sum += lut[a[(size_t)i * k + p]] * lut[b_kn[(size_t)p * n + j]] * scale;
                }
            }
            c[(size_t)i * n + j] = sum;
        }
}

int main(int argc, char** argv) {
    Options o = parse(argc, argv, 1);
    bool warm_given = false;
    for (int i = 1; i < argc; ++i) warm_given |= std::strncmp(argv[i], "--warmup", 8) == 0;
    if (!warm_given) o.warmup = 50;                                    // :601
    if (o.m <= 0 || o.n <= 0 || o.k <= 0 || o.batch <= 0) {
        std::fprintf(stderr, "Invalid problem size: M,N,K and batch must be positive.\n");
        return 1;
    }
    if (o.n % 16 != 0 || o.k % 128 != 0) {
        std::fprintf(stderr, "flat layout needs N %% 16 == 0 and K %% 128 == 0.\n");
        return 1;
    }
    const bool block = o.scale == "block";
    if (block && (o.n % 128 != 0)) {
        std::fprintf(stderr, "block scales need N %% 128 == 0.\n");
        return 1;
    }
    const bool bf16 = o.out == "bf16";
    const size_t M = o.m, N = o.n, K = o.k, B = o.batch, KG = K / 128, NG = N / 128;

    const bool from_file = !o.load_weights.empty();
    if ((from_file || !o.save_weights.empty()) && o.batch != 1) {
        std::fprintf(stderr, "weight files hold one matrix: use -b 1.\n");
        return 1;
    }
    std::vector<uint8_t> ha(B * M * K), hb(B * N * K), hflat(B * N * K);
    fill_e4m3(ha.data(), ha.size(), o.seed, 0, o.dist, 0.0f, 1.0f);
    std::vector<float> hsfa, hsfb;
    if (block) {
        hsfa.resize(B * KG * M);
        hsfb.resize(B * NG * KG);
        b200_fill_uniform(hsfa.data(), hsfa.size(), o.seed, 2, 0.8f, 1.2f);
        b200_fill_uniform(hsfb.data(), hsfb.size(), o.seed, 3, 0.8f, 1.2f);
    }
    uint8_t* da = dev_upload(ha.data(), ha.size());
    uint8_t* dflat = nullptr;
    bool shuffle_ok = true;
    if (from_file) {
        b200_weight_desc wd;
        DRV_B200(b200_weight_file_stat(o.load_weights.c_str(), &wd));
        if (wd.n != o.n || wd.k != o.k || wd.b_layout != B200_B_FLAT_16x16 ||
            wd.scale_mode != (block ? B200_SCALE_BLOCK : B200_SCALE_NONE)) {
            std::fprintf(stderr, "%s holds N=%lld K=%lld layout %d scales %d: not what this run asks for.\n", o.load_weights.c_str(),
                         (long long)wd.n, (long long)wd.k, wd.b_layout, wd.scale_mode);
            return 1;
        }
        DRV_B200(b200_weight_file_read(o.load_weights.c_str(), hflat.data(), hflat.size(), block ? hsfb.data() : nullptr,
                                       block ? hsfb.size() * sizeof(float) : 0));
        std::printf("Loaded pre-shuffled B from %s (checksum ok); no shuffle pass.\n", o.load_weights.c_str());
        dflat = dev_upload(hflat.data(), hflat.size());
        if (o.verify) unshuffle_b_host(hflat.data(), hb.data(), o.n, o.k);   // the host check reads the [K,N] matrix
    } else {
        fill_e4m3(hb.data(), hb.size(), o.seed, 1, o.dist, -0.5f, 0.5f);   // [K,N] per batch (:732)
        uint8_t* dkn = dev_upload(hb.data(), hb.size());
        DRV_CUDA(cudaMalloc(&dflat, hb.size()));
        std::printf("Shuffling B matrix for FlatMM layout (batch=%d)...\n", o.batch);
        for (size_t b = 0; b < B; ++b) DRV_B200(b200_shuffle_b(dkn + b * N * K, dflat + b * N * K, o.n, o.k, 1, nullptr));
        DRV_CUDA(cudaMemcpy(hflat.data(), dflat, hflat.size(), cudaMemcpyDeviceToHost));
        cudaFree(dkn);
        if (o.verify) {
            std::vector<uint8_t> want(N * K);
            for (size_t b = 0; b < B; ++b) {
                shuffle_b_host(hb.data() + b * N * K, want.data(), o.n, o.k);
                shuffle_ok = shuffle_ok && std::memcmp(want.data(), hflat.data() + b * N * K, N * K) == 0;
            }
            std::printf("[shuffle_b] device vs host: %s\n", shuffle_ok ? "BIT-EXACT" : "MISMATCH");
        }
        if (!o.save_weights.empty()) {
            DRV_B200(b200_weight_file_write(o.save_weights.c_str(), B200_B_FLAT_16x16, block ? B200_SCALE_BLOCK : B200_SCALE_NONE, o.n,
                                            o.k, hflat.data(), block ? hsfb.data() : nullptr));
            std::printf("Wrote %s\n", o.save_weights.c_str());
        }
    }
    float *dsfa = nullptr, *dsfb = nullptr;
    if (block) {
        dsfa = dev_upload(hsfa.data(), hsfa.size());
        dsfb = dev_upload(hsfb.data(), hsfb.size());
    }
    void* dc = nullptr;
    DRV_CUDA(cudaMalloc(&dc, B * M * N * (bf16 ? 2 : 4)));

    b200_gemm_args args{};
    args.ptr_a = da; args.ptr_b = dflat; args.ptr_c = dc;
    args.m = o.m; args.n = o.n; args.k = o.k; args.batch = o.batch;
    args.stride_a = o.k; args.stride_b = o.n; args.stride_c = o.n;          // stride_b = N as at :765
    args.stride_a_batch = (int64_t)M * K; args.stride_b_batch = (int64_t)N * K; args.stride_c_batch = (int64_t)M * N;
    if (block) {
        args.ptr_sfa = dsfa; args.ptr_sfb = dsfb;
        args.stride_sfa = o.m; args.stride_sfb = (int64_t)KG;
        args.stride_sfa_batch = (int64_t)(M * KG); args.stride_sfb_batch = (int64_t)(NG * KG);
        args.scale_mode = B200_SCALE_BLOCK;
    }
    args.b_layout = B200_B_FLAT_16x16;
    args.out_dtype = bf16 ? B200_OUT_BF16 : B200_OUT_F32;
    args.tile_hint = o.tile;

    int32_t tile = 0;
    DRV_B200(b200_gemm_check(&args, &tile));
    std::printf("Launching FlatMM kernel: M=%d, N=%d, K=%d, batch=%d, tile_config=%d, sms=%d\n", o.m, o.n, o.k, o.batch, tile,
                b200_sm_count());
    DRV_B200(b200_gemm_a8w8(&args, nullptr));
    DRV_CUDA(cudaDeviceSynchronize());
    if (int st = b200_last_status()) {
        std::fprintf(stderr, "device wait expired, status %d\n", st);
        return 1;
    }

    bool all_valid = shuffle_ok;
    if (o.verify) {
        std::vector<float> hc, ref(M * N);
        fetch_c(hc, dc, B * M * N, bf16);
        for (size_t b = 0; b < B; ++b) {
            gemm_ref_kn(ha.data() + b * M * K, hb.data() + b * N * K, block ? hsfa.data() + b * KG * M : nullptr,
                        block ? hsfb.data() + b * NG * KG : nullptr, ref.data(), o.m, o.n, o.k);
            double me, mr;
            const bool rel = valid_relative(ref.data(), hc.data() + b * M * N, (long long)(M * N), &me, &mr);
            const bool valid = (block || bf16) ? rel : valid_vector(ref.data(), hc.data() + b * M * N, (long long)(M * N), 1e-1f);
            std::printf("[FlatMM batch %zu/%zu: %dx%dx%d] %s (max_err=%.3g, max_ref=%.3g)\n", b + 1, B, o.m, o.n, o.k,
                        valid ? "VALID" : "FAIL", me, mr);
            all_valid = all_valid && valid;
        }
        std::printf("\n[Overall] %s\n", all_valid ? "ALL BATCHES VALID" : "SOME BATCHES FAILED");
    }
    std::printf("\n");
    const double ms = benchmark(args, o.warmup, o.iters, o.overlap);
    std::printf("\n");
    if (o.json) {
        const double bytes = (double)B * (N * K + M * K + (block ? 4.0 * (NG * KG + M * KG) : 0.0) + (bf16 ? 2.0 : 4.0) * M * N);
        std::printf("{\"driver\": \"flatmm_a8w8\", \"m\": %d, \"n\": %d, \"k\": %d, \"batch\": %d, \"ms\": %.5f, \"tflops\": %.2f, \"gbps\": %.1f, \"valid\": %s}\n",
                    o.m, o.n, o.k, o.batch, ms, 2.0 * M * N * K * B / 1e9 / ms, bytes / ms / 1e6, all_valid ? "true" : "false");
    }
    cudaFree(da); cudaFree(dflat); cudaFree(dc);
    if (dsfa) cudaFree(dsfa);
    if (dsfb) cudaFree(dsfb);
    return 0;
}
