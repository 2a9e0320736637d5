// Shared host code of the three command-line drivers.  Each driver keeps the reference program's
// operator surface -- -m/-n/-k/-b (and -v) arguments, NT layout, the printed lines, a host reference
// check, a warm-up + timed benchmark loop -- and reaches the GPU only through the C ABI of
// libb200gemm.so.  The reference mains are opus_gemm/gemm_a8w8_8wave.cc:652-780,
// opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_host.cc:128-294 and
// opus_fmm/flatmm_a8w8_gfx950.cc:683-821.
#pragma once

#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <omp.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "b200gemm.h"

namespace drv {

#define DRV_CUDA(call)                                                                            \
    do {                                                                                          \
        cudaError_t st_ = (call);                                                                 \
        if (st_ != cudaSuccess) {                                                                 \
            std::fprintf(stderr, "CUDA error (%s:%d): %s\n", __FILE__, __LINE__, cudaGetErrorString(st_)); \
            std::exit(1);                                                                         \
        }                                                                                         \
    } while (0)

#define DRV_B200(call)                                                                            \
    do {                                                                                          \
        int rc_ = (call);                                                                         \
        if (rc_ != 0) {                                                                           \
            std::fprintf(stderr, "b200gemm error (%s:%d): %s [%d, cuda %d]\n", __FILE__, __LINE__, \
                         b200_strerror(rc_), rc_, b200_last_cuda_error());                        \
            std::exit(1);                                                                         \
        }                                                                                         \
    } while (0)

struct Options {
    int m = 256, n = 512, k = 256, batch = 8;      // the reference defaults (gemm_a8w8_8wave.cc:666-669)
    int verify = 1;
    int warmup = 200, iters = 100;                 // gemm_a8w8_8wave.cc:616
    uint64_t seed = 1234;
    std::string scale = "";                        // none | tensor | block | mx (driver default if empty)
    std::string out = "f32";                       // f32 | bf16   (the reference writes fp32)
    bool overlap = false;                          // benchmark loop: launches flagged B200_GEMM_INPUTS_READY
    bool act_bf16 = false;                         // blockscale: activations arrive in bf16, fused quantiser
    std::string save_weights = "", load_weights = "";  // flatmm: weight file written after / read instead of the shuffle
    std::string dist = "ref";                      // ref: A~U[0,1) B~U[-.5,.5) as the reference; u11: U[-1,1]; n01: N(0,1)
    int tile = 0;
    int gpus = 1;                                  // blockscale: B sharded along N over this many GPUs of the machine
    bool json = false;
};

// Accepts "-m 4096" and "-m=4096" like gemm_a8w8_blockscale_host.cc:140-173.
inline bool take(int argc, char** argv, int& i, const char* s, const char* l, std::string& val) {
    const char* a = argv[i];
    for (const char* f : {s, l}) {
        if (!f) continue;
        const size_t len = std::strlen(f);
        if (std::strncmp(a, f, len) != 0) continue;
        if (a[len] == '=') {
            val = a + len + 1;
            return true;
        }
        if (a[len] == '\0' && i + 1 < argc) {
            val = argv[++i];
            return true;
        }
    }
    return false;
}

inline Options parse(int argc, char** argv, int default_verify) {
    Options o;
    o.verify = default_verify;
    for (int i = 1; i < argc; ++i) {
        std::string v;
        if (take(argc, argv, i, "-m", "--m", v)) o.m = std::atoi(v.c_str());
        else if (take(argc, argv, i, "-n", "--n", v)) o.n = std::atoi(v.c_str());
        else if (take(argc, argv, i, "-k", "--k", v)) o.k = std::atoi(v.c_str());
        else if (take(argc, argv, i, "-b", "--b", v)) o.batch = std::atoi(v.c_str());
        else if (take(argc, argv, i, "-v", "--verify", v)) o.verify = std::atoi(v.c_str());
        else if (take(argc, argv, i, nullptr, "--seed", v)) o.seed = std::strtoull(v.c_str(), nullptr, 10);
        else if (take(argc, argv, i, nullptr, "--scale", v)) o.scale = v;
        else if (take(argc, argv, i, nullptr, "--out", v)) o.out = v;
        else if (take(argc, argv, i, nullptr, "--dist", v)) o.dist = v;
        else if (take(argc, argv, i, nullptr, "--tile", v)) o.tile = std::atoi(v.c_str());
        else if (take(argc, argv, i, nullptr, "--gpus", v)) o.gpus = std::atoi(v.c_str());
        else if (take(argc, argv, i, nullptr, "--warmup", v)) o.warmup = std::atoi(v.c_str());
        else if (take(argc, argv, i, nullptr, "--iters", v)) o.iters = std::atoi(v.c_str());
        else if (take(argc, argv, i, nullptr, "--save-weights", v)) o.save_weights = v;
        else if (take(argc, argv, i, nullptr, "--load-weights", v)) o.load_weights = v;
        else if (std::strcmp(argv[i], "--json") == 0) o.json = true;
        else if (std::strcmp(argv[i], "--act-bf16") == 0) o.act_bf16 = true;
        else if (std::strcmp(argv[i], "--overlap") == 0) o.overlap = true;
    }
    return o;
}

// ---- host E4M3 / bf16 helpers (NVIDIA's cuda_fp8.h host paths) --------------------------------------
inline uint8_t to_e4m3(float x) { return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)); }
inline const float* e4m3_table() {
    static float lut[256];
    static bool ready = false;
    if (!ready) {
        for (int i = 0; i < 256; ++i) {
            const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(i), __NV_E4M3);
            lut[i] = __half2float(__half(h));
        }
        ready = true;
    }
    return lut;
}
inline float bf16_bits_to_f32(uint16_t b) {
    const uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// Seeded replacement of rand_vector / rand_vector_2d (gemm_a8w8_8wave.cc:566-580): draws float
// values and casts them to E4M3 exactly as static_cast<fp8>(float) does.
inline void fill_e4m3(uint8_t* dst, size_t count, uint64_t seed, uint32_t tensor_id, const std::string& dist, float lo,
                      float hi) {
    std::vector<float> tmp(count);
    if (dist == "n01") b200_fill_normal(tmp.data(), count, seed, tensor_id);
    else if (dist == "u11") b200_fill_uniform(tmp.data(), count, seed, tensor_id, -1.0f, 1.0f);
    else b200_fill_uniform(tmp.data(), count, seed, tensor_id, lo, hi);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < static_cast<long long>(count); ++i) dst[i] = to_e4m3(tmp[i]);
}

// valid_vector (gemm_a8w8_8wave.cc:583-598): absolute threshold, first 10 offenders printed.
inline bool valid_vector(const float* ref, const float* res, long long count, float threshold) {
    int errors = 0;
    for (long long i = 0; i < count; ++i) {
        const float diff = std::fabs(ref[i] - res[i]);
        if (diff > threshold || diff != diff) {
            if (errors < 10) std::printf("Error at %lld: ref=%.6f, result=%.6f, diff=%.6f\n", i, ref[i], res[i], diff);
            if (++errors >= 10) break;
        }
    }
    return errors == 0;
}
// the relative criterion of the benchmark configurations: max|err| <= 1e-2 * max|ref|
inline bool valid_relative(const float* ref, const float* res, long long count, double* max_err, double* max_ref) {
    double me = 0, mr = 0;
    bool nan = false;
#pragma omp parallel for reduction(max : me, mr) reduction(|| : nan)
    for (long long i = 0; i < count; ++i) {
        const double d = std::fabs(static_cast<double>(ref[i]) - res[i]);
        if (d != d) nan = true;
        if (d > me) me = d;
        if (std::fabs(ref[i]) > mr) mr = std::fabs(ref[i]);
    }
    *max_err = me;
    *max_ref = mr;
    return !nan && me <= 1e-2 * mr;
}

// benchmark_kernel (gemm_a8w8_8wave.cc:615-650): warm-up, then `iters` back-to-back launches between two
// events on the default stream; TFlops = 2*M*N*K*batch / time.
// `overlap`: the operands are the same static buffers in every iteration, so the launches may be flagged
// B200_GEMM_INPUTS_READY (a launch starts while the previous one drains; writes to C stay ordered)
inline double benchmark(const b200_gemm_args& args_in, int warmup, int iters, bool overlap = false) {
    b200_gemm_args args = args_in;
    if (overlap) args.flags |= B200_GEMM_INPUTS_READY;
    for (int i = 0; i < warmup; ++i) DRV_B200(b200_gemm_a8w8(&args, nullptr));
    cudaEvent_t e0, e1;
    DRV_CUDA(cudaEventCreate(&e0));
    DRV_CUDA(cudaEventCreate(&e1));
    DRV_CUDA(cudaDeviceSynchronize());
    DRV_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < iters; ++i) DRV_B200(b200_gemm_a8w8(&args, nullptr));
    DRV_CUDA(cudaEventRecord(e1));
    DRV_CUDA(cudaEventSynchronize(e1));
    float total = 0.0f;
    DRV_CUDA(cudaEventElapsedTime(&total, e0, e1));
    DRV_CUDA(cudaEventDestroy(e0));
    DRV_CUDA(cudaEventDestroy(e1));
    const double avg = total / iters;
    const double flop = 2.0 * args.m * args.n * args.k * args.batch;
    std::printf("Kernel Performance: avg_time=%.4f ms, %.2f TFlops\n", avg, flop / 1.0e9 / avg);
    return avg;
}

template <class T>
T* dev_upload(const T* host, size_t count) {
    T* d = nullptr;
    DRV_CUDA(cudaMalloc(&d, count * sizeof(T)));
    DRV_CUDA(cudaMemcpy(d, host, count * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}

// device C (fp32 or bf16) -> host fp32
inline void fetch_c(std::vector<float>& host, const void* dev, size_t count, bool bf16) {
    host.resize(count);
    if (!bf16) {
        DRV_CUDA(cudaMemcpy(host.data(), dev, count * 4, cudaMemcpyDeviceToHost));
        return;
    }
    std::vector<uint16_t> tmp(count);
    DRV_CUDA(cudaMemcpy(tmp.data(), dev, count * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < count; ++i) host[i] = bf16_bits_to_f32(tmp[i]);
}

}  // namespace drv
