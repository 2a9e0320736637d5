// HBM bandwidth probe with the command line and output lines of the reference's bandwidth_memread tool
// (bandwidth_memread/bandwidth_kernel.cu: main :294-366, result line :284): without arguments a sweep of eleven
// buffer sizes, read-only first and read+write second; with one argument a single size given in dwords.
// BANDWIDTH_TEST_LIST=2 selects the second size list, BANDWIDTH_TEST_CASE=N scales the first list by N units
// instead of the SM count (the reference's "CU count" override).  The device work goes through the C ABI of
// libb200gemm.so (b200_membw_read / b200_membw_copy); timing is CUDA events around `loops` launches after a warm-up.
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "b200gemm.h"

#define CK(call)                                                                                   \
    do {                                                                                           \
        cudaError_t st_ = (call);                                                                  \
        if (st_ != cudaSuccess) {                                                                  \
            std::fprintf(stderr, "CUDA error (%s:%d): %s\n", __FILE__, __LINE__, cudaGetErrorString(st_)); \
            std::exit(1);                                                                          \
        }                                                                                          \
    } while (0)

static int env_int(const char* name, int dflt) {
    const char* v = std::getenv(name);
    return v ? std::atoi(v) : dflt;
}

static void human(size_t bytes, char* out, size_t cap) {
    if (bytes < 1024) std::snprintf(out, cap, "%zuB", bytes);
    else if (bytes < (1u << 20)) std::snprintf(out, cap, "%.2fKB", bytes / 1024.0);
    else if (bytes < (1u << 30)) std::snprintf(out, cap, "%.2fMB", bytes / 1048576.0);
    else std::snprintf(out, cap, "%.2fGB", bytes / 1073741824.0);
}

// mode 0: read only, mode 1: read + write.  Returns GB/s (bytes moved: 1x the buffer for ro, 2x for rw).
static double run(int mode, int64_t dwords, bool verify) {
    const size_t bytes = (static_cast<size_t>(dwords) * 4 + 15) / 16 * 16;
    void *a = nullptr, *b = nullptr;
    uint32_t* sum = nullptr;
    CK(cudaMalloc(&a, bytes));
    CK(cudaMalloc(&b, bytes));
    CK(cudaMalloc(&sum, 4));
    // buffers above 1 GiB are filled on the device and not verified (the check would need two host copies)
    verify = verify && bytes <= (1ull << 30);
    std::vector<uint32_t> h;
    uint32_t want = 0;
    if (verify) {
        h.resize(bytes / 4);
        for (size_t i = 0; i < h.size(); ++i) {
            h[i] = static_cast<uint32_t>(i * 2654435761u + 12345u);
            want += h[i];
        }
        CK(cudaMemcpy(a, h.data(), bytes, cudaMemcpyHostToDevice));
    } else {
        CK(cudaMemset(a, 0x5A, bytes));
    }
    CK(cudaMemset(b, 0, bytes));
    CK(cudaMemset(sum, 0, 4));
    auto launch = [&]() {
        const int rc = mode == 0 ? b200_membw_read(a, bytes, sum, nullptr) : b200_membw_copy(a, b, bytes, nullptr);
        if (rc != 0) {
            std::fprintf(stderr, "b200 error: %s\n", b200_strerror(rc));
            std::exit(1);
        }
    };
    launch();
    CK(cudaDeviceSynchronize());
    if (verify) {
        bool ok = true;
        if (mode == 0) {
            uint32_t got = 0;
            CK(cudaMemcpy(&got, sum, 4, cudaMemcpyDeviceToHost));
            ok = got == want;
        } else {
            std::vector<uint32_t> back(bytes / 4);
            CK(cudaMemcpy(back.data(), b, bytes, cudaMemcpyDeviceToHost));
            ok = back == h;
        }
        if (!ok) {
            std::fprintf(stderr, "verification failed (%s, %lld dwords)\n", mode == 0 ? "ro" : "rw", static_cast<long long>(dwords));
            std::exit(2);
        }
    }
    const int warm = 5;
    // enough launches for >= ~2 ms of timed work on small buffers, 20 on large ones
    int loops = static_cast<int>((64ull << 20) * 200 / (bytes + 1));
    loops = loops < 20 ? 20 : (loops > 2000 ? 2000 : loops);
    for (int i = 0; i < warm; ++i) launch();
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    CK(cudaEventRecord(e0));
    for (int i = 0; i < loops; ++i) launch();
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    ms /= loops;
    const double gbs = static_cast<double>(bytes) * (mode == 0 ? 1 : 2) / 1e6 / ms;
    char str[32];
    human(bytes, str, sizeof(str));
    std::printf("%9s(%s) -> %.4fms, %.3f(GB/s)\n", str, mode == 0 ? "[ro]" : "[rw]", ms, gbs);
    std::fflush(stdout);
    CK(cudaEventDestroy(e0));
    CK(cudaEventDestroy(e1));
    CK(cudaFree(a));
    CK(cudaFree(b));
    CK(cudaFree(sum));
    return gbs;
}

int main(int argc, char** argv) {
    CK(cudaSetDevice(0));
    const bool verify = env_int("BANDWIDTH_VERIFY", 1) != 0;
    if (argc > 1) {
        const int64_t dwords = std::atoll(argv[1]);
        if (dwords <= 0) {
            std::fprintf(stderr, "usage: %s [dwords]\n", argv[0]);
            return 1;
        }
        run(0, dwords, verify);
        run(1, dwords, verify);
        return 0;
    }
    const int btc = env_int("BANDWIDTH_TEST_CASE", 0);
    const int list = env_int("BANDWIDTH_TEST_LIST", 0);
    int units = b200_sm_count();
    std::printf("sm:%d, streaming_load:1, streaming_store:1 (%d) timer:gpu\n", units, btc);
    if (btc != 0) units = btc == -1 ? 304 : btc;
    const int64_t blk = 1024;
    std::vector<int64_t> sizes = {20000, 400000, 16711680};
    if (list == 2)
        for (int64_t f : {3, 6, 14, 25, 38, 54, 95, 158}) sizes.push_back(10032 * f * blk);
    else
        for (int64_t f : {116, 212, 476, 820, 1024, 1638, 3276, 5710}) sizes.push_back(f * units * blk);
    std::printf("---------------------------------------------\n");
    for (int64_t d : sizes) {
        run(0, d, verify);
        usleep(200000);
    }
    std::printf("---------------------------------------------\n");
    usleep(2000000);
    for (int64_t d : sizes) {
        run(1, d, verify);
        usleep(200000);
    }
    return 0;
}
