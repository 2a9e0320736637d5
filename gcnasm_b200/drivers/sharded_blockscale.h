// gemm_a8w8_blockscale --gpus R: the block-scale GEMM with B sharded along N over R GPUs of one machine, driven from
// ONE host process through the C ABI only.  The reference program is single-GPU; this is the large-N configuration
// (each GPU keeps N/R weight columns, the activation starts on GPU 0 and is delivered to every GPU once per call).
//
// Per call: GPU 0 uploads the activation from pinned host memory slab by slab (b200_slab_upload), every GPU pushes each
// slab it holds into the next GPU's buffer with a device-to-device copy and then copies the call's number into that
// GPU's ready word (b200_stream_copy; the next GPU's delivery stream waits on the word with b200_flag_wait), and ONE
// GEMM launch per GPU consumes the slabs as batches of a batched problem with one B (B200_GEMM_BATCH_READY).  A GPU
// overwrites its neighbour's buffer two calls later only after the neighbour's credit (its GEMM and its own forwarding
// of that buffer are done).  Nothing here launches a kernel except the GEMMs, the quantisers of the set-up and the checker.
#pragma once

#include "driver_common.h"

namespace drv {

struct ShardDev {
    int dev = 0;
    uint8_t* region = nullptr;           // [2 buffers x slabs x slab bytes | ready words | credit | scratch]
    uint8_t* b = nullptr;                // weight shard [N/R][K]
    float* sfb = nullptr;                // its 128x128 scales
    void* c = nullptr;                   // output shard [M][N/R]
    cudaStream_t compute = nullptr, delivery = nullptr, credit = nullptr;
    cudaEvent_t gemm_done[2] = {nullptr, nullptr}, fwd_done[2] = {nullptr, nullptr};
};

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

inline int run_sharded(const Options& o, int gpus) {
    int have = 0;
    DRV_CUDA(cudaGetDeviceCount(&have));
    if (gpus < 2 || gpus > have) {
        std::fprintf(stderr, "--gpus %d: this machine has %d CUDA device(s)\n", gpus, have);
        return 1;
    }
    const int64_t M = o.m, N = o.n, K = o.k;
    int64_t rows = 0;                                  // rows per slab: largest multiple of 256 <= 2048 that divides M
    for (int64_t r = 256; r <= 2048 && r <= M; r += 256)
        if (M % r == 0) rows = r;
    if (o.batch != 1 || K % 128 != 0 || N % (128 * gpus) != 0 || rows == 0) {
        std::fprintf(stderr, "--gpus: batch 1, K %% 128 == 0, N %% (128 * gpus) == 0 and M a multiple of 256 are required\n");
        return 1;
    }
    const int64_t NS = N / gpus, KG = K / 128, slabs = M / rows;
    const size_t slab = b200_slab_bytes(rows, K);
    const size_t act = 2 * slabs * slab, ready_off = align256(act), credit_off = align256(ready_off + 4 * 2 * slabs);
    const size_t scratch_off = credit_off + 256, region_bytes = scratch_off + 256;
    const bool bf16 = o.out == "bf16";
    const size_t esz = bf16 ? 2 : 4;

    // ---- activation: seeded source, quantised on GPU 0, kept in pinned host memory in the reference's layouts ----
    uint8_t* ha = nullptr;
    float* hsfa = nullptr;
    DRV_CUDA(cudaMallocHost(&ha, M * K));
    DRV_CUDA(cudaMallocHost(&hsfa, KG * M * 4));
    {
        DRV_CUDA(cudaSetDevice(0));
        std::vector<float> xa(M * K);
        if (o.dist == "u11") b200_fill_uniform(xa.data(), xa.size(), o.seed, 0, -1.0f, 1.0f);
        else b200_fill_normal(xa.data(), xa.size(), o.seed, 0);
        float* dxa = dev_upload(xa.data(), xa.size());
        uint8_t* dq = nullptr;
        float* dsf = nullptr;
        DRV_CUDA(cudaMalloc(&dq, M * K));
        DRV_CUDA(cudaMalloc(&dsf, KG * M * 4));
        DRV_B200(b200_quantize_1x128(dxa, dq, dsf, M, K, nullptr));
        DRV_CUDA(cudaMemcpy(ha, dq, M * K, cudaMemcpyDeviceToHost));
        DRV_CUDA(cudaMemcpy(hsfa, dsf, KG * M * 4, cudaMemcpyDeviceToHost));
        cudaFree(dxa); cudaFree(dq); cudaFree(dsf);
    }
    // ---- per GPU: weight shard (its own seeded stream), buffers, streams; neighbours may write into each other ----
    std::vector<ShardDev> g(gpus);
    for (int d = 0; d < gpus; ++d) {
        ShardDev& s = g[d];
        s.dev = d;
        DRV_CUDA(cudaSetDevice(d));
        for (int p : {d - 1, d + 1})
            if (p >= 0 && p < gpus) {
                const cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) DRV_CUDA(e);
                cudaGetLastError();
            }
        DRV_CUDA(cudaMalloc(&s.region, region_bytes));
        DRV_CUDA(cudaMemset(s.region, 0, region_bytes));
        std::vector<float> xb(NS * K);
        if (o.dist == "u11") b200_fill_uniform(xb.data(), xb.size(), o.seed, 16 + d, -1.0f, 1.0f);
        else b200_fill_normal(xb.data(), xb.size(), o.seed, 16 + d);
        float* dxb = dev_upload(xb.data(), xb.size());
        DRV_CUDA(cudaMalloc(&s.b, NS * K));
        DRV_CUDA(cudaMalloc(&s.sfb, (NS / 128) * KG * 4));
        DRV_B200(b200_quantize_128x128(dxb, s.b, s.sfb, NS, K, nullptr));
        DRV_CUDA(cudaDeviceSynchronize());
        cudaFree(dxb);
        DRV_CUDA(cudaMalloc(&s.c, M * NS * esz));
        DRV_CUDA(cudaStreamCreateWithFlags(&s.compute, cudaStreamNonBlocking));
        DRV_CUDA(cudaStreamCreateWithFlags(&s.delivery, cudaStreamNonBlocking));
        DRV_CUDA(cudaStreamCreateWithFlags(&s.credit, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            DRV_CUDA(cudaEventCreateWithFlags(&s.gemm_done[i], cudaEventDisableTiming));
            DRV_CUDA(cudaEventCreateWithFlags(&s.fwd_done[i], cudaEventDisableTiming));
        }
    }
    auto ready = [&](int d, int buf, int64_t s) { return reinterpret_cast<int32_t*>(g[d].region + ready_off) + buf * slabs + s; };
    auto slab_at = [&](int d, int buf, int64_t s) { return g[d].region + (buf * slabs + s) * slab; };

    // ---- one call: delivery down the chain 0 -> 1 -> ... and one GEMM launch per GPU ------------------------------
    auto call = [&](int step) {
        const int buf = step % 2, epoch = step + 1;
        for (int d = 0; d < gpus; ++d) {
            ShardDev& s = g[d];
            DRV_CUDA(cudaSetDevice(d));
            int32_t* tmp = reinterpret_cast<int32_t*>(s.region + scratch_off);
            if (d == 0) {
                // the root's buffer was last read by its own GEMM two calls ago
                if (step >= 2) DRV_CUDA(cudaStreamWaitEvent(s.delivery, s.gemm_done[buf], 0));
                for (int64_t i = 0; i < slabs; ++i) {
                    DRV_B200(b200_slab_upload(ha, hsfa, s.region + buf * slabs * slab, M, K, rows, i, s.delivery));
                    DRV_B200(b200_flag_write(ready(0, buf, i), epoch, s.delivery));
                }
            }
            if (d + 1 < gpus) {
                if (step >= 2) DRV_B200(b200_flag_wait(reinterpret_cast<int32_t*>(s.region + credit_off), step - 1, s.delivery));
                DRV_B200(b200_flag_write(tmp, epoch, s.delivery));
                for (int64_t i = 0; i < slabs; ++i) {
                    if (d > 0) DRV_B200(b200_flag_wait(ready(d, buf, i), epoch, s.delivery));
                    DRV_B200(b200_stream_copy(slab_at(d + 1, buf, i), slab_at(d, buf, i), slab, s.delivery));
                    DRV_B200(b200_stream_copy(ready(d + 1, buf, i), tmp, 4, s.delivery));
                }
            }
            DRV_CUDA(cudaEventRecord(s.fwd_done[buf], s.delivery));
            b200_gemm_args a{};
            a.ptr_a = s.region + buf * slabs * slab;
            a.ptr_b = s.b;
            a.ptr_c = s.c;
            a.m = rows; a.n = NS; a.k = K; a.batch = slabs;
            a.stride_a = K; a.stride_b = K; a.stride_c = NS;
            a.stride_a_batch = (int64_t)slab; a.stride_b_batch = 0; a.stride_c_batch = rows * NS;
            a.ptr_sfa = s.region + buf * slabs * slab + rows * K;
            a.ptr_sfb = s.sfb;
            a.stride_sfa = rows; a.stride_sfb = KG;
            a.stride_sfa_batch = (int64_t)(slab / 4); a.stride_sfb_batch = 0;
            a.scale_mode = B200_SCALE_BLOCK; a.b_layout = B200_B_NK_ROWMAJOR;
            a.out_dtype = bf16 ? B200_OUT_BF16 : B200_OUT_F32;
            a.flags = B200_GEMM_BATCH_READY;
            a.ptr_batch_ready = ready(d, buf, 0);
            a.batch_epoch = epoch;
            DRV_B200(b200_gemm_a8w8(&a, s.compute));
            DRV_CUDA(cudaEventRecord(s.gemm_done[buf], s.compute));
            if (d > 0) {
                // credit to the previous GPU: this buffer may be overwritten
                int32_t* tmpc = tmp + 16;
                DRV_CUDA(cudaStreamWaitEvent(s.credit, s.gemm_done[buf], 0));
                DRV_CUDA(cudaStreamWaitEvent(s.credit, s.fwd_done[buf], 0));
                DRV_B200(b200_flag_write(tmpc, epoch, s.credit));
                DRV_B200(b200_stream_copy(g[d - 1].region + credit_off, tmpc, 4, s.credit));
            }
        }
    };
    auto sync_all = [&]() {
        for (int d = 0; d < gpus; ++d) {
            DRV_CUDA(cudaSetDevice(d));
            DRV_CUDA(cudaDeviceSynchronize());
        }
    };

    std::printf("Launching sharded GEMM: M=%lld, N=%lld (%lld per GPU), K=%lld, gpus=%d, slabs=%lld x %lld rows\n", (long long)M,
                (long long)N, (long long)NS, (long long)K, gpus, (long long)slabs, (long long)rows);
    int step = 0;
    call(step++);
    sync_all();
    bool all_valid = true;
    for (int d = 0; d < gpus; ++d) {
        DRV_CUDA(cudaSetDevice(d));
        if (int st = b200_last_status()) {
            std::fprintf(stderr, "GPU %d: device wait expired, status %d\n", d, st);
            return 1;
        }
    }
    if (o.verify) {
        // 128 rows of every shard against the one-thread-per-output checker kernel (the device mirror of gemm_ref,
        // gemm_a8w8_blockscale_host.cc:66-90), run on the slabs as they were DELIVERED to that GPU
        std::printf("\nValidating every GPU's shard against the checker kernel (128 rows of the last slab)...\n");
        for (int d = 0; d < gpus; ++d) {
            DRV_CUDA(cudaSetDevice(d));
            const int64_t sl = slabs - 1, r0 = rows - 128;
            float* dref = nullptr;
            DRV_CUDA(cudaMalloc(&dref, 128 * NS * 4));
            b200_gemm_args a{};
            a.ptr_a = slab_at(d, 0, sl) + r0 * K;
            a.ptr_b = g[d].b;
            a.ptr_c = dref;
            a.m = 128; a.n = NS; a.k = K; a.batch = 1;
            a.stride_a = K; a.stride_b = K; a.stride_c = NS;
            a.ptr_sfa = reinterpret_cast<float*>(slab_at(d, 0, sl) + rows * K) + r0;
            a.ptr_sfb = g[d].sfb;
            a.stride_sfa = rows; a.stride_sfb = KG;
            a.scale_mode = B200_SCALE_BLOCK; a.out_dtype = B200_OUT_F32;
            DRV_B200(b200_gemm_a8w8_simple(&a, nullptr));
            DRV_CUDA(cudaDeviceSynchronize());
            std::vector<float> ref(128 * NS), got;
            DRV_CUDA(cudaMemcpy(ref.data(), dref, ref.size() * 4, cudaMemcpyDeviceToHost));
            fetch_c(got, static_cast<uint8_t*>(g[d].c) + (sl * rows + r0) * NS * esz, 128 * NS, bf16);
            double me, mr;
            const bool valid = valid_relative(ref.data(), got.data(), (long long)ref.size(), &me, &mr);
            std::printf("[GPU %d: columns %lld..%lld] %s (max_err=%.3g, max_ref=%.3g)\n", d, (long long)(d * NS), (long long)((d + 1) * NS),
                        valid ? "VALID" : "FAIL", me, mr);
            all_valid = all_valid && valid;
            cudaFree(dref);
        }
        std::printf("\n[Overall] %s\n", all_valid ? "ALL SHARDS VALID" : "SOME SHARDS FAILED");
    }
    for (int i = 0; i < o.warmup; ++i) call(step++);
    sync_all();
    DRV_CUDA(cudaSetDevice(0));
    cudaEvent_t e0, e1;
    DRV_CUDA(cudaEventCreate(&e0));
    DRV_CUDA(cudaEventCreate(&e1));
    DRV_CUDA(cudaEventRecord(e0, g[0].compute));
    for (int i = 0; i < o.iters; ++i) call(step++);
    // the timed region ends when the LAST GPU's last GEMM is done: GPU 0's compute stream waits for all of them
    for (int d = 1; d < gpus; ++d) DRV_CUDA(cudaStreamWaitEvent(g[0].compute, g[d].gemm_done[(step - 1) % 2], 0));
    DRV_CUDA(cudaEventRecord(e1, g[0].compute));
    sync_all();
    float total = 0.0f;
    DRV_CUDA(cudaEventElapsedTime(&total, e0, e1));
    const double avg = total / o.iters;
    std::printf("\nKernel Performance: avg_time=%.4f ms, %.2f TFlops (%d GPUs, activation uploaded and delivered every call)\n\n", avg,
                2.0 * M * N * K / 1.0e9 / avg, gpus);
    int status = 0;
    for (int d = 0; d < gpus; ++d) {
        DRV_CUDA(cudaSetDevice(d));
        status |= b200_last_status();
    }
    if (o.json)
        std::printf("{\"driver\": \"gemm_a8w8_blockscale\", \"gpus\": %d, \"m\": %lld, \"n\": %lld, \"k\": %lld, \"ms\": %.5f, \"tflops\": %.2f, \"valid\": %s, \"status\": %d}\n",
                    gpus, (long long)M, (long long)N, (long long)K, avg, 2.0 * M * N * K / 1e9 / avg, all_valid ? "true" : "false", status);
    return (all_valid && status == 0) ? 0 : 1;
}

}  // namespace drv
