#!/usr/bin/env python
"""Benchmark of the A8W8 FP8 block-scale GEMM hot path (one JSON line on stdout).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c5|decode]

A step is one pass of the hot path over one batch of synthetic input: one block-scale FP8 GEMM
C[M,N] = A[M,K] . B[N,K]^T with fp32 scales per 1x128 (A) and 128x128 (B), bf16 output.
At one GPU the workload is the DeepSeek-style shape M=4096, N=7168, K=2048 (seeded N(0,1) data quantised
on the device with group amax/448).  With N GPUs the same shape is column-sharded the way the large-N
configuration prescribes: every rank keeps a 7168-column weight shard (global N = 7168*N_gpus, weak scaling),
rank 0 owns the activation and broadcasts A + SFA over NCCL every step, outputs stay N-sharded.

`value` is device-timed throughput with operands resident in HBM; `e2e` is the same metric through the
host-buffer entry point b200_gemm_a8w8_host (pinned host operands copied in, result copied out, every
step).  `--impl reference` times the CPU restatement of the reference's host GEMM loop (the reference
itself is HIP-only and cannot be built here) on all host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, N per rank, K)
    "c2": (4096, 7168, 2048),
    "c5": (16384, 7168, 8192),
    "cube8192": (8192, 8192, 8192),
}
SEED = 1234
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture
# summarised in profiles/ (None where no capture of that workload exists)
NCU_TRAFFIC_BYTES = {"c2": 32070912}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power) if power else None}


def cpu_reference_arm(args, workload, rank, world):
    """The reference's CPU implementation of the path: its host gemm_ref loop (block-scale variant,
    opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_host.cc:66-90) restated in oracle/oracle.c, OpenMP over
    all host cores.  Each step is a bounded row slab of the workload."""
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import oracle as O

    m, n, k = WORKLOADS[workload]
    rows = 64
    a = O.cast_e4m3(O.fill_normal((rows, k), SEED, 0))
    b = O.cast_e4m3(O.fill_normal((n, k), SEED, 1))
    sfa = O.fill_uniform((k // 128, rows), SEED, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), SEED, 3, 0.8, 1.2)
    t0 = time.perf_counter()
    O.gemm_ref_blockscale(a, b, sfa, sfb, out_bf16=True)
    probe = time.perf_counter() - t0
    # size a step so that the whole run (warm-up + timed steps) stays near 90 s, at most 2 s per step
    target = min(2.0, 90.0 / max(1, args.steps + args.warmup))
    rows = int(min(m, max(16, 64 * (target / max(probe, 1e-3)))))
    rows = max(16, rows - rows % 16)
    a = O.cast_e4m3(O.fill_normal((rows, k), SEED, 0))
    sfa = O.fill_uniform((k // 128, rows), SEED, 2, 0.8, 1.2)
    for _ in range(args.warmup):
        O.gemm_ref_blockscale(a, b, sfa, sfb, out_bf16=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.gemm_ref_blockscale(a, b, sfa, sfb, out_bf16=True)
    dt = time.perf_counter() - t0
    tf = 2.0 * rows * n * k * args.steps / dt / 1e12
    cores = O.num_threads()
    sample = f"{rows} of {m} rows x N={n} x K={k} per step (row slab of the same workload)"
    print(json.dumps({
        "impl": "reference", "metric": "fp8_blockscale_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{workload}_blockscale_M{m}_N{n}x{world}_K{k}", "scales": "A 1x128 fp32 [K/128][M], B 128x128 fp32",
                   "out": "bf16", "seed": SEED, "note": "CPU restatement of the reference host loop (all host threads, row slab "
                   "per step); the HIP reference cannot be built in this image"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline_leg(workload):
    """Bounded CPU sample (about 10-20 s) of the same workload with the oracle, reported beside the GPU number."""
    from oracle import oracle as O

    m, n, k = WORKLOADS[workload]
    b = O.cast_e4m3(O.fill_normal((n, k), SEED, 1))
    sfb = O.fill_uniform((n // 128, k // 128), SEED, 3, 0.8, 1.2)

    def run(rows):
        a = O.cast_e4m3(O.fill_normal((rows, k), SEED, 0))
        sfa = O.fill_uniform((k // 128, rows), SEED, 2, 0.8, 1.2)
        t0 = time.perf_counter()
        O.gemm_ref_blockscale(a, b, sfa, sfb, out_bf16=True)
        return time.perf_counter() - t0

    run(16)
    probe = run(64)
    rows = int(min(m, max(64, 64 * (12.0 / max(probe, 1e-3)))))
    rows -= rows % 16
    dt = run(rows)
    return {"value": 2.0 * rows * n * k / dt / 1e12, "unit": "TFLOP/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{rows} of {m} rows x N={n} x K={k}, one pass, {dt:.1f} s"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--tile", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--serialize", action="store_true", help="do not flag the operands as independent of the previous step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        cpu_reference_arm(args, args.workload, rank, world)
        return

    import torch
    import torch.distributed as dist

    from gcnasm_b200 import _lib as L
    from gcnasm_b200 import api

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # leave 16 SMs to the NCCL kernel of the activation broadcast and keep NCCL within them (config 2 has
        # 448 pair tiles: 66 resident pairs need the same 7 rounds as 74, so the GEMM loses nothing)
        os.environ.setdefault("NCCL_MAX_NCHANNELS", "16")
        os.environ.setdefault("B200GEMM_MAX_SMS", str(torch.cuda.get_device_properties(dev).multi_processor_count - 16))
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node N for --gpus N"

    m, n, k = WORKLOADS[args.workload]
    kg = k // 128
    # ---- synthetic operands: seeded N(0,1) on the host, quantised on the device ----------------------
    # several operand sets are rotated so that consecutive steps never find their inputs in L2
    set_bytes = m * k + n * k + m * n * 2
    nsets = max(2, min(8, int(np.ceil(3 * 126e6 / set_bytes))))
    xb = torch.from_numpy(api.fill_normal((n, k), SEED + rank, 1)).to(dev)
    qb0, sfb0 = api.quantize_128x128(xb)
    del xb
    xa = torch.from_numpy(api.fill_normal((m, k), SEED, 0)).to(dev)
    qa0, sfa0 = api.quantize_1x128(xa)
    del xa
    sets = []
    act_bufs = []
    for i in range(nsets):
        # distinct buffers with the same statistics: row-rotated copies of the quantised operands
        sh = (i * 128) % m
        # A and SFA live back to back in one buffer (one broadcast moves both)
        act = torch.empty(m * k + 4 * kg * m, dtype=torch.uint8, device=dev)
        qa = act[:m * k].view(m, k)
        sfa = act[m * k:].view(torch.float32).view(kg, m)
        qa.copy_(torch.roll(qa0, sh, 0))
        sfa.copy_(torch.roll(sfa0, sh, 1))
        act_bufs.append(act)
        shb = (i * 128) % n
        qb = torch.roll(qb0, shb, 0).contiguous()
        sfb = torch.roll(sfb0, shb // 128, 0).contiguous()
        sets.append((qa, sfa, qb, sfb, torch.empty(m, n, dtype=torch.bfloat16, device=dev)))
    torch.cuda.synchronize()

    # N-sharded mode: rank 0 owns the activation; A and SFA of a set share one buffer so that one broadcast moves
    # both.  The broadcast of step i+1 runs on a side stream while the GEMM of step i computes (the GEMM grid
    # leaves a few SMs to NCCL, see B200GEMM_MAX_SMS); the GEMM of a step waits for its own broadcast.
    comm = torch.cuda.Stream() if world > 1 else None
    pending = {}
    gemm_done = {}

    def post_broadcast(i):
        qa, sfa, qb, sfb, out = sets[i % nsets]
        prev = gemm_done.get(i - nsets)
        with torch.cuda.stream(comm):
            if prev is not None:
                comm.wait_event(prev)              # the GEMM that last read this set's activation has finished
            pending[i] = dist.broadcast(act_bufs[i % nsets], src=0, async_op=True)

    def step(i, last):
        qa, sfa, qb, sfb, out = sets[i % nsets]
        if world > 1:
            if i not in pending:
                post_broadcast(i)
            pending.pop(i).wait()                  # the current stream waits for this step's activation
            if not last:
                post_broadcast(i + 1)
        # the operand sets rotate and are never written inside the loop, so a step's inputs do not depend on the previous
        # step: the launch may overlap the previous kernel's tail; its writes to C still wait for that kernel
        api.gemm_a8w8_blockscale(qa, qb, sfa, sfb, out=out, tile=args.tile, inputs_ready=not args.serialize)
        if world > 1:
            ev = torch.cuda.Event()
            ev.record()
            gemm_done[i] = ev
            gemm_done.pop(i - 2 * nsets, None)

    step_no = [0]

    def run(count):
        for j in range(count):
            step(step_no[0], last=(j == count - 1))
            step_no[0] += 1

    run(args.warmup)
    torch.cuda.synchronize()
    # start the clock sampler BEFORE the barrier: every rank must enter the timed region together
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = api.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(args.steps)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = api.launch_count() - launches0
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    status = api.last_status()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    flop_step = 2.0 * m * n * k * world
    value = flop_step / (ms_step * 1e-3) / 1e12

    # ---- kernel-only duration of the GEMM (roofline numerator), one event pair per launch ------------
    kern_ms = []
    for i in range(min(args.steps, 50)):
        qa, sfa, qb, sfb, out = sets[i % nsets]
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        api.gemm_a8w8_blockscale(qa, qb, sfa, sfb, out=out, tile=args.tile)
        a1.record()
        kern_ms.append((a0, a1))
    torch.cuda.synchronize()
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in kern_ms]))
    # back-to-back launches hide the launch gap, so the loop average is the better per-launch figure at 1 GPU
    launch_ms = ms_step if world == 1 else kern_ms
    peaks = measured_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    achieved = 2.0 * m * n * k / (launch_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "kernel": "gemm_a8w8_pair_sm100_kernel<256x256 pair tile, block-scale>",
                "peak_source": f"2 x bf16 cuBLAS burst ({peaks['bf16_tflops']} TFLOP/s, {peaks['source']}); fp8 issues at twice the bf16 rate",
                "frac_of_nominal_4500": achieved / 4500.0,
                # `achieved` uses the average time per launch over the timed region, in which consecutive launches overlap
                # (the next one starts on SMs the previous one's last, partly filled wave leaves idle); a launch timed
                # alone between two events of its own is reported beside it
                "launch_ms": launch_ms, "isolated_launch_ms": kern_ms,
                "achieved_isolated": 2.0 * m * n * k / (kern_ms * 1e-3) / 1e12,
                "frac_isolated": 2.0 * m * n * k / (kern_ms * 1e-3) / 1e12 / fp8_peak}

    # ---- end to end through the host-buffer entry point ----------------------------------------------
    e2e = None
    if not args.no_e2e:
        qa, sfa, qb, sfb, out = sets[0]
        h = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (qa, qb, sfa, sfb)]
        for dst, src in zip(h, (qa, qb, sfa, sfb)):
            dst.copy_(src)
        hc = torch.empty((m, n), dtype=torch.uint16).pin_memory()
        ha, hb, hsfa, hsfb = (t.numpy() for t in h)
        hcn = hc.numpy()
        esteps = max(3, min(args.steps, 20))

        def e2e_step():
            api.gemm_a8w8_host(ha, hb, hcn, sfa=hsfa, sfb=hsfb, scale_mode=L.SCALE_BLOCK, tile=args.tile)

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(esteps):
            e2e_step()
        s1.record()
        torch.cuda.synchronize()
        ems = s0.elapsed_time(s1)
        if world > 1:
            t = torch.tensor([ems], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
        e2e = {"value": flop_step / (ems / esteps * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(ha.nbytes + hb.nbytes + hsfa.nbytes + hsfb.nbytes), "d2h_bytes_per_step": int(hcn.nbytes),
               "ms_per_step": ems / esteps, "api": "b200_gemm_a8w8_host (pinned host operands in, bf16 result out)"}

    # ---- skinny-M decode on pre-shuffled weights (config 4), reported as HBM GB/s beside the headline ----
    decode = None
    if world == 1 and not args.no_decode:
        dn, dk = 18432, 7168
        peaks_hbm = measured_peaks()["hbm_gbs"]
        wsrc = torch.from_numpy(api.fill_uniform((dn, dk), SEED, 11, -1.0, 1.0)).to(dev)
        wq, wsf = api.quantize_128x128(wsrc)
        del wsrc
        flat = api.shuffle_b(wq, "nk")
        # four weight images (528 MB) are rotated so that no launch finds its weights in L2
        flats = [flat] + [torch.roll(flat, 4096 * (j + 1)).contiguous() for j in range(3)]
        decode = []
        for dm in (1, 16, 64):
            xq, xsf = api.quantize_1x128(torch.from_numpy(api.fill_uniform((dm, dk), SEED, 12, -1.0, 1.0)).to(dev))
            dout = torch.empty(dm, dn, dtype=torch.bfloat16, device=dev)
            for j in range(8):
                api.gemm_a8w8_blockscale(xq, flats[j % 4], xsf, wsf, out=dout, b_flat_n=dn)
            torch.cuda.synchronize()
            # a 20-30 us kernel is shorter than the host-side cost of issuing it from Python, so the launches are
            # captured once in a CUDA graph (one launch per weight image) and the graph is replayed
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for j in range(4):
                        api.gemm_a8w8_blockscale(xq, flats[j], xsf, wsf, out=dout, b_flat_n=dn)
            torch.cuda.current_stream().wait_stream(side)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 200
            d0.record()
            for j in range(reps // 4):
                graph.replay()
            d1.record()
            torch.cuda.synchronize()
            us = d0.elapsed_time(d1) / reps * 1e3
            nbytes = dn * dk + dm * dk + 4 * (dn // 128) * (dk // 128) + 4 * dm * (dk // 128) + 2 * dm * dn
            gbs = nbytes / us / 1e3
            decode.append({"m": dm, "n": dn, "k": dk, "us": us, "gbs": gbs, "bytes": nbytes,
                           "frac_of_measured_hbm": gbs / peaks_hbm, "frac_of_nominal_8000": gbs / 8000.0})
        del flats, flat, wq

    # ---- fused activation quantiser (bf16 -> e4m3 + [K/128][M] scales), config 5's activation matrix ----
    act_quant = None
    if world == 1 and not args.no_decode:
        am, ak = 16384, 8192
        xb = torch.randn(am, ak, device=dev, dtype=torch.float32).to(torch.bfloat16)
        aq = torch.empty(am, ak, dtype=torch.uint8, device=dev)
        asf = torch.empty(ak // 128, am, dtype=torch.float32, device=dev)
        for _ in range(3):
            api.quantize_act_bf16_1x128(xb, q=aq, sfa=asf)
        torch.cuda.synchronize()
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for _ in range(20):
            api.quantize_act_bf16_1x128(xb, q=aq, sfa=asf)
        q1.record()
        torch.cuda.synchronize()
        qus = q0.elapsed_time(q1) / 20 * 1e3
        qbytes = am * ak * 3 + 4 * am * (ak // 128)            # bf16 in, e4m3 out, fp32 scales out: 407 MB > L2
        act_quant = {"m": am, "k": ak, "us": qus, "bytes": qbytes, "gbs": qbytes / qus / 1e3,
                     "frac_of_measured_hbm": qbytes / qus / 1e3 / measured_peaks()["hbm_gbs"]}
        del xb, aq, asf

    # ---- in-repo HBM probe: read-only and read+write streams over 2 GiB ----
    hbm_probe = None
    if world == 1 and not args.no_decode:
        pb = torch.empty(2 << 30, dtype=torch.uint8, device=dev).fill_(3)
        pc = torch.empty_like(pb)
        psum = torch.zeros(1, dtype=torch.int32, device=dev)
        hbm_probe = {"bytes": pb.numel()}
        for name, fn, moved in (("read_gbs", lambda: api.membw_read(pb, psum), 1), ("copy_gbs", lambda: api.membw_copy(pb, pc), 2)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record()
            for _ in range(10):
                fn()
            p1.record()
            torch.cuda.synchronize()
            hbm_probe[name] = moved * pb.numel() / (p0.elapsed_time(p1) / 10) / 1e6
        hbm_probe["measured_peaks_hbm_gbs"] = measured_peaks()["hbm_gbs"]
        del pb, pc

    # ---- a16w16 sibling: bf16 GEMM at 8192^3 against the measured cuBLAS bf16 rate ----
    a16w16 = None
    if world == 1 and not args.no_decode:
        bm = bn = bk = 8192
        xa = (torch.randn(bm, bk, device=dev) * 0.5).to(torch.bfloat16)
        xw = (torch.randn(bn, bk, device=dev) * 0.5).to(torch.bfloat16)
        xo = torch.empty(bm, bn, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            api.gemm_a16w16(xa, xw, out=xo)
        torch.cuda.synchronize()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(10):
            api.gemm_a16w16(xa, xw, out=xo)
        b1.record()
        torch.cuda.synchronize()
        bms = b0.elapsed_time(b1) / 10
        btf = 2.0 * bm * bn * bk / bms / 1e9
        a16w16 = {"m": bm, "n": bn, "k": bk, "ms": bms, "tflops": btf,
                  "frac_of_measured_bf16": btf / measured_peaks()["bf16_tflops"]}
        del xa, xw, xo

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_leg(args.workload)

    if rank == 0:
        line = {
            "metric": "fp8_blockscale_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp32 accumulate, bf16 out)", "data": "synthetic",
            "config": {"workload": f"{args.workload}_blockscale_M{m}_N{n}x{world}_K{k}",
                       "scales": "A 1x128 fp32 [K/128][M], B 128x128 fp32", "out": "bf16",
                       "parallelism": f"N-sharded x{world}, A+SFA NCCL broadcast per step" if world > 1 else "single GPU",
                       "l2": f"rotating {nsets} operand sets ({nsets * set_bytes / 1e6:.0f} MB) larger than the 126 MB L2",
                       "seed": SEED,
                       "launch": "each step one launch; consecutive launches chained by programmatic dependent launch"
                                 + ("" if args.serialize else ", operands flagged independent of the previous step")},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "kernel_ms": kern_ms, "device_status": status,
            "decode": decode, "act_quant": act_quant, "hbm_probe": hbm_probe, "a16w16": a16w16,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
