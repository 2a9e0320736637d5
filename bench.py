#!/usr/bin/env python
"""Benchmark of the A8W8 FP8 block-scale GEMM hot path (one JSON line on stdout).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sections a,b,...]

Headline (every N): the column-parallel block-scale GEMM of the large-N configuration, M=16384, N=57344, K=8192,
seeded N(0,1) data quantised on the device (A 1x128, B 128x128, amax/448), bf16 output.  B is sharded along N over
the N ranks (57344/N columns each: STRONG scaling, the whole problem at N=1); the root owns the activation and
broadcasts A + SFA over NCCL every step, in 2048-row slabs on a side stream, while one persistent GEMM launch per
rank consumes the slabs as they land (gcnasm_b200.sharded.ColumnShardedGemm).  Outputs stay N-sharded.  A step is
`calls_per_step` such calls back to back (so that the timed region is long enough for the clock sampler);
`value` = whole-job FLOP / device time, operands resident in HBM; `e2e` = the same call with the activation coming
from pinned host memory on the root and every rank's C shard going back to pinned host memory, every step.
After the timed loop every rank recomputes sampled rows of its shard with the device checker kernel
(`parity_checked`).

At N=1 the line also carries the other configurations as sections: `c2` (4096x7168x2048 block-scale: serialised and
overlapped launches, and end to end through b200_gemm_a8w8_host), `cube8192_blockscale`, `cube8192_mx` (MXFP8),
`c1_per_tensor`, `decode` (skinny-M on pre-shuffled weights, HBM GB/s), `act_quant`, `hbm_probe`, `a16w16`.

`--impl reference` times the reference's own host GEMM loop on the host cores: the reference's gemm_ref compiled
from its source (oracle/_ref) when that binary is present, else its line-by-line restatement (oracle/oracle.c).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# torchrun exports OMP_NUM_THREADS=1; the seeded host generators and the CPU arm are OpenMP code and the ranks of one
# box share its cores (must happen before anything loads libgomp)
if "LOCAL_WORLD_SIZE" in os.environ and os.environ.get("OMP_NUM_THREADS", "1") == "1":
    os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // int(os.environ["LOCAL_WORLD_SIZE"])))

import numpy as np  # noqa: E402

C5 = (16384, 57344, 8192)          # M, N (whole problem), K
SEED = 1234
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from ncu captures of exactly these
# launches (columns per launch -> bytes): the whole problem on one GPU, and the per-rank launch of 8 ranks
C5_DRAM_BYTES = {57344: 10.37e9, 7168: 824.9e6}
ALL_SECTIONS = ("c2", "cube8192_blockscale", "cube8192_mx", "c1_per_tensor", "decode", "act_quant", "hbm_probe", "a16w16")


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
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples; with t_begin/t_end only those taken inside the timed region count."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power, inside = [], [], set(), [], 0
        for ts, ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            if t_begin is not None and not (t_begin <= ts <= t_end + 0.05):
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            inside += 1
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples inside the timed region"], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": inside,
                "power_w_max": max(power) if power else None, "window": "samples taken inside the timed region only"}


# ------------------------------------------------------------------------------------------------------------
# CPU: the reference's host loop (the --impl reference arm and the cpu_baseline leg)
# ------------------------------------------------------------------------------------------------------------
def _cpu_gemm_runner():
    """Returns (kind, run(a, b, sfa, sfb) -> seconds, cores).  'reference' = the reference's own gemm_ref compiled from its
    source by oracle/ref_build.py (built with the reference Makefile's flags); 'port' = the C restatement."""
    from oracle import oracle as O
    from oracle import ref as R

    cores = O.num_threads()
    if R.available():
        def run(a, b, sfa, sfb):
            t0 = time.perf_counter()
            R.gemm_ref_blockscale(a, b, sfa, sfb, flavour="fast")
            return time.perf_counter() - t0
        return "reference", run, cores

    def run(a, b, sfa, sfb):
        t0 = time.perf_counter()
        O.gemm_ref_blockscale(a, b, sfa, sfb)
        return time.perf_counter() - t0
    return "port", run, cores


def _cpu_operands(rows, n, k):
    from oracle import oracle as O

    a = O.cast_e4m3(O.fill_normal((rows, k), SEED, 0))
    b = O.cast_e4m3(O.fill_normal((n, k), SEED, 1))
    sfa = O.fill_uniform((k // 128, rows), SEED, 2, 0.8, 1.2)
    sfb = O.fill_uniform((n // 128, k // 128), SEED, 3, 0.8, 1.2)
    return a, b, sfa, sfb


CPU_N = 7168   # the CPU legs use one 7168-column shard of the weights: the loop's cost per output element does not depend on N


def cpu_reference_arm(args, rank, world):
    """--impl reference: the reference's CPU implementation of the path -- its host gemm_ref loop (block-scale variant,
    opus_gemm/block_scale_gemm/gemm_a8w8_blockscale_host.cc:66-90), OpenMP over all host cores.  Each step is a bounded
    row slab of the headline workload."""
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    m, n, k = C5
    kind, run, cores = _cpu_gemm_runner()
    a, b, sfa, sfb = _cpu_operands(16, CPU_N, k)
    probe = run(a, b, sfa, sfb)
    # size a step so that the whole run (warm-up + timed steps) stays near 90 s, at most 2 s per step
    target = min(2.0, 90.0 / max(1, args.steps + args.warmup))
    rows = int(min(m, max(16, 16 * (target / max(probe, 1e-3)))))
    rows = max(16, rows - rows % 16)
    a, b, sfa, sfb = _cpu_operands(rows, CPU_N, k)
    for _ in range(args.warmup):
        run(a, b, sfa, sfb)
    dt = sum(run(a, b, sfa, sfb) for _ in range(args.steps))
    tf = 2.0 * rows * CPU_N * k * args.steps / dt / 1e12
    sample = (f"{rows} of {m} rows x {CPU_N} of {n} columns x K={k} per step (a slab of the same workload; fp32 output as "
              "the reference's loop writes it)")
    note = ("the reference's own gemm_ref, compiled from its source with the flags of its Makefile (oracle/_ref)" if kind == "reference"
            else "line-by-line C restatement of the reference's gemm_ref (oracle/oracle.c); oracle/_ref is not present on this machine")
    print(json.dumps({
        "impl": "reference", "metric": "fp8_blockscale_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": workload_config(world), "note": note,
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline_leg():
    """Bounded CPU sample (10-20 s) of the headline workload, reported beside the GPU number."""
    m, n, k = C5
    kind, run, cores = _cpu_gemm_runner()
    a, b, sfa, sfb = _cpu_operands(16, CPU_N, k)
    run(a, b, sfa, sfb)
    probe = run(a, b, sfa, sfb)
    rows = int(min(m, max(16, 16 * (12.0 / max(probe, 1e-3)))))
    rows -= rows % 16
    a, b, sfa, sfb = _cpu_operands(rows, CPU_N, k)
    dt = run(a, b, sfa, sfb)
    return {"value": 2.0 * rows * CPU_N * k / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"{rows} of {m} rows x {CPU_N} of {n} columns x K={k}, one pass, {dt:.1f} s"}


def workload_config(world):
    """The same dictionary in both arms (what the workload IS; what a run measured about itself goes under "run")."""
    m, n, k = C5
    return {"workload": f"c5_blockscale_M{m}_N{n}_K{k}_sharded_over_{world}",
            "scales": "A 1x128 fp32 [K/128][M], B 128x128 fp32", "out": "bf16", "seed": SEED,
            "parallelism": (f"B column-sharded x{world} ({n // world} columns per rank), A+SFA sent from rank 0 to every rank every call "
                            "in row slabs, outputs stay sharded" if world > 1 else "single GPU, whole problem"),
            "l2": "operands of one call (A+SFA 138 MB, B shard >= 59 MB, C shard >= 235 MB) exceed the 126 MB L2; two activation "
                  "and two output buffers alternate"}


# ------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sections", default="all", help="comma-separated extra sections at N=1 (all, none, or names)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--min-timed-s", type=float, default=0.5)
    ap.add_argument("--delivery", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the activation slabs reach the ranks (copy-engine chain, or NCCL broadcasts)")
    ap.add_argument("--comm-sms", type=int, default=0, help="SMs left to NCCL beside the persistent GEMM grid (N > 1); 0 = the package's default")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        cpu_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    from gcnasm_b200 import _lib as L
    from gcnasm_b200 import api
    from gcnasm_b200.sharded import ColumnShardedGemm, configure_overlap, default_comm_sms, shard_bounds

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    if world > 1:
        if args.delivery == "nccl":
            args.comm_sms = args.comm_sms or default_comm_sms(world)
            configure_overlap(world, sms, args.comm_sms)
        else:
            args.comm_sms = 0                      # the copy engines deliver: the GEMM keeps every SM
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)     # NCCL's kernels before pending GEMM blocks
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node N for --gpus N"
    peaks = measured_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops"]

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def timed(fn, reps, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def allmax(x):
        if world == 1:
            return float(x)
        t = torch.tensor([float(x)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- operands of the headline workload ---------------------------------------------------------------
    m, n_total, k = C5
    n0, n1 = shard_bounds(n_total, world, rank)
    n = n1 - n0
    kg = k // 128
    chunk = 7168                                   # weight rows generated, uploaded and quantised at a time
    qb = torch.empty(n, k, dtype=torch.uint8, device=dev)
    sfb = torch.empty(n // 128, kg, dtype=torch.float32, device=dev)
    for c0 in range(0, n, chunk):
        # every 7168-row block of B is its own seeded stream (tensor ids 16, 17, ...), so a rank's shard does not
        # depend on how many ranks there are
        xb = torch.from_numpy(api.fill_normal((chunk, k), SEED, 16 + (n0 + c0) // chunk)).to(dev)
        q, s = api.quantize_128x128(xb)
        qb[c0:c0 + chunk].copy_(q)
        sfb[c0 // 128:(c0 + chunk) // 128].copy_(s)
        del xb, q, s
    op = ColumnShardedGemm(qb, sfb, n_total, delivery=args.delivery)
    plan = op.plan_slabs(m, k, dev, nbuf=2)
    delivery_used, delivery_note = op.delivery, op.delivery_note       # "nccl" with a note if the GPUs cannot map each other
    if rank == 0:
        # two activations (N(0,1), two seeded streams), quantised once straight into the two ring buffers; they
        # stay resident in HBM, and every step broadcasts one of them again
        for bi in range(plan.nbuf):
            _, a3, sfa3 = op.slab_views(bi)
            for s in range(plan.slabs):
                xa = torch.from_numpy(api.fill_normal((plan.rows, k), SEED, 1000 * bi + s)).to(dev)
                q, sf = api.quantize_1x128(xa)
                a3[s].copy_(q)
                sfa3[s].copy_(sf)
                del xa, q, sf
    outs = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()

    # ---- the step: post the next call's activation, run this call ----------------------------------------------
    state = {"next": 0, "posted": -1}

    def post(i):
        if state["posted"] < i:
            op.post(i, prefilled=True)
            state["posted"] = i

    def call():
        i = state["next"]
        post(i)
        post(i + 1)                 # the next call's slabs travel behind this call's GEMM (two activation buffers)
        op.run(i, outs[i % 2])
        state["next"] = i + 1

    def one_call_ms(burst=8):
        # steady-state time of a call (a burst back to back): a single call on an idle device shows its whole delivery
        # and would make the timed region come out shorter than asked for
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(burst):
            call()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / burst

    call()
    call()
    t_call = allmax(one_call_ms())
    calls_per_step = int(min(64, max(1, np.ceil(args.min_timed_s * 1e3 / (max(args.steps, 1) * t_call)))))
    for _ in range(args.warmup):
        for _ in range(calls_per_step):
            call()
    torch.cuda.synchronize()
    # start the clock sampler BEFORE the barrier: every rank must enter the timed region together
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = api.launch_count()
    t_begin = time.time()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(args.steps):
        for _ in range(calls_per_step):
            call()
    e1.record()
    torch.cuda.synchronize()
    t_end = time.time()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = api.launch_count() - launches0
    ms = allmax(e0.elapsed_time(e1))
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    status = api.last_status()
    ms_step = ms / args.steps
    flop_call = 2.0 * m * n_total * k
    value = flop_call * calls_per_step / (ms_step * 1e-3) / 1e12

    # ---- parity inside the run: sampled rows of this rank's shard against the device checker kernel ----------
    last = state["next"] - 1
    torch.cuda.synchronize()
    perr, pref = 0.0, 0.0
    for row0 in (plan.rows - 128, m - plan.rows + 256):          # one block in the first slab, one in the last
        e_, r_ = op.check_rows(last, outs[last % 2], row0, 128)
        perr, pref = max(perr, e_), max(pref, r_)
    torch.cuda.synchronize()
    parity_ok = perr <= 1e-2 * pref
    parity = {"checked": bool(allmax(0.0 if parity_ok else 1.0) == 0.0), "max_err_over_max_ref": allmax(perr / max(pref, 1e-30)),
              "tolerance": 1e-2, "what": "2 x 128 rows x all shard columns per rank, b200_gemm_a8w8_simple on the delivered slabs"}

    # ---- the dominant kernel on its own: serialised launches of this rank's GEMM, slabs already delivered ------
    _, a3, sfa3 = op.slab_views(0)
    ready_all = torch.full((plan.slabs,), 1 << 30, dtype=torch.int32, device=dev)
    out3 = outs[0].view(plan.slabs, plan.rows, n)

    def local_gemm():
        api.gemm_a8w8_blockscale(a3, qb, sfa3, sfb, out=out3, batch_ready=ready_all, batch_epoch=1)

    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    # kernel duration = launches of this one kernel back to back in stream order (the reference's benchmark protocol,
    # gemm_a8w8_blockscale_host.cc:99-121), nothing else running; a launch timed alone on an idle device is reported
    # beside it (it includes the launch latency)
    reps = max(20, min(400, int(300.0 / max(t_call, 0.1))))       # about 0.3 s of launches: a sustained figure, like the loop's
    for _ in range(3):
        local_gemm()
    torch.cuda.synchronize()
    k0, k1 = ev(), ev()
    k0.record()
    for _ in range(reps):
        local_gemm()
    k1.record()
    torch.cuda.synchronize()
    kern_ms = allmax(k0.elapsed_time(k1) / reps)
    kern = []
    for _ in range(5):
        a0, a1 = ev(), ev()
        a0.record()
        local_gemm()
        a1.record()
        torch.cuda.synchronize()
        kern.append(a0.elapsed_time(a1))
    idle_ms = allmax(float(np.mean(kern)))
    # One call on its own, delivery included: every rank idle, then post + run.  What it takes beyond the kernel is the
    # part of the delivery that a single call cannot hide (the first slab's way down to the last rank).  With NCCL the
    # whole delivery is also timed without any GEMM beside it.
    def drain():
        i = state["next"]
        if state["posted"] >= i:                   # a step posted ahead by the loop: run it so that the ring stays in step
            op.run(i, outs[i % 2])
            state["next"] = i + 1

    delivery = None
    if world > 1:
        iso, dl = [], []
        for _ in range(4):
            drain()
            i = state["next"]
            torch.cuda.synchronize()
            dist.barrier()
            c0, c1 = ev(), ev()
            c0.record()
            op.post(i, prefilled=True)
            state["posted"] = i
            op.run(i, outs[i % 2])
            c1.record()
            torch.cuda.synchronize()
            state["next"] = i + 1
            iso.append(c0.elapsed_time(c1))
        if op.delivery == "nccl":
            for _ in range(4):
                drain()
                i = state["next"]
                torch.cuda.synchronize()
                dist.barrier()
                d0, d1 = ev(), ev()
                with torch.cuda.stream(op._comm):
                    d0.record()
                op.post(i, prefilled=True)
                state["posted"] = i
                with torch.cuda.stream(op._comm):
                    d1.record()
                torch.cuda.synchronize()
                dl.append(d0.elapsed_time(d1))
            drain()
        torch.cuda.synchronize()
        dbytes = plan.slabs * plan.bytes_per_slab
        iso_ms = allmax(float(np.median(iso)))
        delivery = {"how": ("ncclBroadcast per slab on a side stream, NCCL held to %s channels" % os.environ.get("NCCL_MAX_NCHANNELS")
                            if op.delivery == "nccl" else
                            "copy-engine pushes down the chain of ranks (b200_stream_copy over peer-mapped memory), no SM"),
                    "slabs": plan.slabs, "bytes": dbytes, "isolated_call_ms": iso_ms, "kernel_ms": kern_ms,
                    "exposed_in_isolated_call_ms": iso_ms - kern_ms}
        if dl:
            dms = allmax(float(np.median(dl)))
            delivery.update({"ms_alone": dms, "gbs_alone": dbytes / dms / 1e6})
    flop_local = 2.0 * m * n * k
    achieved = flop_local / (kern_ms * 1e-3) / 1e12
    traffic = C5_DRAM_BYTES.get(n)
    roofline = {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                "traffic": traffic,
                "traffic_source": ("ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum -k regex:gemm_a8w8_pair, one launch of "
                                   "exactly this shape, captured separately (a constant in this script, not measured in this run)" if traffic else
                                   "no ncu capture of this rank count's launch (captured: 1 and 8 ranks; B re-reads do not scale with N)"),
                "kernel": "gemm_a8w8_pair_sm100_kernel<PairCfg<256, block-scale, row-major B>>",
                "kernel_ms": kern_ms, "launches_timed": reps, "timing": "launches of this kernel alone, back to back in stream order",
                "kernel_ms_idle_device": idle_ms,
                "peak_source": f"2 x bf16 cuBLAS burst ({peaks['bf16_tflops']} TFLOP/s, {peaks['source']}): no FP8 figure is measured; "
                               "FP8 issues at twice the bf16 rate",
                "frac_of_nominal_4500": achieved / 4500.0, "algorithmic_flop_per_launch": flop_local,
                # the timed loop itself: consecutive calls overlap (programmatic dependent launch, slabs delivered ahead)
                "loop_ms_per_call": ms_step / calls_per_step,
                "frac_loop": (flop_local / (ms_step / calls_per_step * 1e-3) / 1e12) / fp8_peak}

    # ---- end to end: activation from pinned host memory on the root, C shard back to pinned host memory -------
    e2e = None
    if not args.no_e2e:
        ha = hsfa = None
        if rank == 0:
            ha = torch.empty(m, k, dtype=torch.uint8).pin_memory()
            hsfa = torch.empty(kg, m, dtype=torch.float32).pin_memory()
            _, a3_, sfa3_ = op.slab_views(0)
            ha.copy_(a3_.reshape(m, k))
            hsfa.copy_(torch.cat(list(sfa3_), dim=1))
        hc = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
        d2h = torch.cuda.Stream()
        copied = [None, None]

        def e2e_call():
            i = state["next"]
            if copied[i % 2] is not None:
                torch.cuda.current_stream().wait_event(copied[i % 2])      # the copy-back that last read this C buffer
            op.post(i, a=ha, sfa=hsfa)
            op.run(i, outs[i % 2])
            done = torch.cuda.Event()
            done.record()
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                hc.copy_(outs[i % 2], non_blocking=True)                  # overlaps the next call's upload and GEMM
                copied[i % 2] = torch.cuda.Event()
                copied[i % 2].record()
            state["next"] = i + 1
            state["posted"] = i

        esteps = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_call()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s0, s1 = ev(), ev()
        s0.record()
        for _ in range(esteps):
            e2e_call()
        torch.cuda.current_stream().wait_stream(d2h)
        s1.record()
        torch.cuda.synchronize()
        ems = allmax(s0.elapsed_time(s1))
        got = hc[plan.rows - 128:plan.rows].float()
        same = bool(torch.equal(got, outs[(state["next"] - 1) % 2][plan.rows - 128:plan.rows].float().cpu()))
        e2e = {"value": flop_call / (ems / esteps * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(m * k + 4 * kg * m), "d2h_bytes_per_step": int(m * n * 2) * world,
               "ms_per_step": ems / esteps, "steps": esteps, "result_on_host_matches_device": same,
               "api": "ColumnShardedGemm.post(a=, sfa= in pinned host memory) -> b200_slab_upload on the root, NCCL slab broadcast, "
                      "run(); every rank copies its bf16 C shard to pinned host memory; weights stay resident (as deployed)",
               "h2d_note": "uploaded by rank 0 only; d2h counts all ranks' shards"}

    # ---- sections at N=1 ---------------------------------------------------------------------------------------
    sections = {}
    want = ALL_SECTIONS if args.sections == "all" else tuple(s for s in args.sections.split(",") if s and s != "none")
    op.close()
    del outs, op, qb, sfb
    torch.cuda.empty_cache()
    if world == 1:
        for name in want:
            sections[name] = SECTION_FNS[name](torch, api, L, dev, peaks, timed)
            torch.cuda.empty_cache()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_leg()

    if rank == 0:
        line = {
            "metric": "fp8_blockscale_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp32 accumulate, bf16 out)", "data": "synthetic",
            "config": workload_config(world),
            "run": {"calls_per_step": calls_per_step, "ms_per_call": ms_step / calls_per_step,
                    "slabs": f"{plan.slabs} x {plan.rows} rows, {plan.bytes_per_slab} bytes each, {plan.nbuf} activation buffers",
                    "launch": "one GEMM launch per call (slabs = batches, ready words), chained by programmatic dependent launch",
                    "delivery": (delivery_used + (": " + delivery_note if delivery_note else "")) if world > 1 else "none (single rank)",
                    "comm_sms": args.comm_sms if world > 1 else 0, "gemm_sms": int(L.lib().b200_sm_count())},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "parity_checked": parity["checked"], "parity": parity, "device_status": status, "inner_repeats": calls_per_step,
            "delivery": delivery,
        }
        line.update(sections)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------------------
# sections (single GPU)
# ------------------------------------------------------------------------------------------------------------
def _blockscale_operands(torch, api, dev, m, n, k, nsets):
    xb = torch.from_numpy(api.fill_normal((n, k), SEED, 1)).to(dev)
    qb0, sfb0 = api.quantize_128x128(xb)
    del xb
    xa = torch.from_numpy(api.fill_normal((m, k), SEED, 0)).to(dev)
    qa0, sfa0 = api.quantize_1x128(xa)
    del xa
    sets = []
    for i in range(nsets):
        # distinct buffers with the same statistics: row-rotated copies of the quantised operands
        sh, shb = (i * 128) % m, (i * 128) % n
        sets.append((torch.roll(qa0, sh, 0).contiguous(), torch.roll(sfa0, sh, 1).contiguous(), torch.roll(qb0, shb, 0).contiguous(),
                     torch.roll(sfb0, shb // 128, 0).contiguous(), torch.empty(m, n, dtype=torch.bfloat16, device=dev)))
    return sets


def _gemm_section(torch, api, dev, peaks, sets, m, n, k, run, reps):
    """Serialised (each launch on an idle device, the reference's in-order protocol without the launch gap) and
    overlapped (consecutive independent launches) figures of one GEMM shape."""
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    flop = 2.0 * m * n * k
    for i in range(6):
        run(sets[i % len(sets)], False)
    torch.cuda.synchronize()
    ser = []
    for i in range(reps):
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        run(sets[i % len(sets)], False)
        a1.record()
        torch.cuda.synchronize()
        ser.append(a0.elapsed_time(a1))
    ser_ms = float(np.mean(ser))

    def loop(inputs_ready, count):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(count):
            run(sets[i % len(sets)], inputs_ready)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / count

    count = int(max(50, min(3000, 300.0 / max(ser_ms, 1e-3))))
    loop(False, 20)
    b2b_ms = loop(False, count)            # back to back in stream order, the reference's benchmark protocol
    ovl_ms = loop(True, count)             # operands flagged independent of the previous launch
    tf = lambda ms_: flop / (ms_ * 1e-3) / 1e12
    # ms = kernel duration: launches back to back in stream order, each waiting for its predecessor (the reference's
    # benchmark protocol); overlapped_* = consecutive INDEPENDENT launches (B200_GEMM_INPUTS_READY: the next one starts
    # on SMs the previous one's last, partly filled wave leaves idle); idle_device_ms = one launch alone, launch latency included
    return {"m": m, "n": n, "k": k, "flop": flop,
            "ms": b2b_ms, "tflops": tf(b2b_ms), "frac_of_2x_bf16": tf(b2b_ms) / fp8_peak, "frac_of_nominal_4500": tf(b2b_ms) / 4500.0,
            "overlapped_launch_ms": ovl_ms, "overlapped_tflops": tf(ovl_ms), "frac_overlapped": tf(ovl_ms) / fp8_peak,
            "idle_device_ms": ser_ms, "launches": count, "operand_sets": len(sets)}


def section_c2(torch, api, L, dev, peaks, timed):
    m, n, k = 4096, 7168, 2048
    sets = _blockscale_operands(torch, api, dev, m, n, k, 5)

    def run(s, ready):
        api.gemm_a8w8_blockscale(s[0], s[2], s[1], s[3], out=s[4], inputs_ready=ready)

    out = _gemm_section(torch, api, dev, peaks, sets, m, n, k, run, 50)
    out["l2"] = "5 operand sets (409 MB) rotate: no launch finds its inputs in the 126 MB L2"
    # end to end through the host-buffer entry (the reference main()'s copy-in / launch / copy-out data path)
    qa, sfa, qb, sfb, _ = sets[0]
    h = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (qa, qb, sfa, sfb)]
    for dst, src in zip(h, (qa, qb, sfa, sfb)):
        dst.copy_(src)
    hc = torch.empty((m, n), dtype=torch.uint16).pin_memory()
    ha, hb, hsfa, hsfb = (t.numpy() for t in h)
    hcn = hc.numpy()
    ems = timed(lambda: api.gemm_a8w8_host(ha, hb, hcn, sfa=hsfa, sfb=hsfb, scale_mode=L.SCALE_BLOCK), 10)
    out["host_entry"] = {"ms": ems, "tflops": 2.0 * m * n * k / ems / 1e9, "h2d_bytes": int(ha.nbytes + hb.nbytes + hsfa.nbytes + hsfb.nbytes),
                         "d2h_bytes": int(hcn.nbytes), "api": "b200_gemm_a8w8_host (all operands from pinned host memory, bf16 C back)"}
    return out


def section_cube_blockscale(torch, api, L, dev, peaks, timed):
    m = n = k = 8192
    sets = _blockscale_operands(torch, api, dev, m, n, k, 2)

    def run(s, ready):
        api.gemm_a8w8_blockscale(s[0], s[2], s[1], s[3], out=s[4], inputs_ready=ready)

    out = _gemm_section(torch, api, dev, peaks, sets, m, n, k, run, 20)
    out["target"] = "north_star: >= 0.70 of the nominal 4.5 PFLOP/s; reference publishes 0.4057 ms on MI355X (fp32 out)"
    return out


def section_cube_mx(torch, api, L, dev, peaks, timed):
    m = n = k = 8192
    xa = torch.from_numpy(api.fill_normal((m, k), SEED, 0)).to(dev)
    qa, _, sa = api.quantize_mx32(xa)
    del xa
    xb = torch.from_numpy(api.fill_normal((n, k), SEED, 1)).to(dev)
    qb, _, sb = api.quantize_mx32(xb)
    del xb
    sets = [(qa, sa, qb, sb, torch.empty(m, n, dtype=torch.bfloat16, device=dev)),
            (qa.clone(), sa.clone(), qb.clone(), sb.clone(), torch.empty(m, n, dtype=torch.bfloat16, device=dev))]

    def run(s, ready):
        api.gemm_a8w8_mx(s[0], s[2], s[1], s[3], out=s[4])

    return _gemm_section(torch, api, dev, peaks, sets, m, n, k, run, 20)


def section_c1(torch, api, L, dev, peaks, timed):
    """Config 1: 256 x 512 x 1024, per-tensor scales, bf16 out -- two tiles' worth of work, launch-latency bound."""
    m, n, k = 256, 512, 1024
    qa, sa = api.quantize_tensor(torch.from_numpy(api.fill_uniform((m, k), SEED, 0, -1.0, 1.0)).to(dev))
    qb, sb = api.quantize_tensor(torch.from_numpy(api.fill_uniform((n, k), SEED, 1, -1.0, 1.0)).to(dev))
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    api.gemm_a8w8(qa, qb, sa, sb, out=out)
    torch.cuda.synchronize()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(20):
                api.gemm_a8w8(qa, qb, sa, sb, out=out)
    torch.cuda.current_stream().wait_stream(side)
    us_graph = timed(graph.replay, 50) / 20 * 1e3
    us_plain = timed(lambda: api.gemm_a8w8(qa, qb, sa, sb, out=out), 200) * 1e3
    flop = 2.0 * m * n * k
    return {"m": m, "n": n, "k": k, "us_per_launch_graph": us_graph, "us_per_launch_python_loop": us_plain,
            "tflops_graph": flop / us_graph / 1e6, "note": "0.27 GFLOP per launch: bound by launch latency, not by the tensor pipe"}


def section_decode(torch, api, L, dev, peaks, timed):
    dn, dk = 18432, 7168
    wsrc = torch.from_numpy(api.fill_uniform((dn, dk), SEED, 11, -1.0, 1.0)).to(dev)
    wq, wsf = api.quantize_128x128(wsrc)
    del wsrc
    flat = api.shuffle_b(wq, "nk")
    # four weight images (528 MB) are rotated so that no launch finds its weights in L2
    flats = [flat] + [torch.roll(flat, 4096 * (j + 1)).contiguous() for j in range(3)]
    rows = []
    for dm in (1, 16, 64):
        xq, xsf = api.quantize_1x128(torch.from_numpy(api.fill_uniform((dm, dk), SEED, 12, -1.0, 1.0)).to(dev))
        dout = torch.empty(dm, dn, dtype=torch.bfloat16, device=dev)

        def one(j, ready=True):
            api.gemm_a8w8_blockscale(xq, flats[j % 4], xsf, wsf, out=dout, b_flat_n=dn, inputs_ready=ready)

        for j in range(8):
            one(j)
        torch.cuda.synchronize()
        # a 20-30 us kernel is shorter than the host-side cost of issuing it from Python, so the launches are
        # captured once in a CUDA graph (one launch per weight image) and the graph is replayed
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for j in range(4):
                    one(j)
        torch.cuda.current_stream().wait_stream(side)
        us = timed(graph.replay, 50) / 4 * 1e3
        # the same launches without a graph and without the weights vouched for (each waits for its predecessor
        # before it requests its first tile), issued from Python one by one; and one launch alone on an idle device
        us_loop = timed(lambda: [one(j, False) for j in range(4)], 25) / 4 * 1e3
        alone = []
        for j in range(12):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            one(j, False)
            a1.record()
            torch.cuda.synchronize()
            alone.append(a0.elapsed_time(a1) * 1e3)
        nbytes = dn * dk + dm * dk + 4 * (dn // 128) * (dk // 128) + 4 * dm * (dk // 128) + 2 * dm * dn
        gbs = nbytes / us / 1e3
        rows.append({"m": dm, "n": dn, "k": dk, "us": us, "gbs": gbs, "bytes": nbytes,
                     "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_nominal_8000": gbs / 8000.0,
                     "timing": "CUDA graph of 4 launches (one per weight image), weights flagged resident",
                     "us_python_loop_no_flag": us_loop, "us_single_launch_idle_device": float(np.median(alone)),
                     "gbs_single_launch": nbytes / float(np.median(alone)) / 1e3})
    return rows


def section_act_quant(torch, api, L, dev, peaks, timed):
    am, ak = 16384, 8192
    xb = torch.randn(am, ak, device=dev, dtype=torch.float32).to(torch.bfloat16)
    aq = torch.empty(am, ak, dtype=torch.uint8, device=dev)
    asf = torch.empty(ak // 128, am, dtype=torch.float32, device=dev)
    qus = timed(lambda: api.quantize_act_bf16_1x128(xb, q=aq, sfa=asf), 20) * 1e3
    qbytes = am * ak * 3 + 4 * am * (ak // 128)            # bf16 in, e4m3 out, fp32 scales out: 407 MB > L2
    return {"m": am, "k": ak, "us": qus, "bytes": qbytes, "gbs": qbytes / qus / 1e3,
            "frac_of_measured_hbm": qbytes / qus / 1e3 / peaks["hbm_gbs"]}


def section_hbm_probe(torch, api, L, dev, peaks, timed):
    pb = torch.empty(2 << 30, dtype=torch.uint8, device=dev).fill_(3)
    pc = torch.empty_like(pb)
    psum = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {"bytes": pb.numel()}
    for name, fn, moved in (("read_gbs", lambda: api.membw_read(pb, psum), 1), ("copy_gbs", lambda: api.membw_copy(pb, pc), 2)):
        out[name] = moved * pb.numel() / timed(fn, 10) / 1e6
    out["measured_peaks_hbm_gbs"] = peaks["hbm_gbs"]
    return out


def section_a16w16(torch, api, L, dev, peaks, timed):
    bm = bn = bk = 8192
    xa = (torch.randn(bm, bk, device=dev) * 0.5).to(torch.bfloat16)
    xw = (torch.randn(bn, bk, device=dev) * 0.5).to(torch.bfloat16)
    xo = torch.empty(bm, bn, dtype=torch.bfloat16, device=dev)
    bms = timed(lambda: api.gemm_a16w16(xa, xw, out=xo), 10)
    btf = 2.0 * bm * bn * bk / bms / 1e9
    return {"m": bm, "n": bn, "k": bk, "ms": bms, "tflops": btf, "frac_of_measured_bf16": btf / peaks["bf16_tflops"]}


SECTION_FNS = {"c2": section_c2, "cube8192_blockscale": section_cube_blockscale, "cube8192_mx": section_cube_mx,
               "c1_per_tensor": section_c1, "decode": section_decode, "act_quant": section_act_quant,
               "hbm_probe": section_hbm_probe, "a16w16": section_a16w16}


if __name__ == "__main__":
    main()
