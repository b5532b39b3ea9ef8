"""Benchmark of the quantized frozen-base LoRA linear on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + backward (dX, dA, dB) of the LoRA'd quantized linear over one
batch of synthetic activations; under torchrun each rank processes its own batch shard and
the LoRA gradients (one flat f32 bucket) are sum-allreduced over NCCL, which is the only
collective the data-parallel path has.  Rank 0 prints ONE JSON line.

Workload (`config.workload` = "cfg2"): fp8 e4m3 frozen MLP up-projection 3072 -> 12288 with
per-output-channel f32 scales from absmax, weights N(0, 0.02), LoRA rank 32 alpha 32, bf16
activations 8192 tokens x 3072 N(0,1), seeded dY.  FLOPs per step follow the single
algorithmic definition 4*N*K*M + 6*N*r*(K+M) = 1261.11 GFLOP; dequantisation, scaling, bias
and casts count as zero.

`--impl reference` times the reference's own op sequence on the host cores instead (dequantize
to a full f32 weight on every pass, f32 sgemm, LoRA as separate sgemms — the restatement in
oracle/, since loractl itself is Rust on burn and cannot be built here), on a bounded token
sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (scheme, K = d_in, M = d_out, rank, alpha, tokens, group)
    "cfg2": ("fp8", 3072, 12288, 32, 32.0, 8192, 0),
    "cfg1": ("int4", 3072, 3072, 16, 16.0, 4096, 64),
    # the MLP up-projection (3072 -> 12288) of a double-stream block, int4 block 64, rank 16, on the
    # block's 4096 image + 512 text tokens
    "cfg3up": ("int4", 3072, 12288, 16, 16.0, 4608, 64),
}
METRIC = "LoRA-linear fwd+bwd TFLOP/s"
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the dominant kernel, from
# an ncu capture of the two frozen-GEMM launches of one step (summarised under profiles/): forward 392.7 MB, backward
# 830.0 MB, averaged like `achieved` is over the two launches of a step.
NCU_TRAFFIC_BYTES = {"cfg2": (392.67e6 + 829.97e6) / 2}


def step_flops(n, k, m, r):
    return 4 * n * k * m + 6 * n * r * (k + m)


def main_gemm_flops(n, k, m, r):
    """Algorithmic FLOPs of the two launches of the dominant kernel per step: the frozen GEMM of
    the forward (2NKM) with the fused LoRA up-projection (2NrM), and of the backward (2NKM) with
    the fused dH.A^T (2NrK)."""
    return 4 * n * k * m + 2 * n * r * (k + m)


# ---------------------------------------------------------------------------------------------
# CPU restatement of the reference's op sequence (the `cpu_baseline` / `--impl reference` leg)
# ---------------------------------------------------------------------------------------------
_CPU_WEIGHTS: dict = {}


def cpu_reference_rate(workload: str, sample_tokens: int, reps: int, seed: int = 5, threads: int = 0):
    """Times fwd+bwd of the reference's sequence in numpy f32 on `threads` BLAS threads (0 = all host
    cores; 1 = what the reference's ndarray backend resolves to, matrixmultiply without threading).
    Returns (tflops, seconds_per_step, threads used)."""
    import numpy as np

    from oracle import lq_oracle as O

    scheme, k, m, r, alpha, _, group = WORKLOADS[workload]
    rng = np.random.default_rng(seed)
    if (workload, seed) not in _CPU_WEIGHTS:  # quantizing 38 M weights in numpy takes longer than the timed steps
        w = (rng.standard_normal((m, k), dtype=np.float32) * np.float32(0.02))
        _CPU_WEIGHTS[(workload, seed)] = O.fp8_quantize(w, per_channel=True) if scheme == "fp8" else O.quantize(w, group, 4)
        del w
    q0, q1 = _CPU_WEIGHTS[(workload, seed)]
    dequant = (lambda: O.fp8_dequant(q0, q1)) if scheme == "fp8" else (lambda: O.dequantize(q0, q1, group))
    rng = np.random.default_rng(seed + 1)
    n = sample_tokens
    x = rng.standard_normal((n, k), dtype=np.float32)
    dy = rng.standard_normal((n, m), dtype=np.float32)
    a = rng.standard_normal((k, r), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((r, m), dtype=np.float32) * np.float32(0.01)
    s = alpha / r

    def one_step():
        y, h = O.lora_linear_fwd(x, dequant(), a, b, s)       # dequantize -> f32 [M,K] every pass
        dx, da, db = O.lora_linear_bwd(dy, x, dequant(), a, b, s)  # ... and again in the backward
        return float(y[0, 0]) + float(dx[0, 0]) + float(da[0, 0]) + float(db[0, 0])

    # torchrun exports OMP_NUM_THREADS=1; the baseline is defined on all host cores, so size the
    # BLAS pool explicitly and report the thread count actually used
    cores = threads if threads > 0 else len(os.sched_getaffinity(0))
    try:
        from threadpoolctl import threadpool_limits
        limiter = threadpool_limits(limits=cores)
    except Exception:
        limiter = None
        if threads == 1:
            raise
    try:
        one_step()
        t0 = time.perf_counter()
        for _ in range(reps):
            one_step()
        dt = (time.perf_counter() - t0) / reps
    finally:
        if limiter is not None:
            limiter.restore_original_limits()
    return step_flops(n, k, m, r) / dt / 1e12, dt, cores


def run_reference(args):
    """`--impl reference`: the reference's op sequence on the host cores (numpy port of the oracle), on
    the bench's own workload at its full token count, all host threads; beside it the single-threaded
    rate (what burn-ndarray's matrixmultiply resolves to) and the config-1 figures."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = args.workload
    scheme, k, m, r, alpha, tokens, group = WORKLOADS[wl]
    reps = max(1, min(args.steps, 3))
    # warm-up counted inside cpu_reference_rate (one untimed step); extra warm-ups are pointless on CPU
    tf, dt, cores = cpu_reference_rate(wl, tokens, reps)
    tf1, dt1, _ = cpu_reference_rate(wl, min(tokens, 256), 1, threads=1)
    c1 = WORKLOADS["cfg1"]
    c1_all, c1_dt, _ = cpu_reference_rate("cfg1", c1[5], 2)
    c1_one, c1_dt1, _ = cpu_reference_rate("cfg1", min(c1[5], 512), 1, threads=1)
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": reps, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "scheme": scheme, "d_in": k, "d_out": m, "rank": r, "alpha": alpha,
                   "tokens_per_gpu": tokens, "parallelism": "host cores"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"fwd+bwd on all {tokens} tokens, {reps} reps, numpy f32 (BLAS threads = host cores)"},
        "cpu_single_thread": {"value": tf1, "unit": "TFLOP/s", "cores": 1, "ms_per_step": dt1 * 1e3,
                              "sample": f"fwd+bwd on {min(tokens, 256)} of {tokens} tokens, 1 rep, 1 BLAS thread"},
        "cpu_cfg1": {"all_cores": {"value": c1_all, "unit": "TFLOP/s", "cores": cores, "ms_per_step": c1_dt * 1e3,
                                   "sample": f"int4 3072x3072 rank 16, all {c1[5]} tokens, f32"},
                     "single_thread": {"value": c1_one, "unit": "TFLOP/s", "cores": 1, "ms_per_step": c1_dt1 * 1e3,
                                       "sample": f"int4 3072x3072 rank 16, {min(c1[5], 512)} of {c1[5]} tokens, f32"}},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text()) if p.exists() else {}


def measure_fp8_peak(dev):
    """No fp8 peak is in MEASURED_PEAKS.json: measure one here the way the bf16 one was measured
    (library GEMM, 8192^3, best of 13 single launches, CUDA events) and use it as the denominator
    of the native-fp8 fractions."""
    import torch

    a8 = torch.randn(8192, 8192, device=dev).to(torch.float8_e4m3fn)
    b8 = torch.randn(8192, 8192, device=dev).to(torch.float8_e4m3fn).t()
    one = torch.ones((), device=dev)
    best = 1e9
    for _ in range(13):
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        q1.record()
        torch.cuda.synchronize()
        best = min(best, q0.elapsed_time(q1))
    return 2 * 8192 ** 3 / (best * 1e-3) / 1e12


def measure_linear_quick(dev, wl: str, steps: int, rank_seed: int = 0):
    """One single-linear workload (fwd + bwd, inputs resident, CUDA graph replay): median of five
    regions of `steps` replays, per-kernel-class times from an eager pass, frozen-GEMM fraction of
    the measured bf16 burst peak."""
    import torch

    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    lib = L.lib()
    scheme, k, m, r, alpha, n, group = WORKLOADS[wl]
    s_ = alpha / r
    g = torch.Generator(device=dev).manual_seed(5)
    w = torch.randn((m, k), generator=g, device=dev) * 0.02
    wq = lb.fp8_quantize(w, per_channel=True) if scheme == "fp8" else lb.quantize_linear_weight(w, 4, group)
    del w
    g = torch.Generator(device=dev).manual_seed(7 + rank_seed)
    a = torch.randn((k, r), generator=g, device=dev) / (k ** 0.5)
    b = torch.randn((r, m), generator=g, device=dev) * 0.01
    # inputs and outputs of one step must exceed the 126 MB L2, else consecutive steps would be served
    # from it: smaller workloads rotate through several input sets (a "step" call runs one of each)
    footprint = 4 * n * (k + m)
    n_sets = max(1, -(-int(1.6 * 126e6) // footprint))
    xs = [torch.randn((n, k), generator=g, device=dev).to(torch.bfloat16) for _ in range(n_sets)]
    dys = [torch.randn((n, m), generator=g, device=dev).to(torch.bfloat16) for _ in range(n_sets)]
    da, db = torch.zeros((k, r), device=dev), torch.zeros((r, m), device=dev)
    mir = Q.lora_mirror(a, b)

    def step():
        for x, dy in zip(xs, dys):
            y, h = Q.linear_fwd_raw(wq, x, a, b, s_, mirror=mir)
            Q.linear_bwd_raw(wq, dy, x, h, a, b, s_, da_out=da, db_out=db, mirror=mir)

    for _ in range(3):
        step()
    lb.check_device_status(dev)
    lib.lq_profile_enable(1)
    lib.lq_profile_collect(None, None, 0)
    for _ in range(steps):
        step()
    nk = lib.lq_profile_kinds()
    msk, cnt = (C.c_double * nk)(), (C.c_uint64 * nk)()
    lib.lq_profile_collect(msk, cnt, nk)
    lib.lq_profile_enable(0)
    kinds = {lib.lq_profile_kind_name(i).decode(): (msk[i], int(cnt[i])) for i in range(nk)}
    gph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        step()
        with torch.cuda.graph(gph, stream=side):
            step()
    torch.cuda.current_stream(dev).wait_stream(side)
    for _ in range(3):
        gph.replay()
    regions = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            gph.replay()
        e1.record()
        torch.cuda.synchronize()
        regions.append(e0.elapsed_time(e1) / (steps * n_sets))
    lb.check_device_status(dev)
    ms = statistics.median(regions)
    peaks = load_peaks()
    peak = peaks.get("bf16_tflops", 1590.0)
    gm_ms, gm_n = kinds.get("gemm_main", (0.0, 0))
    gemm_tf = (main_gemm_flops(n, k, m, r) / 2) / (gm_ms / max(gm_n, 1) * 1e-3) / 1e12 if gm_n else None
    fl = step_flops(n, k, m, r)
    return {
        "workload": wl, "scheme": scheme, "d_in": k, "d_out": m, "rank": r, "tokens": n, "group": group,
        "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "regions_ms": regions,
        "frac_of_bf16_burst": fl / (ms * 1e-3) / 1e12 / peak,
        "gemm_tflops": gemm_tf, "gemm_frac": gemm_tf / peak if gemm_tf else None, "peak": peak,
        "by_kernel_ms_per_step": {kk: v[0] / (steps * n_sets) for kk, v in kinds.items() if v[1]},
        "l2": f"{n_sets} rotating input/output sets of {footprint / 1e6:.0f} MB = {n_sets * footprint / 1e6:.0f} MB > 126 MB L2",
    }

class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons for one GPU while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def median_sm_mhz(self, t0, t1):
        """Median SM clock of the samples taken between two wall-clock times (None without samples)."""
        vals = []
        for (t, r) in list(self.rows):
            if t0 <= t <= t1:
                try:
                    vals.append(float(r.split(",")[0]))
                except ValueError:
                    pass
        return statistics.median(vals) if vals else None

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for (t, r) in self.rows if t0 <= t <= t1 + 0.2] or [r for (_, r) in self.rows[-3:]]
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            f = [v.strip() for v in r.split(",")]
            try:
                sm.append(float(f[0]))
                smax.append(float(f[1]))
            except (ValueError, IndexError):
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_ours(args):
    import torch
    import torch.distributed as dist

    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    wl = args.workload
    scheme, k, m, r, alpha, n, group = WORKLOADS[wl]
    s = alpha / r
    lib = L.lib()

    # ---- synthetic, seeded inputs; weights identical on every rank, data seeded per rank ----
    g = torch.Generator(device=dev).manual_seed(5)
    w = torch.randn((m, k), generator=g, device=dev, dtype=torch.float32) * 0.02
    wq = lb.fp8_quantize(w, per_channel=True) if scheme == "fp8" else lb.quantize_linear_weight(w, 4, group)
    del w
    g = torch.Generator(device=dev).manual_seed(7)
    a = torch.randn((k, r), generator=g, device=dev) / (k ** 0.5)
    b = torch.randn((r, m), generator=g, device=dev) * 0.01
    gd = torch.Generator(device="cpu").manual_seed(100 + rank)
    x_host = torch.randn((n, k), generator=gd, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    dy_host = torch.randn((n, m), generator=gd, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    dy = dy_host.to(dev)
    bucket = torch.zeros(k * r + r * m, device=dev, dtype=torch.float32)  # flat LoRA-gradient bucket
    da = bucket[: k * r].view(k, r)
    db = bucket[k * r:].view(r, m)
    y_host = torch.empty((n, m), dtype=torch.bfloat16).pin_memory()
    dx_host = torch.empty((n, k), dtype=torch.bfloat16).pin_memory()
    g_host = torch.empty_like(bucket, device="cpu").pin_memory()

    fp8c = args.compute == "fp8"
    if fp8c:
        if scheme != "fp8":
            raise SystemExit("--compute fp8 needs a scaled-fp8 workload (cfg2)")
        wq.prepare_fp8_backward()

    # the factors' bf16 operand mirror: a trainer refreshes it once after each optimizer update
    # (`lq_lora_mirror_update`), outside forward and backward; A and B do not change here
    mirror = Q.lora_mirror(a, b)

    def step(xd, dyd):
        y, h = Q.linear_fwd_raw(wq, xd, a, b, s, fp8_compute=fp8c, mirror=mirror)
        dx, _, _ = Q.linear_bwd_raw(wq, dyd, xd, h, a, b, s, da_out=da, db_out=db, fp8_compute=fp8c, mirror=mirror)
        if world > 1:
            dist.all_reduce(bucket)  # the only exchange of the data-parallel path
        return y, dx

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step(x, dy)
    lb.check_device_status(dev)

    sampler = ClockSampler(local) if rank == 0 else None
    t_wall0 = time.time()

    # ---- value: inputs resident in HBM; per-kernel-class times from the library's event pairs ----
    lib.lq_profile_enable(1)
    lib.lq_profile_collect(None, None, 0)
    launches0 = lib.lq_kernel_launch_count()
    eager_ms = timed(lambda: step(x, dy), args.steps)
    launches = lib.lq_kernel_launch_count() - launches0
    nk = lib.lq_profile_kinds()
    ms_kind = (C.c_double * nk)()
    cnt_kind = (C.c_uint64 * nk)()
    lib.lq_profile_collect(ms_kind, cnt_kind, nk)
    lib.lq_profile_enable(0)
    lb.check_device_status(dev)
    kinds = {lib.lq_profile_kind_name(i).decode(): (ms_kind[i], int(cnt_kind[i])) for i in range(nk)}

    # `value` is timed on a CUDA graph of the step (the library's launches are capturable: fixed
    # workspace, tensor maps passed by value), replayed `steps` times, so that launch latency between
    # the ~18 kernels of a step is not what is measured; the NCCL all-reduce stays outside the graph.
    def capture(fn):
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            fn()  # sizes this stream's workspace before capture
            with torch.cuda.graph(g, stream=side):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        return g

    def local_step(f8):
        y_, h_ = Q.linear_fwd_raw(wq, x, a, b, s, fp8_compute=f8, mirror=mirror)
        Q.linear_bwd_raw(wq, dy, x, h_, a, b, s, da_out=da, db_out=db, fp8_compute=f8, mirror=mirror)

    use_graph = not args.no_graph
    if use_graph:
        graph = capture(lambda: local_step(fp8c))

        def graph_step():
            graph.replay()
            if world > 1:
                dist.all_reduce(bucket)

        for _ in range(3):
            graph_step()
    else:
        graph_step = lambda: step(x, dy)
    # `value`: the median of five timed regions of K steps each (every region bracketed by a barrier
    # and a device synchronisation, timed with CUDA events, max over ranks)
    regions_ms = [timed(graph_step, args.steps) for _ in range(5)]
    total_ms = statistics.median(regions_ms)
    lb.check_device_status(dev)


    # Scaled-fp8 workloads: also time the same step with native e4m3 MMA (LQ_BF16_W8A8), reported
    # beside the headline under "native_fp8" (the headline itself stays the bf16-compute path).
    native_fp8 = None
    if scheme == "fp8" and not fp8c:
        wq.prepare_fp8_backward()

        def step8():
            y8, h8 = Q.linear_fwd_raw(wq, x, a, b, s, fp8_compute=True)
            Q.linear_bwd_raw(wq, dy, x, h8, a, b, s, da_out=da, db_out=db, fp8_compute=True)
            if world > 1:
                dist.all_reduce(bucket)

        for _ in range(3):
            step8()
        lib.lq_profile_enable(1)
        lib.lq_profile_collect(None, None, 0)
        timed(step8, args.steps)  # eager pass: per-kernel-class times
        ms_k8 = (C.c_double * nk)()
        cnt_k8 = (C.c_uint64 * nk)()
        lib.lq_profile_collect(ms_k8, cnt_k8, nk)
        lib.lq_profile_enable(0)
        lb.check_device_status(dev)
        k8 = {lib.lq_profile_kind_name(i).decode(): (ms_k8[i], int(cnt_k8[i])) for i in range(nk)}
        if use_graph:
            graph8 = capture(lambda: local_step(True))

            def graph_step8():
                graph8.replay()
                if world > 1:
                    dist.all_reduce(bucket)

            for _ in range(3):
                graph_step8()
            ms8 = timed(graph_step8, args.steps)
        else:
            ms8 = timed(step8, args.steps)
        g8_ms, g8_n = k8.get("gemm_main", (0.0, 0))
        native_fp8 = {
            "value": step_flops(n, k, m, r) * world / (ms8 / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s",
            "ms_per_step": ms8 / args.steps, "dtype": "fp8 e4m3 x e4m3, f32 accumulate (bf16 in/out)",
            "gemm_tflops": (main_gemm_flops(n, k, m, r) / 2) / (g8_ms / max(g8_n, 1) * 1e-3) / 1e12 if g8_n else None,
            "by_kernel_ms_per_step": {kk: v[0] / args.steps for kk, v in k8.items() if v[1]},
            "tolerance": "Y, dX within 5e-2 of peak vs the f32 oracle (tests/test_gpu_w8a8.py)",
        }

    # The reference's dead-graph guards (crates/loractl-bench/src/lib.rs:35-104): twice the steps must
    # take about twice as long (ratio in [1.7, 2.3]) and the outputs must be finite and non-zero.
    ms_2x = timed(graph_step, 2 * args.steps)
    y_chk, dx_chk = step(x, dy)
    plausible = bool(torch.isfinite(y_chk).all() and torch.isfinite(dx_chk).all() and torch.isfinite(bucket).all()
                     and float(y_chk.float().abs().max()) > 0 and float(bucket.abs().max()) > 0)
    sanity = {"x2_ratio": ms_2x / total_ms, "ok": 1.7 <= ms_2x / total_ms <= 2.3, "plausible": plausible}

    # ---- e2e: host buffers in, results out, through the same public calls ----
    # Every step copies its inputs from pinned host memory and its results (Y, dX, dA, dB) back.
    # Copies run on their own streams, double-buffered, so step i's compute overlaps step i+1's
    # upload and step i-1's download (PCIe is full duplex); all of it is inside the timed region.
    s_h2d, s_d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_cmp = torch.cuda.current_stream(dev)
    xbuf = [torch.empty_like(x) for _ in range(2)]
    dybuf = [torch.empty_like(dy) for _ in range(2)]
    buckets = [bucket, torch.zeros_like(bucket)]
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]
    counter = [0]

    def e2e_step():
        i = counter[0] & 1
        counter[0] += 1
        with torch.cuda.stream(s_h2d):
            s_h2d.wait_event(ev_cmp[i])  # the compute that last read this buffer pair is done
            xbuf[i].copy_(x_host, non_blocking=True)
            dybuf[i].copy_(dy_host, non_blocking=True)
            ev_up[i].record(s_h2d)
        s_cmp.wait_event(ev_up[i])
        s_cmp.wait_event(ev_down[i])  # this slot's gradient bucket has been downloaded
        bk = buckets[i]
        y, h = Q.linear_fwd_raw(wq, xbuf[i], a, b, s, fp8_compute=fp8c, mirror=mirror)
        dx, _, _ = Q.linear_bwd_raw(wq, dybuf[i], xbuf[i], h, a, b, s, da_out=bk[: k * r].view(k, r),
                                    db_out=bk[k * r:].view(r, m), fp8_compute=fp8c, mirror=mirror)
        if world > 1:
            dist.all_reduce(bk)
        ev_cmp[i].record(s_cmp)
        with torch.cuda.stream(s_d2h):
            s_d2h.wait_event(ev_cmp[i])
            y_host.copy_(y, non_blocking=True)
            dx_host.copy_(dx, non_blocking=True)
            g_host.copy_(bk, non_blocking=True)
            y.record_stream(s_d2h)
            dx.record_stream(s_d2h)
            ev_down[i].record(s_d2h)

    def e2e_loop(steps):
        for _ in range(steps):
            e2e_step()
        s_cmp.wait_stream(s_d2h)  # the timed region ends when the last result is on the host
        s_cmp.wait_stream(s_h2d)

    e2e_steps = max(4, min(args.steps, 20))
    e2e_loop(4)
    sync_all()
    e2e_ms = timed(lambda: e2e_loop(e2e_steps), 1)
    t_wall1 = time.time()

    # ---- further keys of the default line: the other workloads of the path, measured in the same run ----
    extras = {}
    sustained = None
    if not args.no_extras and wl == "cfg2" and not fp8c:
        # config 1 (int4 block 64, 3072 x 3072, rank 16, 4096 tokens) on this rank's GPU
        extras["int4_cfg1"] = measure_linear_quick(dev, "cfg1", max(args.steps, 10), rank)
        extras["int4_cfg3up"] = measure_linear_quick(dev, "cfg3up", max(args.steps, 10), rank)
        if world == 1:
            # the packed-weight stream at <= 64 tokens (one GPU; the sites do not shard)
            sres, hbm_peak = measure_stream(dev, 10)
            extras["stream"] = {
                "unit": "GB/s of packed weight bytes per whole site (weight kernel + finalize), CUDA graph replay",
                "hbm_peak_gbs": hbm_peak,
                "sites": {key: {"stream_bytes_per_site": v["stream_bytes_per_site"], "distinct_sites": v["sites"],
                                "by_tokens": {t: {"site_us": d["site_us"], "gbs": d["site_stream_gbs"],
                                                  "frac": d["frac_of_hbm"], "grouped4_site_us": d["grouped4_site_us"],
                                                  "grouped4_frac": d["grouped4_frac_of_hbm"],
                                                  "bwd_site_us": d["bwd_site_us"], "bwd_frac": d["bwd_frac_of_hbm"]}
                                              for t, d in v["by_tokens"].items()}}
                          for key, v in sres.items()},
            }
        # `sustained`: one region of at least two seconds, the regime a training loop runs in (the SM clock
        # settles well below its burst value under the power cap); compared with the sustained cuBLAS peak.
        # It runs after every burst measurement so that none of them inherits a hot, power-capped chip.
        sus_steps = max(args.steps, int(2000.0 / max(total_ms / args.steps, 1e-3)) + 1)
        t_sus0 = time.time()
        sus_ms = timed(graph_step, sus_steps)
        t_sus1 = time.time()
        sus_peak = load_peaks().get("bf16_tflops_sustained")
        sus_tf = step_flops(n, k, m, r) / (sus_ms / sus_steps * 1e-3) / 1e12  # per GPU
        sustained = {"value": sus_tf * world, "unit": "TFLOP/s", "seconds": sus_ms * 1e-3, "steps": sus_steps,
                     "peak": sus_peak, "frac": sus_tf / sus_peak if sus_peak else None,
                     "sm_mhz_median": sampler.median_sm_mhz(t_sus0, t_sus1) if sampler else None}
        # config 5: the 24-block stack, global batch 8 sharded over the ranks, rank 32, recompute on
        # resident bf16 copies of the frozen weights (16 GB of the 180) and one gradient all-reduce after the
        # sweep: the fastest of the combinations measured on 8 GPUs
        extras["model_step"] = measure_train_step(dev, world, rank, 24, 8, 32, steps=3, warmup=2,
                                                  weight_copies="resident", reduce_every=24, two_streams=True)
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    flops = step_flops(n, k, m, r)
    ms_per_step = total_ms / args.steps
    value = flops * world / (ms_per_step * 1e-3) / 1e12
    e2e_value = flops * world / (e2e_ms / e2e_steps * 1e-3) / 1e12
    h2d = x_host.numel() * 2 + dy_host.numel() * 2
    d2h = y_host.numel() * 2 + dx_host.numel() * 2 + g_host.numel() * 4

    if rank == 0:
        peaks = {}
        p = ROOT / "MEASURED_PEAKS.json"
        if p.exists():
            peaks = json.loads(p.read_text())
        timed_s = total_ms * 1e-3
        if peaks:
            peak_kind = "sustained" if timed_s > 0.5 else "burst"
            peak = peaks["bf16_tflops_sustained"] if peak_kind == "sustained" else peaks["bf16_tflops"]
            peak_src = f"measured ({peak_kind} cuBLAS bf16, MEASURED_PEAKS.json)"
        else:
            peak, peak_src = 1590.0, "fallback (earlier measurement on this pool)"
        fp8_peak = measure_fp8_peak(dev) if scheme == "fp8" else None
        if fp8c:
            peak = fp8_peak
            peak_src = "measured in this run (burst, torch._scaled_mm e4m3 8192^3, best of 13)"
        gm_ms, gm_n = kinds.get("gemm_main", (0.0, 0))
        achieved = (main_gemm_flops(n, k, m, r) / 2) / (gm_ms / max(gm_n, 1) * 1e-3) / 1e12 if gm_n else None
        roofline = {
            "bound": "tensor", "kernel": "umma_gemm2_kernel (frozen GEMM on CTA pairs + fused LoRA K extension)",
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None,
            "peak_source": peak_src, "traffic": None if fp8c else NCU_TRAFFIC_BYTES.get(wl),
            "traffic_unit": "bytes per launch (ncu, full-size launch)",
            "algorithmic_bytes_per_launch": 2 * n * k + 2 * m * k + 2 * n * m,
            "launches_timed": gm_n, "avg_launch_ms": gm_ms / max(gm_n, 1),
            "share_of_step": gm_ms / eager_ms if eager_ms else None,
            "eager_ms_per_step": eager_ms / args.steps,
            "by_kernel_ms_per_step": {kk: v[0] / args.steps for kk, v in kinds.items() if v[1]},
        }
        cpu_tf, cpu_dt, cores = cpu_reference_rate(wl, min(n, 1024), 3)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8 e4m3 x e4m3, f32 accumulate (bf16 in/out)" if fp8c else "bf16",
            "data": "synthetic",
            "config": {"workload": wl, "scheme": scheme, "d_in": k, "d_out": m, "rank": r, "alpha": alpha,
                       "tokens_per_gpu": n, "parallelism": f"dp{world}",
                       "l2": f"inputs larger than L2 (X+dY+Y+dX = {4 * n * (k + m) / 1e6:.0f} MB per step vs 126 MB)",
                       "launch": "eager" if args.no_graph else "CUDA graph of the step, replayed",
                       "lora_mirror": "bf16 operand mirror of A, B built once before the timed region"},
            "roofline": roofline,
            "cpu_baseline": {"value": cpu_tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                             "sample": f"fwd+bwd on {min(n, 1024)} of {n} tokens, 3 reps, numpy f32"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "regions_ms_per_step": [v / args.steps for v in regions_ms],
            "sustained": sustained,
            "sanity": sanity,
            "native_fp8": native_fp8,
            "model": {"step_flops": flops, "main_gemm_flops": main_gemm_flops(n, k, m, r),
                      "packed_stream_bytes": (k * m + 4 * m) if scheme == "fp8" else (k * m // 2 + 4 * k * m // group)},
            "clocks": clocks,
        }
        if native_fp8 is not None and fp8_peak:
            native_fp8["peak"] = fp8_peak
            native_fp8["peak_source"] = "measured in this run (burst, torch._scaled_mm e4m3 8192^3, best of 13)"
            native_fp8["frac"] = native_fp8["value"] / world / fp8_peak
            if native_fp8.get("gemm_tflops"):
                native_fp8["gemm_frac"] = native_fp8["gemm_tflops"] / fp8_peak
        line.update(extras)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_stream(args):
    """The packed-weight-stream regime (`--regime stream`): int4 3072 x 3072 (the single-linear headline
    site, block 64, rank 16) forward at N in {1, 8, 16, 64} tokens.  40 distinct sites (212 MB
    of packed weights, more than the 126 MB L2; also 10 int4 and 10 scaled-fp8 12288 x 3072 sites,
    the latter the headline workload's weight at 1, 8 and 16 tokens) run back to back inside one CUDA graph, so every
    launch streams its weight from HBM and launch latency is not the thing measured.  Reports the
    algorithmic packed-stream bytes (K*M/2 + 4*K*M/64 = 5,308,416 B per site) per second, for
    the whole site (weight kernel with H = X.A folded in at N <= 16, finalize) and for the weight
    kernel alone (stream_small_fwd_kernel, register dequant + mma.sync, at N <= 16;
    fused_small_fwd_kernel, shared-memory dequant + tcgen05, above)."""
    import torch

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    tokens = tuple(int(t) for t in args.stream_tokens.split(","))
    all_results, hbm = measure_stream(dev, max(args.steps, 10), tokens, args.stream_only)
    r = 16
    head = all_results.get("3072x12288-fp8") or next(iter(all_results.values()))
    best = head["by_tokens"].get("8") or next(iter(head["by_tokens"].values()))
    line = {
        "metric": "packed-weight stream GB/s (cfg2 weight: scaled fp8 3072 -> 12288, forward, 8 tokens)",
        "value": best["site_stream_gbs"], "unit": "GB/s", "n_gpus": 1, "steps": max(args.steps, 10), "warmup": 3,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg2-stream", "sites": head["sites"], "d_in": 3072, "d_out": 12288, "rank": r,
                   "l2": "10 distinct weights = 378 MB > 126 MB L2", "launch": "CUDA graph replay"},
        # the site is two launches (weight kernel with H = X.A folded in, finalize); per-kernel event times of
        # launches this short include the launch gap, so the whole-site rate is the one reported against HBM
        "roofline": {"bound": "hbm", "kernel": "stream_small_fp8_kernel + fused_finalize_kernel (whole site)",
                     "achieved": best["site_stream_gbs"], "peak": hbm, "unit": "GB/s", "frac": best["site_stream_gbs"] / hbm,
                     "traffic": None, "algorithmic_bytes_per_launch": head["stream_bytes_per_site"]},
        "by_site": all_results,
    }
    print(json.dumps(line))


def measure_stream(dev, reps: int, token_counts=(1, 8, 16, 64), only=None):
    """The three site shapes of the stream regime at the given token counts; returns
    ({site: {...}}, hbm peak GB/s).  Every rate carries its fraction of the measured HBM copy rate."""
    import torch

    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import quant as Q

    lib = L.lib()
    peaks = {}
    if (ROOT / "MEASURED_PEAKS.json").exists():
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    hbm = peaks.get("hbm_gbs", 6650.0)
    r, s = 16, 1.0
    g = torch.Generator(device=dev).manual_seed(5)
    all_results = {}
    # (d_out, d_in, sites): the cfg1 workload's 3072 x 3072 site, and the 3072 -> 12288 MLP up-projection
    # of configs 3/5 held as int4 (21.2 MB of packed weight per site)
    for m, k, sites, scheme in ((3072, 3072, 40, "int4"), (12288, 3072, 10, "int4"), (12288, 3072, 10, "fp8")):
        if only and only != (f"{k}x{m}" if scheme == "int4" else f"{k}x{m}-fp8"):
            continue  # `--stream-only`: one site shape, for a short profiler capture
        weights = []
        for _ in range(sites):
            w = torch.randn((m, k), generator=g, device=dev) * 0.02
            weights.append(lb.quantize_linear_weight(w, 4, 64) if scheme == "int4" else lb.fp8_quantize(w, True))
        del w
        a = torch.randn((k, r), generator=g, device=dev) / (k ** 0.5)
        b = torch.randn((r, m), generator=g, device=dev) * 0.01
        stream_bytes = (k * m // 2 + 4 * k * m // 64) if scheme == "int4" else (k * m + 4 * m)
        results = {}
        for n in (token_counts if scheme == "int4" else tuple(t for t in token_counts if t <= 16)):
            x = torch.randn((n, k), generator=g, device=dev).to(torch.bfloat16)

            def chain():
                y = None
                for wq in weights:
                    y, _ = Q.linear_fwd_raw(wq, x, a, b, s, want_h=False)
                return y

            for _ in range(3):
                chain()
            lb.check_device_status(dev)
            # per-kernel-class time, eager launches (event pairs around every launch)
            lib.lq_profile_enable(1)
            lib.lq_profile_collect(None, None, 0)
            for _ in range(3):
                chain()
            nk = lib.lq_profile_kinds()
            ms_kind, cnt_kind = (C.c_double * nk)(), (C.c_uint64 * nk)()
            lib.lq_profile_collect(ms_kind, cnt_kind, nk)
            lib.lq_profile_enable(0)
            kinds = {lib.lq_profile_kind_name(i).decode(): (ms_kind[i], int(cnt_kind[i])) for i in range(nk)}
            fused_ms = kinds["gemm_main"][0] / max(kinds["gemm_main"][1], 1)
            # whole-site time, graph replay; int4 sites also as groups of four sites that share X
            # (one launch pair per group: `lq_linear_fwd_grouped`)
            def chain_grouped():
                y = None
                for i0 in range(0, len(weights), 4):
                    outs = Q.linear_fwd_grouped_raw([(wq, a, b, s) for wq in weights[i0:i0 + 4]], x, want_h=False)
                    y = outs[-1][0]
                return y

            def replay_time(fn):
                for _ in range(2):
                    fn()
                graph = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    fn()
                    with torch.cuda.graph(graph, stream=side):
                        fn()
                torch.cuda.current_stream(dev).wait_stream(side)
                for _ in range(3):
                    graph.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize()
                lb.check_device_status(dev)
                return e0.elapsed_time(e1) / (reps * sites)

            site_ms = replay_time(chain)
            grouped_ms = replay_time(chain_grouped) if (scheme == "int4" and n <= 16) else None
            # the backward of the same sites (dX through the packed stream, dA, dB): int4, <= 16 tokens
            bwd_ms = None
            if scheme == "int4" and n <= 16:
                dy = torch.randn((n, m), generator=g, device=dev).to(torch.bfloat16)
                _, h_keep = Q.linear_fwd_raw(weights[0], x, a, b, s)

                def chain_bwd():
                    out = None
                    for wq in weights:
                        out = Q.linear_bwd_raw(wq, dy, x, h_keep, a, b, s)
                    return out

                bwd_ms = replay_time(chain_bwd)
            results[str(n)] = {
                "site_us": site_ms * 1e3, "site_stream_gbs": stream_bytes / (site_ms * 1e-3) / 1e9,
                "frac_of_hbm": stream_bytes / (site_ms * 1e-3) / 1e9 / hbm,
                "grouped4_site_us": grouped_ms * 1e3 if grouped_ms else None,
                "grouped4_frac_of_hbm": stream_bytes / (grouped_ms * 1e-3) / 1e9 / hbm if grouped_ms else None,
                "bwd_site_us": bwd_ms * 1e3 if bwd_ms else None,
                "bwd_frac_of_hbm": stream_bytes / (bwd_ms * 1e-3) / 1e9 / hbm if bwd_ms else None,
                "fused_kernel_us": fused_ms * 1e3,
                "fused_kernel_stream_gbs": stream_bytes / (fused_ms * 1e-3) / 1e9,
                "by_kernel_us": {kk: v[0] / max(v[1], 1) * 1e3 for kk, v in kinds.items() if v[1]},
            }
        key = f"{k}x{m}" if scheme == "int4" else f"{k}x{m}-fp8"
        all_results[key] = {"stream_bytes_per_site": stream_bytes, "sites": sites, "scheme": scheme, "by_tokens": results}
        del weights
    return all_results, hbm


def run_load(args):
    """`--regime load`: streaming quantize-at-load of one double-stream block's linears (both
    streams: adaLN modulation 3072 -> 18432, joint qkv 3072 -> 9216, out 3072 -> 3072, MLP up
    3072 -> 12288 and down 12288 -> 3072) from a synthetic scaled-fp8 safetensors checkpoint with
    per-output-channel weight_scale sidecars (340 MB) into packed int4 block-64 handles.  The file is
    written to a temporary directory first and is in the page cache when the timed loads run.
    `value` = checkpoint bytes per second through `loader.load_quant_module` (host copy, upload,
    fused requantize kernel, all overlapped); the roofline entry is the requantize kernel alone
    against HBM (1 byte read, 0.5 + 4/64 bytes written per element)."""
    import tempfile

    import numpy as np
    import torch

    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import loader as LD

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    lib = L.lib()
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    hbm = peaks.get("hbm_gbs", 6650.0)
    h, mlp = 3072, 12288
    dims = {"mod": (6 * h, h), "qkv": (3 * h, h), "out": (h, h), "up": (mlp, h), "down": (h, mlp)}
    g = torch.Generator(device=dev).manual_seed(5)
    tensors = {}
    elems = 0
    for stream in ("img", "txt"):
        for name, (m, k) in dims.items():
            w = torch.randn((m, k), generator=g, device=dev) * 0.02
            f8 = lb.fp8_quantize(w, True)
            wb, sc = f8.unpack()
            key = f"blocks.0.{stream}.{name}.weight"
            tensors[key] = ("F8_E4M3", (m, k), wb.cpu().numpy().tobytes())
            tensors[key + "_scale"] = ("F32", (m,), sc.cpu().numpy().astype("<f4").tobytes())
            elems += m * k
            del w, f8, wb, sc
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "block_fp8.safetensors")
        LD.write_safetensors(path, tensors, {"format": "pt"})
        file_bytes = os.path.getsize(path)
        del tensors
        for _ in range(max(2, min(args.warmup, 3))):
            handles, _, rep = LD.load_quant_module(path, dev, bits=4, block=64)
            del handles
        reps = max(3, min(args.steps, 10))
        launches0 = lib.lq_kernel_launch_count()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            handles, _, rep = LD.load_quant_module(path, dev, bits=4, block=64)
            del handles  # the timed region includes freeing the previous load's 191 MB of handles
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / reps
        launches = lib.lq_kernel_launch_count() - launches0
        # the requantize kernel alone: event pairs around every launch, in a separate pass
        lib.lq_profile_enable(1)
        lib.lq_profile_collect(None, None, 0)
        for _ in range(reps):
            handles, _, rep = LD.load_quant_module(path, dev, bits=4, block=64)
            del handles
        torch.cuda.synchronize()
        nk = lib.lq_profile_kinds()
        ms_kind, cnt_kind = (C.c_double * nk)(), (C.c_uint64 * nk)()
        lib.lq_profile_collect(ms_kind, cnt_kind, nk)
        lib.lq_profile_enable(0)
        kinds = {lib.lq_profile_kind_name(i).decode(): (ms_kind[i], int(cnt_kind[i])) for i in range(nk)}
    q_ms, q_n = kinds["quantize"]
    kernel_bytes = elems * (1 + 0.5 + 4 / 64) * reps
    achieved = kernel_bytes / (q_ms * 1e-3) / 1e9
    # CPU restatement of the reference's route for one site: LUT decode x scale to f32 on the host,
    # then group absmax / round / clamp (numpy, one process)
    from oracle import lq_oracle as O

    rng = np.random.default_rng(5)
    wq_b, wq_s = O.fp8_quantize((rng.standard_normal((h, h), dtype=np.float32) * np.float32(0.02)), True)
    t1 = time.perf_counter()
    O.quantize(O.fp8_dequant(wq_b, wq_s), 64, 4)
    cpu_dt = time.perf_counter() - t1
    line = {
        "metric": "quantize-at-load GB/s (checkpoint bytes, scaled fp8 -> int4 block 64)", "value": file_bytes / dt / 1e9,
        "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": 2, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "dtype": "u8 -> u4 (f32 arithmetic)", "data": "synthetic",
        "config": {"workload": "block-fp8-load", "tensors": 10, "elements": elems, "file_bytes": file_bytes,
                   "packed_bytes": rep.packed_bytes, "source": "page cache"},
        "roofline": {"bound": "hbm", "kernel": "quantize16_kernel<Fp8Src>", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                     "frac": achieved / hbm, "traffic": None,
                     "algorithmic_bytes_per_launch": elems * (1 + 0.5 + 4 / 64) / 10, "launches_timed": q_n,
                     "avg_launch_ms": q_ms / max(q_n, 1)},
        "cpu_baseline": {"value": (h * h) / cpu_dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": "one 3072 x 3072 fp8 site: numpy LUT decode x scale, then quantize"},
        "gpu_launches": int(launches),
    }
    print(json.dumps(line))


def mmdit_step_flops(cfg, lora_rank: int, n_blocks: int, global_batch: int) -> int:
    """FLOP model of one training step of the double-stream stack (the counterpart of
    crates/loractl-core/src/bench.rs:274-311 for this block): linears + LoRA + joint attention,
    forward + recomputed forward + backward; the frozen weights get no gradient, so a linear's
    backward is dX only (1x its forward) plus the LoRA terms (2x); attention backward is 2x."""
    h, tokens = cfg.hidden, cfg.img_tokens + cfg.txt_tokens
    p_stream = 4 * h * h + 2 * h * cfg.mlp
    lin_fwd = 2 * tokens * p_stream + 2 * 2 * h * 6 * h  # both streams' projections + the two modulations
    lora_fwd = 2 * tokens * lora_rank * (2 * h + 4 * h + 2 * h + 2 * (h + cfg.mlp))
    att_fwd = 4 * tokens * tokens * h
    flops_block = 2 * (lin_fwd + lora_fwd + att_fwd) + (lin_fwd + 2 * lora_fwd + 2 * att_fwd)
    return flops_block * n_blocks * global_batch


def measure_train_step(dev, world: int, rank: int, n_blocks: int, batch: int, lora_rank: int, steps: int,
                       warmup: int, weight_copies: str = "none", graphs: bool = True, reduce_every: int = 1,
                       two_streams: bool = False):
    """Times `steps` training steps of the double-stream stack on this rank's shard of the global
    batch (max over ranks, CUDA events, barrier + synchronize on both sides).  Returns the result
    dict on every rank; the process group, if any, is the caller's."""
    import torch
    import torch.distributed as dist

    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200.harness import BlockConfig, BlockStack, Trainer

    cfg = BlockConfig()
    global_batch = max(batch, world)
    lo, hi = lb.dp.shard_range(global_batch, rank, world)
    b = hi - lo
    stack = BlockStack(n_blocks, cfg, lora_rank, float(lora_rank), dev, seed=5, weight_copies=weight_copies,
                       two_cuda_streams=two_streams)
    trainer = Trainer(stack, lr=1e-4, graphs=graphs, reduce_every=reduce_every)
    g = torch.Generator(device=dev).manual_seed(100 + rank)  # per-rank data, identical weights
    h = cfg.hidden
    x0 = torch.randn((b, cfg.img_tokens, h), generator=g, device=dev, dtype=torch.bfloat16)
    txt = torch.randn((b, cfg.txt_tokens, h), generator=g, device=dev, dtype=torch.bfloat16)
    cond = torch.randn((b, h), generator=g, device=dev, dtype=torch.bfloat16)
    noise = torch.randn(x0.shape, generator=g, device=dev, dtype=torch.bfloat16)
    t = torch.rand((b,), generator=g, device=dev) * 0.9 + 0.05

    def one():
        return trainer.step(x0, txt, cond, t, noise)

    losses = [one() for _ in range(max(warmup, 2))]
    lb.check_device_status(dev)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = L.lib().lq_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        losses.append(one())
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        tm = torch.tensor([ms], device=dev)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm.item())
    launches = L.lib().lq_kernel_launch_count() - launches0
    lb.check_device_status(dev)
    tokens = cfg.img_tokens + cfg.txt_tokens
    step_fl = mmdit_step_flops(cfg, lora_rank, n_blocks, global_batch)
    n_params = sum(p.numel() for p in stack.lora_parameters())
    out = {
        "metric": "MMDiT LoRA train steps/s", "value": steps / (ms * 1e-3), "unit": "steps/s",
        "n_gpus": world, "steps": steps, "warmup": max(warmup, 2), "ms_per_step": ms / steps,
        "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "mmdit-double-stream", "blocks": n_blocks, "hidden": h, "heads": cfg.heads,
                   "mlp": cfg.mlp, "lora_rank": lora_rank, "global_batch": global_batch,
                   "samples_per_gpu": b, "tokens_per_sample": tokens, "quant": "int4 block 64",
                   "grad_checkpointing": True, "parallelism": f"dp{world}",
                   "cuda_streams": "text chain beside the image chain (2 streams per block)" if two_streams else "one",
                   "grad_allreduce": f"one slice per {reduce_every} block(s), started from the reverse sweep",
                   "cuda_graphs": "one per block forward, one head, one per block replay + backward" if graphs
                   else "none (eager launches)",
                   "weight_copies": {"none": "none (every call dequantises into the workspace)",
                                     "resident": "resident bf16 copy of every frozen weight (no dequantisation pass)",
                                     "block": "two arenas of one block's bf16 copies, refilled one block ahead "
                                              "of the sweep on a side stream"}[weight_copies]},
        "model": {"step_flops": step_fl, "tflops": step_fl / (ms / steps * 1e-3) / 1e12,
                  "lora_params": n_params, "grad_bucket_bytes": stack.flat.numel * 4},
        "tokens_per_s": tokens * global_batch * steps / (ms * 1e-3),
        "loss_first": losses[0], "loss_last": losses[-1], "gpu_launches": int(launches),
    }
    del trainer, stack
    torch.cuda.empty_cache()
    return out


def run_train_step(args):
    """`--regime step`: LoRA training steps/s of a double-stream MMDiT block stack (the two model
    workloads: hidden 3072, 24 heads, MLP 12288, every linear int4 block-64 + LoRA, 4096 image + 512
    text tokens per sample, bf16 activations, block-checkpoint recompute, flow-matching MSE loss),
    data-parallel over the ranks torchrun started, LoRA gradients all-reduced in one flat bucket.
    `--blocks`, `--batch` and `--rank` pick the workload: the defaults are the one-block workload (batch 1,
    rank 16); `--blocks 24 --batch 8 --rank 32` is the full stack.  `--model gpt2` runs the text
    workload instead (12 layers, 768 wide, int4 block-64 base, rank 8 on q/k/v/o, batch 8 x 1024)."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.model == "gpt2":
        line = measure_gpt2_step(dev, world, rank, args.steps, args.warmup, graphs=not args.no_graph)
    else:
        line = measure_train_step(dev, world, rank, args.blocks, args.batch, args.rank, args.steps, args.warmup,
                                  weight_copies=args.weight_copies, graphs=not args.no_graph,
                                  reduce_every=args.reduce_every if args.reduce_every > 0 else args.blocks,
                                  two_streams=not args.one_stream)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_gpt2_step(dev, world: int, rank: int, steps: int, warmup: int, batch: int = 8, seq: int = 1024,
                      graphs: bool = True):
    """The text workload: GPT-2-small-shaped decoder (12 layers, 768, 12 heads, MLP 3072, vocabulary
    50257; crates/loractl-core/src/gpt2.rs:93-103), every per-block projection int4 block 64, LoRA rank 8
    on q/k/v/o, seeded uniform token ids, next-token cross-entropy, AdamW on the flat adapter bucket;
    data parallel over the ranks (batch sharded, gradients all-reduced)."""
    import torch
    import torch.distributed as dist

    import loractl_b200 as lb
    from loractl_b200 import _lib as L
    from loractl_b200 import dp
    from loractl_b200 import gpt2 as G
    from loractl_b200.adapters import LoraConfig, TargetSpec, build_adapters
    from loractl_b200.optim import AdamW, FlatAdapters, nonfinite_flag

    cfg = G.Gpt2Config.gpt2_small()
    torch.manual_seed(5)
    model = G.Gpt2(cfg, split_qkv=True).to(dev)
    with torch.no_grad():
        gw = torch.Generator(device=dev).manual_seed(5)
        for _, base in model.base_linears():
            base.as_plain().weight.copy_(torch.randn(base.as_plain().weight.shape, generator=gw, device=dev) * 0.02)
            base.as_plain().bias.zero_()
        model.wte.weight.copy_(torch.randn(model.wte.weight.shape, generator=gw, device=dev) * 0.02)
        model.wpe.weight.copy_(torch.randn(model.wpe.weight.shape, generator=gw, device=dev) * 0.01)
    model.into_quantized(4, block=64)
    model = model.to(torch.bfloat16)
    lcfg = LoraConfig(rank=8, alpha=8.0, targets=[TargetSpec(r"attn\.(q|k|v|c_proj)$")])
    torch.manual_seed(5)
    adapters = build_adapters(model.injectable_sites(), lcfg, dev)
    with torch.no_grad():
        g2 = torch.Generator(device=dev).manual_seed(6)
        for d in adapters.deltas:
            d.lora_b.copy_(torch.randn(d.lora_b.shape, generator=g2, device=dev) * 0.01)
    flat = FlatAdapters(adapters, dev)
    optim = AdamW(flat)
    global_batch = max(batch, world)
    lo, hi = dp.shard_range(global_batch, rank, world)
    gd = torch.Generator(device=dev).manual_seed(100 + rank)
    ids = torch.randint(0, cfg.vocab_size, (hi - lo, seq), generator=gd, device=dev)

    flat.refresh_mirrors()
    graphed = None
    if graphs:  # forward + loss + backward as one CUDA graph (ids are a fixed tensor here)
        from loractl_b200.harness import GraphedLossStep

        graphed = GraphedLossStep(lambda: G.next_token_loss(model(ids, adapters, dtype=torch.bfloat16), ids), dev)

    def one():
        flat.zero_grad()
        if graphed is not None:
            loss = graphed.replay()
        else:
            loss = G.next_token_loss(model(ids, adapters, dtype=torch.bfloat16), ids)
            loss.backward()
        flat.gather_autograd_grads()
        nonfinite_flag(flat.grads, flat.flag)
        scale = dp.sync_gradients(flat.grads, flat.flag)
        optim.step(1e-4, grad_scale=scale, skip_flag=flat.flag)
        flat.refresh_mirrors()  # the factors changed: every bf16 operand mirror in one batched launch
        return loss

    losses = [float(one()) for _ in range(max(warmup, 3))]
    lb.check_device_status(dev)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = L.lib().lq_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for _ in range(steps):
        last = one()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        tm = torch.tensor([ms], device=dev)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm.item())
    launches = L.lib().lq_kernel_launch_count() - launches0
    lb.check_device_status(dev)
    e, inner, tok = cfg.n_embd, cfg.n_inner, global_batch * seq
    lin = 2 * tok * (4 * e * e + 2 * e * inner) * cfg.n_layer          # frozen projections, forward
    lora = 2 * tok * 8 * (2 * e) * 4 * cfg.n_layer                      # rank-8 down + up on q/k/v/o
    att = 4 * global_batch * seq * seq * e * cfg.n_layer // 2           # causal: half the score matrix
    head = 2 * tok * e * cfg.vocab_size
    step_fl = (lin + lora + att + head) + (lin + 2 * lora + 2 * att + head)  # forward + backward (no weight grads)
    return {
        "metric": "text-model LoRA train steps/s", "value": steps / (ms * 1e-3), "unit": "steps/s", "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms / steps, "higher_is_better": True,
        "scaling": "strong", "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "gpt2-small-shaped decoder", "layers": cfg.n_layer, "hidden": e, "heads": cfg.n_head,
                   "mlp": inner, "vocab": cfg.vocab_size, "lora_rank": 8, "lora_sites": "q, k, v, o",
                   "global_batch": global_batch, "seq_len": seq, "quant": "int4 block 64", "parallelism": f"dp{world}",
                   "cuda_graphs": "forward + loss + backward as one graph" if graphs else "none (eager launches)"},
        "model": {"step_flops": step_fl, "tflops": step_fl / (ms / steps * 1e-3) / 1e12,
                  "lora_params": sum(p.numel() for d in adapters.deltas for p in (d.lora_a, d.lora_b))},
        "tokens_per_s": tok * steps / (ms * 1e-3), "loss_first": losses[0], "loss_last": float(last),
        "gpu_launches": int(launches),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", type=int, default=1, help="--regime step: blocks in the stack (full stack: 24)")
    ap.add_argument("--batch", type=int, default=1, help="--regime step: global batch (full stack: 8)")
    ap.add_argument("--rank", type=int, default=16, help="--regime step: LoRA rank (full stack: 32)")
    ap.add_argument("--regime", default="tensor", choices=["tensor", "stream", "step", "load"],
                    help="tensor: the headline fwd+bwd step; stream: packed-weight stream at <= 64 tokens; "
                         "step: LoRA training steps/s of a double-stream MMDiT block stack; "
                         "load: streaming quantize-at-load of one block from a scaled-fp8 checkpoint")
    ap.add_argument("--model", default="mmdit", choices=["mmdit", "gpt2"], help="--regime step: which caller of the path")
    ap.add_argument("--weight-copies", nargs="?", const="resident", default="resident", choices=["none", "resident", "block"],
                    help="--regime step: bf16 copies of the frozen weights. resident: of every weight, for the whole "
                         "run; block: two arenas of one block's copies, refilled one block ahead on a side stream")
    ap.add_argument("--one-stream", action="store_true",
                    help="--regime step: a block's text and image chains one after the other on one CUDA stream "
                         "(default: the text chain on a second stream beside the image chain)")
    ap.add_argument("--reduce-every", type=int, default=0,
                    help="--regime step: blocks per gradient all-reduce of the reverse sweep (1 = per block; "
                         "0 = all blocks: one all-reduce after the sweep)")
    ap.add_argument("--stream-tokens", default="1,8,16,64", help="--regime stream: token counts, comma separated")
    ap.add_argument("--stream-only", default=None, choices=["3072x3072", "3072x12288", "3072x12288-fp8"],
                    help="--regime stream: only this site shape (short runs for a profiler capture)")
    ap.add_argument("--no-extras", action="store_true",
                    help="tensor regime: skip the extra keys (int4_cfg1, stream, model_step) of the default line")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager launches instead of a CUDA graph of the step")
    ap.add_argument("--compute", default="bf16", choices=["bf16", "fp8"],
                    help="bf16: weights dequantised to bf16, bf16 MMA (parity-grade); fp8: native e4m3 MMA "
                         "on the stored fp8 weight with per-token e4m3 activations (scaled-fp8 workloads only)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.regime == "stream":
        run_stream(args)
    elif args.regime == "step":
        run_train_step(args)
    elif args.regime == "load":
        run_load(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
