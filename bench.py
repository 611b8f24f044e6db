#!/usr/bin/env python
"""Benchmark of the Winograd F(2x2,3x3) convolution path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--variant OPTSTS64] [--precision fp32]

Headline: a step is one pass of the operator (filter transform + fused kernel) over the
ResNet-style 3x3 layer sweep at batch 128 per GPU: (C=K=64, 56x56), (128, 28x28), (256, 14x14),
(512, 7x7), stride 1, pad 1, fp32, layouts CHWN / CRSK / KHWN.  With N GPUs every rank runs the
sweep on its own 128 images (batch-sharded, no collective on the data path: weak scaling).  The
metric is effective TFLOP/s with the direct-convolution flop count 2*N*K*C*H*W*9 per layer,
summed over the job.  One JSON line is printed by rank 0.

The same line carries, measured in the same process: the four staging variants per layer
(`variants`), the reference bench's first shape N=32 (`config1`), the two wide stress layers
(`layer_a` GEMM-bound, `layer_b` transform/HBM-bound), the filter transform and the layout
adapters against the HBM roofline (`fx`, `adapters`), the tensor-core path with its error against
fp64 (`tensor_core`, `accuracy`), cuDNN (`cudnn`), and the ResNet-34 3x3 stack at N=1024 split
over the ranks - strong scaling - with the one-GPU time measured in the same job (`stack_n1024`).

`--impl reference` times the reference's own kernels (oracle/_ref, built from the reference
checkout for sm_100a) on the same workload; if that library or a GPU is absent it times the
CPU restatement of the path instead.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = [(128, 64, 64, 56), (128, 128, 128, 28), (128, 256, 256, 14), (128, 512, 512, 7)]  # N, C, K, H=W
WORKLOAD = "resnet3x3_sweep_N128: (C=K=64,56x56) (128,28x28) (256,14x14) (512,7x7), stride 1, pad 1"
METRIC = "effective TFLOP/s (direct-conv flops 2*N*K*C*H*W*9) over the N=128 ResNet 3x3 layer sweep"
VARIANTS = ("BASE", "OPTSTS64", "OPTSTS64_CMP", "OPTLDS64")
CONFIG1 = (32, 64, 64, 56)
LAYER_A = (64, 1024, 1024, 14)
LAYER_B = (256, 32, 64, 112)
# ResNet-34's stride-1 3x3 layers: (C=K, H=W, how many)
STACK = [(64, 56, 6), (128, 28, 8), (256, 14, 12), (512, 7, 6)]
STACK_BATCH = 1024
# dram__bytes_read.sum + dram__bytes_write.sum per wino_fp32_kernel launch, averaged over the four
# layers of one step, from an ncu capture of this very command at full size.
DRAM_TRAFFIC_PER_LAUNCH = 79.89e6
DRAM_TRAFFIC_SOURCE = "ncu capture of `bench.py --steps 2 --warmup 3 --no-extras` (two 1-pass metrics, 8 launches), kernel as of the capture"


def direct_flops(N, C, K, HW):
    return 2.0 * N * K * C * HW * HW * 9


def gemm_flops(N, C, K, HW):
    t = (HW + 1) // 2
    return 2.0 * 16 * N * t * t * C * K


def tensor_bytes(N, C, K, HW):
    """Unique bytes of input + filter + output."""
    return 4.0 * (N * C * HW * HW + 9 * C * K + N * K * HW * HW)


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML while a region runs."""
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, torch, device, period=0.005):
        super().__init__(daemon=True)
        self.period, self.samples, self.reasons, self.max_mhz = period, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = nvml_handle(pynvml, torch, device)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self._halt.is_set():
            try:
                self.samples.append(float(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                try:
                    mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def nvml_handle(pynvml, torch, device):
    try:
        uuid = str(torch.cuda.get_device_properties(device).uuid)
        return pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
    except Exception:
        return pynvml.nvmlDeviceGetHandleByIndex(device)


def bind_to_gpu_cores(torch, device):
    """Restricts this process to the CPU cores NVML reports as local to its GPU, so that the pinned host
    buffers allocated afterwards land on that socket's memory (first touch).  Only this process's
    own scheduling affinity is changed.  Returns a short description for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = nvml_handle(pynvml, torch, device)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus and cpus != os.sched_getaffinity(0):
            os.sched_setaffinity(0, cpus)
            return f"bound to the {len(cpus)} cores local to the GPU"
        return "cores local to the GPU = all allowed cores (nothing to bind)"
    except Exception as exc:
        return f"not bound ({type(exc).__name__})"


class Reference:
    """The reference's kernels from oracle/_ref (ctypes); None-like when unavailable."""

    def __init__(self, variant):
        path = os.path.join(ROOT, "oracle", "_ref", f"libref_{variant}.so")
        self.lib = None
        if os.path.exists(path):
            L = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
            vp, ci = ctypes.c_void_p, ctypes.c_int
            L.ref_upload_tables.restype = ci
            L.ref_convolutionForward.restype = ci
            L.ref_convolutionForward.argtypes = [vp, ci, ci, vp, ci, ci, ci, ci, vp, vp, ctypes.c_uint] + [ci] * 11
            self.lib = L

    def setup(self):
        if self.lib.ref_upload_tables() != 0:
            raise RuntimeError("reference constant tables could not be uploaded")

    def forward(self, x, g, y, ws, N, C, HW, K):
        td = (HW + 1) // 2
        return self.lib.ref_convolutionForward(x.data_ptr(), HW, HW, g.data_ptr(), HW, HW, N, K, y.data_ptr(),
                                               ws.data_ptr(), 0, td, N, 4, td * 4, C, K, C, 3, 3, 4, 2)


def cpu_baseline(sample_passes=3):
    """Multithreaded fp32 direct convolution (the oracle's port; the reference has no CPU path),
    timed on this host: the whole four-layer sweep, best of `sample_passes`."""
    import numpy as np
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "liboracle.so"))
    f = ctypes.POINTER(ctypes.c_float)
    lib.oc_direct_f32_omp.argtypes = [f, f, f] + [ctypes.c_int] * 5
    lib.oc_num_threads.restype = ctypes.c_int
    rng = np.random.default_rng(0)
    bufs = []
    for N, C, K, HW in LAYERS:
        x = rng.uniform(-1, 1, (C, HW, HW, N)).astype(np.float32)
        g = (rng.standard_normal((C, 3, 3, K)) * 0.05).astype(np.float32)
        bufs.append((x, g, np.empty((K, HW, HW, N), np.float32)))
    best = None
    for _ in range(sample_passes):
        t0 = time.perf_counter()
        for (N, C, K, HW), (x, g, y) in zip(LAYERS, bufs):
            lib.oc_direct_f32_omp(x.ctypes.data_as(f), g.ctypes.data_as(f), y.ctypes.data_as(f), N, C, K, HW, HW)
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    flops = sum(direct_flops(*L) for L in LAYERS)
    return {"value": flops / best * 1e-12, "unit": "TFLOP/s", "cores": int(lib.oc_num_threads()), "kind": "port",
            "sample": f"whole four-layer N=128 sweep, best of {sample_passes} passes, {best * 1e3:.1f} ms per pass",
            "ms_per_step": best * 1e3}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--variant", default="OPTSTS64")
    ap.add_argument("--precision", default="fp32", choices=["fp32", "tf32", "bf16"])
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--e2e-depth", type=int, default=3, help="plan sets used in rotation by the end-to-end measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tensor-core", action="store_true", help="skip the extra TF32/BF16 measurements")
    ap.add_argument("--no-cudnn", action="store_true", help="skip the cuDNN baselines")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip variants / config1 / layer_a / layer_b / fx / adapters / accuracy / stack_n1024")
    ap.add_argument("--layers", default=None,
                    help="override the workload, e.g. '64,64,64,56;128,256,256,14' (N,C,K,H=W per layer); "
                         "for profiling small cases, not for reported numbers")
    args = ap.parse_args()
    global LAYERS, WORKLOAD
    if args.layers:
        LAYERS = [tuple(int(v) for v in item.split(",")) for item in args.layers.split(";")]
        WORKLOAD = "custom: " + args.layers
    if args.warmup < 3:
        args.warmup = 3

    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")      # keep stdout for the one JSON line
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    have_gpu = torch.cuda.is_available()

    ref = Reference(args.variant) if args.impl == "reference" else None
    if args.impl == "reference" and (ref.lib is None or not have_gpu):
        # CPU port of the path on the host cores; rank 0 only.
        if rank == 0:
            cb = cpu_baseline()
            print(json.dumps({
                "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
                "steps": 3, "warmup": 0, "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD},
                "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0,
                "note": "reference kernels (oracle/_ref) or a GPU not available: timed the CPU restatement of the path"}))
        return
    if not have_gpu:
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    host_binding = bind_to_gpu_cores(torch, local_rank)

    from opencnn_b200 import api, build
    ours = args.impl == "ours"
    refs = {}
    if ours:
        api.variant_name(args.variant)       # loads the CUDA library or raises: no fallback
    else:
        ref.setup()
        refs[args.variant] = ref

    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)

    def make_layer(N, C, K, HW, sigma=0.05):
        x = torch.rand((C, HW, HW, N), device=dev, generator=gen) * 2 - 1
        g = torch.randn((C, 3, 3, K), device=dev, generator=gen) * sigma
        y = torch.empty((K, HW, HW, N), device=dev)
        ws = torch.empty((C, 4, 4, K), device=dev)
        return dict(N=N, C=C, K=K, HW=HW, x=x, g=g, y=y, ws=ws)

    def shape_of(L):
        return (L["N"], L["C"], L["K"], L["HW"])

    def ref_for(variant):
        if variant not in refs:
            r = Reference(variant)
            if r.lib is None:
                return None
            r.setup()
            refs[variant] = r
        return refs[variant]

    def run_layer(L, variant=None, precision=None):
        variant = variant or args.variant
        if ours:
            e = api.conv3x3(L["x"], L["g"], L["y"], L["ws"], L["N"], L["C"], L["HW"], L["HW"], L["K"],
                            precision=precision or args.precision, stream=stream, variant=variant)
        else:
            e = ref_for(variant).forward(L["x"], L["g"], L["y"], L["ws"], L["N"], L["C"], L["HW"], L["K"])
        if e != 0:
            raise RuntimeError(f"operator returned cudaError {e}")

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def time_calls(fn, calls, warm=1):
        """The reference's protocol (src/openCNN_winograd.cu:426-444): warm-up, then `calls` back-to-back calls
        between two events; ms per call."""
        for _ in range(warm):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(calls):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / calls

    def time_split(Ls, variant, precision, reps, skip):
        """Filter transform and fused kernel timed separately (events around each launch), layers interleaved
        in order so that every launch finds its tensors evicted from L2 by the others; mean us per layer."""
        ev = [[tuple(torch.cuda.Event(enable_timing=True) for _ in range(3)) for _ in Ls] for _ in range(reps)]
        for r in range(reps):
            for i, L in enumerate(Ls):
                a, b, c = ev[r][i]
                a.record()
                e1 = api.filter_transform(L["g"], L["ws"], L["C"], L["K"], precision=precision, stream=stream, variant=variant)
                b.record()
                e2 = api.winograd_forward(L["x"], L["ws"], L["y"], L["N"], L["C"], L["HW"], L["HW"], L["K"],
                                          precision=precision, stream=stream, variant=variant)
                c.record()
                if e1 or e2:
                    raise RuntimeError(f"split entries returned cudaError {e1} / {e2}")
        torch.cuda.synchronize()
        out = []
        for i, L in enumerate(Ls):
            fx = statistics.mean(ev[r][i][0].elapsed_time(ev[r][i][1]) for r in range(skip, reps))
            fu = statistics.mean(ev[r][i][1].elapsed_time(ev[r][i][2]) for r in range(skip, reps))
            out.append((fx * 1e3, fu * 1e3))
        return out

    layers = [make_layer(*shp) for shp in LAYERS]

    def step():
        for L in layers:
            run_layer(L)

    # ---- device-resident timing (the headline) ------------------------------------------------
    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(torch, local_rank)
    sync_all()
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    sync_all()
    clocks = sampler.stop()                      # the clocks of the timed region, nothing else
    ms_total = max_over_ranks(t0.elapsed_time(t1))
    ms_per_step = ms_total / args.steps
    flops_step = sum(direct_flops(*L) for L in LAYERS) * world
    value = flops_step / (ms_per_step * 1e-3) * 1e-12

    # ---- per-kernel durations of the headline layers, taken right after the headline loop (the peak
    # probes below load the chip far more heavily, and kernels timed just after them run slower) ------
    headline_split = time_split(layers, args.variant, args.precision, reps=30, skip=5) if ours else None

    # ---- peaks ---------------------------------------------------------------------------------
    peaks = {}
    if ours:
        peak = peak_busy = None
        peak_src = "measured live: fma.rn.f32x2 issue-rate probe (opencnn_b200/csrc/peaks.cu), best of 3"
        try:
            pl = ctypes.CDLL(build.peaks_lib_path())
            out = ctypes.c_double(0.0)
            for fn_name in ("opencnn_peaks_fp32_tflops", "opencnn_peaks_fp32_tflops_busy"):
                fn = getattr(pl, fn_name)
                fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
                if fn(20000, 3, ctypes.byref(out)) == 0 and out.value > 0:
                    if fn_name.endswith("busy"):
                        peak_busy = out.value
                    else:
                        peak = out.value
        except (OSError, AttributeError):
            pass
        if peak is None:
            peak, peak_src = 148 * 128 * 2 * 1.965e9 * 1e-12, "nominal 148 SMs x 128 lanes x 2 x 1.965 GHz (probe library missing)"
        peaks.update(fp32_tflops=peak, fp32_source=peak_src, fp32_busy_operands_tflops=peak_busy)
        try:
            mp = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            peaks.update(hbm_gbs=float(mp["hbm_gbs"]), bf16_tflops=float(mp["bf16_tflops"]),
                         source="MEASURED_PEAKS.json (driver-measured copy bandwidth and cuBLAS bf16 burst): of measured")
        except Exception:
            peaks.update(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback 6.65 TB/s and 1.59 PFLOP/s (MEASURED_PEAKS.json absent): of fallback")
        if not args.no_tensor_core:
            # TF32 dense peak: the same kind of measurement as the driver's bf16 figure (library GEMM 8192^3,
            # best of 10), with TF32 operands.  A denominator only; nothing of the operator runs through it.
            old_tf32 = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            a_ = torch.randn(8192, 8192, device=dev)
            b_ = torch.randn(8192, 8192, device=dev)
            best = None
            for i in range(12):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch.matmul(a_, b_)
                e1.record()
                torch.cuda.synchronize()
                if i >= 2:
                    best = e0.elapsed_time(e1) if best is None else min(best, e0.elapsed_time(e1))
            torch.backends.cuda.matmul.allow_tf32 = old_tf32
            del a_, b_
            peaks.update(tf32_tflops=2.0 * 8192 ** 3 / (best * 1e-3) * 1e-12,
                         tf32_source="measured live: torch.matmul 8192^3 with TF32 operands (cuBLAS), best of 10 (burst)")

    # ---- dominant kernel -> roofline ------------------------------------------------------------
    per_layer, roof = [], None
    if ours:
        split = headline_split
        tot_gemm = tot_ms = 0.0
        for L, (fx, fu) in zip(layers, split):
            shp = shape_of(L)
            per_layer.append({"N": L["N"], "C": L["C"], "K": L["K"], "HW": L["HW"], "fx_us": fx, "fused_us": fu,
                              "fused_gemm_tflops": gemm_flops(*shp) / fu * 1e-6,
                              "eff_tflops": direct_flops(*shp) / (fx + fu) * 1e-6})
            tot_gemm += gemm_flops(*shp)
            tot_ms += fu * 1e-3
        achieved = tot_gemm / (tot_ms * 1e-3) * 1e-12
        roof = {"bound": "fp32", "kernel": "wino_fp32_kernel", "achieved": achieved, "peak": peaks["fp32_tflops"],
                "unit": "TFLOP/s", "frac": achieved / peaks["fp32_tflops"], "traffic": DRAM_TRAFFIC_PER_LAUNCH,
                "traffic_source": DRAM_TRAFFIC_SOURCE,
                "work": "Winograd-domain GEMM flops 2*16*N*ceil(W/2)^2*C*K per launch, summed over the four layers, "
                        "over the sum of the four mean launch durations (CUDA events, this stream)",
                "peak_source": peaks["fp32_source"],
                "peak_busy_operands": peaks["fp32_busy_operands_tflops"],
                "note": "the FFMA path is bound by the FP32 pipe, not by HBM or the tensor pipe; `peak` is the "
                        "issue-rate peak (operands that barely change); the same probe on operands that keep "
                        "changing, as in a real contraction, sustains `peak_busy_operands` on this part"}

    extras = not args.no_extras and not args.layers

    # ---- the four staging variants, per layer ---------------------------------------------------
    variants = None
    if extras:
        variants = {}
        for v in VARIANTS:
            if ours:
                rows = time_split(layers, v, "fp32", reps=15, skip=3)
                variants[v] = {"fx_us": [r[0] for r in rows], "fused_us": [r[1] for r in rows]}
            elif ref_for(v) is not None:
                variants[v] = {"operator_us": [time_calls(lambda L=L: run_layer(L, variant=v), 20) * 1e3 for L in layers]}

    # ---- one layer at a time: the reference bench's first shape and the two stress layers -----------
    def one_layer(shp, calls, precisions):
        L = make_layer(*shp)
        out = {"shape_N_C_K_HW": list(shp), "calls": calls,
               "protocol": "1 warm-up, then back-to-back operator calls (filter transform included) between two events"}
        for prec in precisions:
            ms = time_calls(lambda: run_layer(L, precision=prec), calls)
            row = {"operator_us": ms * 1e3, "eff_tflops": direct_flops(*shp) / ms * 1e-9}
            if ours:
                (fx, fu), = time_split([L], args.variant, prec, reps=max(6, calls // 4), skip=2)
                row.update(fx_us=fx, fused_us=fu, gemm_tflops=gemm_flops(*shp) / fu * 1e-6)
                pk = {"fp32": peaks["fp32_tflops"], "bf16": peaks["bf16_tflops"], "tf32": peaks.get("tf32_tflops")}[prec]
                if pk:
                    row["roofline"] = {"bound": "fp32" if prec == "fp32" else "tensor", "achieved": row["gemm_tflops"],
                                       "peak": pk, "unit": "TFLOP/s", "frac": row["gemm_tflops"] / pk}
                row["hbm"] = {"bound": "hbm", "achieved": tensor_bytes(*shp) / (fu * 1e-6) * 1e-9, "peak": peaks["hbm_gbs"],
                              "unit": "GB/s", "frac": tensor_bytes(*shp) / (fu * 1e-6) * 1e-9 / peaks["hbm_gbs"],
                              "bytes": tensor_bytes(*shp), "work": "unique input + filter + output bytes over the fused kernel's time"}
            out[prec] = row
        del L
        torch.cuda.empty_cache()
        return out

    config1 = layer_a = layer_b = None
    if extras:
        precs = ["fp32"] + (["tf32", "bf16"] if ours and not args.no_tensor_core else [])
        config1 = one_layer(CONFIG1, 100, precs)
        layer_a = one_layer(LAYER_A, 20, precs)
        layer_b = one_layer(LAYER_B, 20, precs)

    # ---- HBM-bound helpers: filter transform at C=K=1024, layout adapters on the largest sweep tensor -------
    fx_sec = adapters = None
    if extras and ours:
        C = K = 1024
        g = torch.randn((C, 3, 3, K), device=dev, generator=gen) * 0.05
        ws = torch.empty((C, 4, 4, K), device=dev)
        fx_sec = {"C": C, "K": K}
        for prec, out_b in (("fp32", 4), ("tf32", 4), ("bf16", 2)):
            # 105 MB is below the L2 size, so between calls a 256 MB buffer is rewritten to evict it
            flush = torch.empty(64 * 1024 * 1024, device=dev)
            ts = []
            for i in range(12):
                flush.fill_(float(i))
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                api.filter_transform(g, ws, C, K, precision=prec, stream=stream, variant=args.variant)
                e1.record()
                torch.cuda.synchronize()
                if i >= 2:
                    ts.append(e0.elapsed_time(e1))
            us = statistics.mean(ts) * 1e3
            nbytes = C * K * (9 * 4 + 16 * out_b)
            fx_sec[prec] = {"us": us, "bytes": nbytes, "gbs": nbytes / us * 1e-3, "frac_of_hbm_peak": nbytes / us * 1e-3 / peaks["hbm_gbs"]}
            del flush
        fx_sec["how"] = "L2 flushed between calls (256 MB fill); algorithmic bytes C*K*(9*4 + 16*element size); kernel fx_kernel / fx_tc_kernel"
        del g, ws
        N, C, K, HW = LAYERS[0]
        src = torch.randn((N, C, HW, HW), device=dev, generator=gen)
        dst = torch.empty((C, HW, HW, N), device=dev)
        back = torch.empty((N, K, HW, HW), device=dev)
        adapters = {"shape_N_C_HW": [N, C, HW], "bytes": 2.0 * src.numel() * 4, "kernel": "transpose_kernel"}
        for name, fn in (("nchw_to_chwn", lambda: api.nchw_to_chwn(src, dst, N, C, HW, HW, stream=stream, variant=args.variant)),
                         ("khwn_to_nkhw", lambda: api.khwn_to_nkhw(dst, back, N, K, HW, HW, stream=stream, variant=args.variant))):
            ms = time_calls(fn, 20, warm=2)
            adapters[name] = {"us": ms * 1e3, "gbs": adapters["bytes"] / ms * 1e-6,
                              "frac_of_hbm_peak": adapters["bytes"] / ms * 1e-6 / peaks["hbm_gbs"]}
        adapters["how"] = "20 back-to-back calls; 205 MB moved per call (> L2), read + write"
        del src, dst, back
        torch.cuda.empty_cache()

    # ---- accuracy against an fp64 direct convolution (library conv2d in double, on the first 32 images) ----
    def round_operand(t, prec):
        if prec == "bf16":
            return t.bfloat16().float()
        if prec == "tf32":                                    # round to nearest even at 10 mantissa bits
            u = t.view(torch.int32)
            u = (u + 0xFFF + ((u >> 13) & 1)) & ~0x1FFF
            return u.view(torch.float32)
        return t

    def error_vs_fp64(L, prec):
        import torch.nn.functional as F
        x, g = round_operand(L["x"], prec).contiguous(), round_operand(L["g"], prec).contiguous()
        y = torch.empty_like(L["y"])
        e = api.conv3x3(x, g, y, L["ws"], L["N"], L["C"], L["HW"], L["HW"], L["K"], precision=prec, stream=stream,
                        variant=args.variant)
        if e != 0:
            raise RuntimeError(f"operator returned cudaError {e}")
        n = min(32, L["N"])
        truth = F.conv2d(x[..., :n].permute(3, 0, 1, 2).double(), g.permute(3, 0, 1, 2).double(), padding=1)   # N K H W
        got = y[..., :n].permute(3, 0, 1, 2).double()
        rms = float(truth.pow(2).mean().sqrt())
        return float((got - truth).abs().max()) / rms

    accuracy = None
    if extras and ours:
        precs = ["fp32"] + (["tf32", "bf16"] if not args.no_tensor_core else [])
        accuracy = {"how": "max |y - fp64 direct convolution| / rms(truth) on the first 32 images of each N=128 layer; "
                           "tf32 / bf16: operands rounded once from the seeded fp32 tensors, truth computed from the rounded operands",
                    "layers": [list(shp) for shp in LAYERS]}
        for prec in precs:
            accuracy[prec] = {"max_err_over_rms": [error_vs_fp64(L, prec) for L in layers]}

    # ---- tensor-core path (additive option of the same operator; not the headline) ----------
    tensor_core = None
    if ours and args.precision == "fp32" and not args.no_tensor_core:
        tensor_core = {"peak_bf16_tflops": peaks["bf16_tflops"], "peak_source": peaks["source"],
                       "peak_tf32_tflops": peaks["tf32_tflops"], "peak_tf32_source": peaks["tf32_source"]}
        for prec in ("bf16", "tf32"):
            split = time_split(layers, args.variant, prec, reps=20, skip=3)
            rows, tg, td, tt = [], 0.0, 0.0, 0.0
            for L, (fx, fu) in zip(layers, split):
                shp = shape_of(L)
                rows.append({"fx_us": fx, "fused_us": fu, "eff_tflops": direct_flops(*shp) / (fx + fu) * 1e-6,
                             "gemm_tflops": gemm_flops(*shp) / fu * 1e-6})
                tg += gemm_flops(*shp); td += direct_flops(*shp); tt += (fx + fu) * 1e-3
            tf_fused = sum(r_["fused_us"] for r_ in rows) * 1e-6
            pk = peaks["bf16_tflops"] if prec == "bf16" else peaks["tf32_tflops"]
            tensor_core[prec] = {"layers": rows, "eff_tflops": td / (tt * 1e-3) * 1e-12, "ms_per_step": tt,
                                 "roofline": {"bound": "tensor", "kernel": "wino_tc_kernel (wino_tc64_kernel on the 64-filter layer: the library's own dispatch)", "achieved": tg / tf_fused * 1e-12,
                                              "peak": pk, "unit": "TFLOP/s", "frac": tg / tf_fused * 1e-12 / pk}}
            if accuracy and prec in accuracy:
                tensor_core[prec]["max_err_over_rms"] = accuracy[prec]["max_err_over_rms"]

    # ---- cuDNN (library baseline): through torch, and through the legacy API the reference uses ----------
    cudnn = None
    if ours and world == 1 and not args.no_cudnn:
        import torch.nn.functional as F
        cudnn = {"how": "torch.nn.functional.conv2d, cudnn.benchmark=True, 20 timed calls per layer after 5 warm-ups; "
                        "fp32 = TF32 disabled, NCHW; tf32 = TF32 allowed, channels_last", "version": torch.backends.cudnn.version()}
        old = (torch.backends.cudnn.benchmark, torch.backends.cudnn.allow_tf32)
        torch.backends.cudnn.benchmark = True
        for name, tf32, fmt in (("fp32_nchw", False, torch.contiguous_format), ("tf32_channels_last", True, torch.channels_last)):
            torch.backends.cudnn.allow_tf32 = tf32
            us = []
            for (N, C, K, HW) in LAYERS:
                xx = torch.randn(N, C, HW, HW, device=dev).to(memory_format=fmt)
                ww = (torch.randn(K, C, 3, 3, device=dev) * 0.05).to(memory_format=fmt)
                for _ in range(5):
                    F.conv2d(xx, ww, padding=1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(20):
                    F.conv2d(xx, ww, padding=1)
                b.record()
                torch.cuda.synchronize()
                us.append(a.elapsed_time(b) * 1e3 / 20)
                del xx, ww
            cudnn[name] = {"us_per_layer": us, "eff_tflops": sum(direct_flops(*L) for L in LAYERS) / (sum(us) * 1e-6) * 1e-12}
        torch.backends.cudnn.benchmark, torch.backends.cudnn.allow_tf32 = old
        # legacy API, true fp32 arithmetic (CUDNN_FMA_MATH): every algorithm, cudnnFind's ranking, and the
        # reference's pinned algorithm 6 - in a process of its own (system cuDNN)
        probe = build.cudnn_probe_path()
        if os.path.exists(probe) and extras:
            torch.cuda.synchronize()
            legacy = {"how": "opencnn_b200/csrc/cudnn_probe.cu: cudnnConvolutionForward, NCHW fp32, CUDNN_FMA_MATH, 1 warm-up + 20 calls per algorithm",
                      "layers": []}
            for (N, C, K, HW) in LAYERS:
                try:
                    res = subprocess.run([probe, str(N), str(C), str(HW), str(HW), str(K), "20"], capture_output=True,
                                         text=True, timeout=120, env={**os.environ, "CUDA_VISIBLE_DEVICES": os.environ.get("CUDA_VISIBLE_DEVICES", str(local_rank))})
                    r = json.loads(res.stdout.strip().splitlines()[-1])
                except Exception as exc:
                    r = {"error": f"{type(exc).__name__}: {exc}"}
                if "algos" in r:
                    a6 = next((a for a in r["algos"] if a["algo"] == 6), None)
                    legacy["layers"].append({"best_fp32": r.get("best_fp32"), "algo6_winograd_us": a6 and a6.get("us"),
                                             "algo6_why": a6 and a6.get("why"),
                                             "all_us": {a["name"]: a.get("us") for a in r["algos"]},
                                             "find_first": (r.get("find") or [None])[0]})
                    legacy["version"] = r.get("cudnn_version")
                else:
                    legacy["layers"].append(r)
            cudnn["legacy_api_fma_math"] = legacy

    # ---- ResNet-34 3x3 stack at N=1024, batch split over the ranks (strong scaling) ----------------
    stack = None
    if extras and args.precision == "fp32" and STACK_BATCH % (32 * world) == 0:
        def build_stack(n):
            stages = []
            for (C, HW, count) in STACK:
                sigma = (2.0 / (9 * C)) ** 0.5
                a = torch.rand((C, HW, HW, n), device=dev, generator=gen) * 2 - 1
                b = torch.empty((C, HW, HW, n), device=dev)
                filt = [torch.randn((C, 3, 3, C), device=dev, generator=gen) * sigma for _ in range(count)]
                ws = torch.empty((C, 4, 4, C), device=dev)
                stages.append((C, HW, n, a, b, filt, ws))
            return stages

        def run_stack(stages):
            # within a stage every layer's KHWN output is the next layer's CHWN input (C = K): two buffers in turn
            for (C, HW, n, a, b, filt, ws) in stages:
                src, dst = a, b
                for g in filt:
                    run_layer(dict(N=n, C=C, K=C, HW=HW, x=src, g=g, y=dst, ws=ws))
                    src, dst = dst, src

        def time_stack(stages, reps):
            run_stack(stages)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                run_stack(stages)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        n_local = STACK_BATCH // world
        stages = build_stack(n_local)
        sync_all()
        ms_stack = max_over_ranks(time_stack(stages, 3))
        del stages
        torch.cuda.empty_cache()
        flops = sum(direct_flops(STACK_BATCH, C, C, HW) * cnt for (C, HW, cnt) in STACK)
        stack = {"batch": STACK_BATCH, "images_per_gpu": n_local, "layers": sum(c for _, _, c in STACK), "scaling": "strong",
                 "ms_per_stack": ms_stack, "eff_tflops": flops / ms_stack * 1e-9,
                 "how": "6x(64,56) 8x(128,28) 12x(256,14) 6x(512,7) layers, weights N(0, 2/(9C)), input U(-1,1); each layer's "
                        "output feeds the next of its stage; 1 warm-up pass + 3 timed passes between two events, max over ranks"}
        if world > 1:
            # the one-GPU time of the same job: rank 0 alone runs all 1024 images while the others wait
            ms_one = 0.0
            if rank == 0:
                full = build_stack(STACK_BATCH)
                ms_one = time_stack(full, 2)
                del full
                torch.cuda.empty_cache()
            sync_all()
            ms_one = max_over_ranks(ms_one)
            stack.update(ms_per_stack_one_gpu=ms_one, speedup=ms_one / ms_stack, strong_efficiency=ms_one / ms_stack / world)
        else:
            stack.update(ms_per_stack_one_gpu=ms_stack, speedup=1.0, strong_efficiency=1.0)

    # ---- end to end with host buffers -------------------------------------------------------
    host = []
    for L in layers:
        hx = torch.empty(L["x"].shape, pin_memory=True).copy_(L["x"].cpu())
        hg = torch.empty(L["g"].shape, pin_memory=True).copy_(L["g"].cpu())
        hy = torch.empty(L["y"].shape, pin_memory=True)
        host.append((hx, hg, hy))
    h2d = sum(hx.numel() * 4 + hg.numel() * 4 for hx, hg, _ in host)
    d2h = sum(hy.numel() * 4 for _, _, hy in host)
    copy_only = [False]
    if ours:
        # `depth` plan sets (device buffers + stream) and host output buffers per layer, used in rotation, so
        # that the uploads of one step overlap the downloads of the steps before (PCIe is full duplex).
        # A plan is waited for before it is used again; the timed region ends after every step has landed.
        max_depth = max(1, args.e2e_depth)
        plans = [[api.HostPlan(L["N"], L["C"], L["HW"], L["HW"], L["K"], precision=args.precision, variant=args.variant)
                  for L in layers] for _ in range(max_depth)]
        host_out = [[hy for _, _, hy in host]] + [[torch.empty(hy.shape, pin_memory=True) for _, _, hy in host]
                                                  for _ in range(max_depth - 1)]
        e2e_count = [0]
        depth_box = [max_depth]          # how many of the sets are in rotation

        def e2e_step():
            if depth_box[0] == 0:                         # one layer after the other, one copy in flight at a time
                for p, (hx, hg, _), hy in zip(plans[0], host, host_out[0]):
                    fn = p.copy_async if copy_only[0] else p.run_async
                    if fn(hx.data_ptr(), hg.data_ptr(), hy.data_ptr()) != 0 or p.wait() != 0:
                        raise RuntimeError("host plan failed")
                return
            slot = e2e_count[0] % depth_box[0]
            e2e_count[0] += 1
            for p in plans[slot]:                         # the step `depth` back used this slot: its results must be home
                if p.wait() != 0:
                    raise RuntimeError("host plan failed")
            for p, (hx, hg, _), hy in zip(plans[slot], host, host_out[slot]):
                fn = p.copy_async if copy_only[0] else p.run_async
                if fn(hx.data_ptr(), hg.data_ptr(), hy.data_ptr()) != 0:
                    raise RuntimeError("host plan failed")

        def e2e_drain():
            for slot in range(max_depth):
                for p in plans[slot]:
                    if p.wait() != 0:
                        raise RuntimeError("host plan failed")

        # Untimed trial: how many sets to rotate.  One GPU alone is limited by its own PCIe link and gains from
        # three; eight GPUs share the host's copy bandwidth, which on the boxes measured delivers more with few
        # copies in flight, so the strictly sequential form (one copy at a time per GPU) is a candidate too.
        trial = {}
        for d in range(0, max_depth + 1):               # 0: strictly sequential (one layer after the other)
            depth_box[0] = d
            for _ in range(2):
                e2e_step()
            e2e_drain()
            sync_all()
            t0 = time.perf_counter()
            for _ in range(8):
                e2e_step()
            e2e_drain()
            trial[d] = max_over_ranks(time.perf_counter() - t0)
        # the same on every rank (the times are maxima over ranks); within 2 % the deeper rotation wins
        best = min(trial.values())
        depth_box[0] = max(d for d, t in trial.items() if t <= 1.02 * best)
    else:
        def e2e_step():
            for L, (hx, hg, hy) in zip(layers, host):
                L["x"].copy_(hx, non_blocking=True)
                L["g"].copy_(hg, non_blocking=True)
                if not copy_only[0]:
                    run_layer(L)
                hy.copy_(L["y"], non_blocking=True)
            torch.cuda.synchronize()

        def e2e_drain():
            torch.cuda.synchronize()

    def time_e2e():
        for _ in range(3):
            e2e_step()
        e2e_drain()
        sync_all()
        w0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        e2e_drain()
        torch.cuda.synchronize()
        return max_over_ranks((time.perf_counter() - w0) * 1e3) / args.e2e_steps

    e2e_ms = time_e2e()
    copy_only[0] = True                           # the same copies, same rotation, no kernels: the floor
    floor_ms = time_e2e()
    copy_only[0] = False
    e2e = {"value": flops_step / (e2e_ms * 1e-3) * 1e-12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": args.e2e_steps,
           "copy_floor_ms": floor_ms, "frac_of_copy_floor": floor_ms / e2e_ms,
           "copy_floor_gbs_all_gpus": (h2d + d2h) * world / floor_ms * 1e-6,
           "limiter": "host<->device copies (PCIe and, with several GPUs, the host's memory system), not a kernel and "
                      "not NCCL: `copy_floor_ms` is the same step with the kernels left out",
           "host_binding": host_binding,
           "how": "pinned host buffers -> opencnn_host_plan_run_async per layer (H2D, FX, fused kernel, D2H on the "
                  "plan's stream); up to three plan sets in rotation (how many - or none: layer after layer - is settled by a short untimed trial) so "
                  "uploads of a step overlap downloads of the steps before; every step's outputs are waited for "
                  "inside the timed region" if ours else
                  "pinned host buffers; per layer H2D, reference call, D2H on the default stream; one sync per step"}
    if ours:
        e2e["plan_sets_in_rotation"] = depth_box[0]
        for slot in plans:
            for p in slot:
                p.close()
        for v in ([args.variant] + (list(VARIANTS) if variants else [])):
            status = api.last_device_status(v)
            if status != 0:
                raise RuntimeError(f"device status word = {status} ({v}): a bounded wait ran out; results invalid")

    cb = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and ours:
        try:
            full = cpu_baseline()
            cb = {k: full[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except OSError as exc:
            cb = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port", "sample": f"oracle library missing: {exc}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32" if args.precision == "fp32" else args.precision, "data": "synthetic",
            "config": {"workload": WORKLOAD, "images_per_gpu": LAYERS[0][0], "global_batch": LAYERS[0][0] * world,
                       "variant": args.variant, "precision": args.precision, "parallelism": f"batch-sharded x{world}",
                       "l2": "each layer has its own buffers; one step touches 398 MB > 126 MB L2 before a buffer is reused",
                       "note": "the headline keeps 128 images per GPU (weak scaling); the N=1024 stack split over the GPUs "
                               "(strong scaling) is the `stack_n1024` section"},
            "us_per_layer": ms_per_step * 1e3 / len(LAYERS),
            "e2e": e2e, "gpu_launches": 2 * len(LAYERS) * args.steps, "clocks": clocks,
            "variants": variants, "config1": config1, "layer_a": layer_a, "layer_b": layer_b, "stack_n1024": stack,
        }
        if not ours:
            line["impl"] = "reference"
            line["cpu_baseline"] = {"value": value, "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                    "sample": "the reference has no CPU implementation: its own CUDA kernels "
                                              "(oracle/_ref, built for sm_100a) were timed on the GPU"}
        else:
            line["roofline"] = roof
            line["cpu_baseline"] = cb
            line["layers"] = per_layer
            line["fx"] = fx_sec
            line["adapters"] = adapters
            line["accuracy"] = accuracy
            line["tensor_core"] = tensor_core
            line["cudnn"] = cudnn
            line["peaks"] = peaks
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
