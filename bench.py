#!/usr/bin/env python
"""Benchmark of the Winograd F(2x2,3x3) convolution path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--variant OPTSTS64] [--precision fp32]

A step is one pass of the operator (filter transform + fused kernel) over the ResNet-style 3x3
layer sweep at batch 128 per GPU: (C=K=64, 56x56), (128, 28x28), (256, 14x14), (512, 7x7),
stride 1, pad 1, fp32, layouts CHWN / CRSK / KHWN.  With N GPUs every rank runs the sweep on
its own 128 images (batch-sharded, no collective on the data path: weak scaling).  The metric
is effective TFLOP/s with the direct-convolution flop count 2*N*K*C*H*W*9 per layer, summed
over the job.  One JSON line is printed by rank 0.

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
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = [(128, 64, 64, 56), (128, 128, 128, 28), (128, 256, 256, 14), (128, 512, 512, 7)]  # N, C, K, H=W
WORKLOAD = "resnet3x3_sweep_N128: (C=K=64,56x56) (128,28x28) (256,14x14) (512,7x7), stride 1, pad 1"
METRIC = "effective TFLOP/s (direct-conv flops 2*N*K*C*H*W*9) over the N=128 ResNet 3x3 layer sweep"
# dram__bytes_read.sum + dram__bytes_write.sum per wino_fp32_kernel launch, averaged over the four
# layers of one step: ncu capture of this very command at full size (profiles/bench_dram_traffic.md).
DRAM_TRAFFIC_PER_LAUNCH = 81.05e6


def direct_flops(N, C, K, HW):
    return 2.0 * N * K * C * HW * HW * 9


def gemm_flops(N, C, K, HW):
    t = (HW + 1) // 2
    return 2.0 * 16 * N * t * t * C * K


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML while a region runs."""
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, torch, device, period=0.02):
        super().__init__(daemon=True)
        self.period, self.samples, self.reasons, self.max_mhz = period, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(device).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device)
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
    ap.add_argument("--no-cudnn", action="store_true", help="skip the cuDNN (torch conv2d) baseline")
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

    from opencnn_b200 import api, build
    if args.impl == "ours":
        api.variant_name(args.variant)       # loads the CUDA library or raises: no fallback
    else:
        ref.setup()

    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    layers = []
    for (N, C, K, HW) in LAYERS:
        x = torch.rand((C, HW, HW, N), device=dev, generator=gen) * 2 - 1
        g = torch.randn((C, 3, 3, K), device=dev, generator=gen) * 0.05
        y = torch.empty((K, HW, HW, N), device=dev)
        ws = torch.empty((C, 4, 4, K), device=dev)
        layers.append(dict(N=N, C=C, K=K, HW=HW, x=x, g=g, y=y, ws=ws))
    stream = torch.cuda.current_stream().cuda_stream

    def run_layer(L):
        if args.impl == "ours":
            e = api.conv3x3(L["x"], L["g"], L["y"], L["ws"], L["N"], L["C"], L["HW"], L["HW"], L["K"],
                            precision=args.precision, stream=stream, variant=args.variant)
        else:
            e = ref.forward(L["x"], L["g"], L["y"], L["ws"], L["N"], L["C"], L["HW"], L["K"])
        if e != 0:
            raise RuntimeError(f"operator returned cudaError {e}")

    def step():
        for L in layers:
            run_layer(L)

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

    # ---- device-resident timing -------------------------------------------------------------
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
    ms_total = max_over_ranks(t0.elapsed_time(t1))
    ms_per_step = ms_total / args.steps
    flops_step = sum(direct_flops(*L) for L in LAYERS) * world
    value = flops_step / (ms_per_step * 1e-3) * 1e-12

    # ---- per-kernel durations (dominant kernel for the roofline), same buffers, same order ----
    per_layer = []
    roof = None
    if args.impl == "ours":
        reps = 30
        ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
                torch.cuda.Event(enable_timing=True)) for _ in layers] for _ in range(reps)]
        for r in range(reps):
            for i, L in enumerate(layers):
                a, b, c = ev[r][i]
                a.record()
                api.filter_transform(L["g"], L["ws"], L["C"], L["K"], stream=stream, variant=args.variant)
                b.record()
                api.winograd_forward(L["x"], L["ws"], L["y"], L["N"], L["C"], L["HW"], L["HW"], L["K"],
                                     precision=args.precision, stream=stream, variant=args.variant)
                c.record()
        torch.cuda.synchronize()
        tot_gemm, tot_ms = 0.0, 0.0
        for i, L in enumerate(layers):
            fx = statistics.mean(ev[r][i][0].elapsed_time(ev[r][i][1]) for r in range(5, reps))
            fu = statistics.mean(ev[r][i][1].elapsed_time(ev[r][i][2]) for r in range(5, reps))
            shp = (L["N"], L["C"], L["K"], L["HW"])
            per_layer.append({"N": L["N"], "C": L["C"], "K": L["K"], "HW": L["HW"], "fx_us": fx * 1e3,
                              "fused_us": fu * 1e3, "fused_gemm_tflops": gemm_flops(*shp) / fu * 1e-9,
                              "eff_tflops": direct_flops(*shp) / (fx + fu) * 1e-9})
            tot_gemm += gemm_flops(*shp)
            tot_ms += fu
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
        achieved = tot_gemm / (tot_ms * 1e-3) * 1e-12
        roof = {"bound": "fp32", "kernel": "wino_fp32_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": DRAM_TRAFFIC_PER_LAUNCH,
                "work": "Winograd-domain GEMM flops 2*16*N*ceil(W/2)^2*C*K per launch, summed over the four layers, "
                        "over the sum of the four mean launch durations (CUDA events, this stream)",
                "peak_source": peak_src,
                "peak_busy_operands": peak_busy,
                "note": "the FFMA path is bound by the FP32 pipe, not by HBM or the tensor pipe; `peak` is the "
                        "issue-rate peak (operands that barely change); the same probe on operands that keep "
                        "changing, as in a real contraction, sustains `peak_busy_operands` on this part"}
    # ---- tensor-core path (additive option of the same operator; not the headline) ----------
    tensor_core = None
    if args.impl == "ours" and args.precision == "fp32" and not args.no_tensor_core:
        peak_bf16, peak_src = 1590.0, "fallback 1.59 PFLOP/s (MEASURED_PEAKS.json absent)"
        try:
            mp = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            peak_bf16, peak_src = float(mp["bf16_tflops"]), "MEASURED_PEAKS.json bf16_tflops (cuBLAS burst)"
        except Exception:
            pass
        tensor_core = {"peak_bf16_tflops": peak_bf16, "peak_source": peak_src,
                       "peak_tf32_tflops": peak_bf16 / 2, "peak_tf32_source": "half the bf16 figure (hardware rate ratio)"}
        for prec in ("bf16", "tf32"):
            reps_tc = 20
            evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
                     torch.cuda.Event(enable_timing=True)) for _ in layers] for _ in range(reps_tc)]
            for r in range(reps_tc):
                for i, L in enumerate(layers):
                    a, b, c = evs[r][i]
                    a.record()
                    api.filter_transform(L["g"], L["ws"], L["C"], L["K"], precision=prec, stream=stream, variant=args.variant)
                    b.record()
                    e = api.winograd_forward(L["x"], L["ws"], L["y"], L["N"], L["C"], L["HW"], L["HW"], L["K"],
                                             precision=prec, stream=stream, variant=args.variant)
                    c.record()
                    if e != 0:
                        raise RuntimeError(f"tensor-core path returned cudaError {e}")
            torch.cuda.synchronize()
            rows, tg, td, tt = [], 0.0, 0.0, 0.0
            for i, L in enumerate(layers):
                fx = statistics.mean(evs[r][i][0].elapsed_time(evs[r][i][1]) for r in range(3, reps_tc))
                fu = statistics.mean(evs[r][i][1].elapsed_time(evs[r][i][2]) for r in range(3, reps_tc))
                shp = (L["N"], L["C"], L["K"], L["HW"])
                rows.append({"fx_us": fx * 1e3, "fused_us": fu * 1e3, "eff_tflops": direct_flops(*shp) / (fx + fu) * 1e-9,
                             "gemm_tflops": gemm_flops(*shp) / fu * 1e-9})
                tg += gemm_flops(*shp); td += direct_flops(*shp); tt += fx + fu
            tf_fused = sum(r_["fused_us"] for r_ in rows) * 1e-6
            pk = peak_bf16 if prec == "bf16" else peak_bf16 / 2
            tensor_core[prec] = {"layers": rows, "eff_tflops": td / (tt * 1e-3) * 1e-12, "ms_per_step": tt,
                                 "roofline": {"bound": "tensor", "kernel": "wino_tc_kernel", "achieved": tg / tf_fused * 1e-12,
                                              "peak": pk, "unit": "TFLOP/s", "frac": tg / tf_fused * 1e-12 / pk}}
    # ---- cuDNN through torch (library baseline, NCHW tensors of the same shapes) ------------
    cudnn = None
    if args.impl == "ours" and world == 1 and not args.no_cudnn:
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
    clocks = sampler.stop()

    # ---- end to end with host buffers -------------------------------------------------------
    host = []
    for L in layers:
        hx = torch.empty(L["x"].shape, pin_memory=True).copy_(L["x"].cpu())
        hg = torch.empty(L["g"].shape, pin_memory=True).copy_(L["g"].cpu())
        hy = torch.empty(L["y"].shape, pin_memory=True)
        host.append((hx, hg, hy))
    h2d = sum(hx.numel() * 4 + hg.numel() * 4 for hx, hg, _ in host)
    d2h = sum(hy.numel() * 4 for _, _, hy in host)
    if args.impl == "ours":
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
                    if p.run(hx.data_ptr(), hg.data_ptr(), hy.data_ptr()) != 0:
                        raise RuntimeError("host plan failed")
                return
            slot = e2e_count[0] % depth_box[0]
            e2e_count[0] += 1
            for p in plans[slot]:                         # the step two back used this slot: its results must be home
                if p.wait() != 0:
                    raise RuntimeError("host plan failed")
            for p, (hx, hg, _), hy in zip(plans[slot], host, host_out[slot]):
                if p.run_async(hx.data_ptr(), hg.data_ptr(), hy.data_ptr()) != 0:
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
        for d in range(0, max_depth + 1):               # 0: strictly sequential (HostPlan.run per layer)
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
                run_layer(L)
                hy.copy_(L["y"], non_blocking=True)
            torch.cuda.synchronize()

        def e2e_drain():
            torch.cuda.synchronize()
    for _ in range(3):
        e2e_step()
    e2e_drain()
    sync_all()
    w0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()
    e2e_drain()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - w0) * 1e3) / args.e2e_steps
    e2e = {"value": flops_step / (e2e_ms * 1e-3) * 1e-12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": args.e2e_steps,
           "how": "pinned host buffers -> opencnn_host_plan_run_async per layer (H2D, FX, fused kernel, D2H on the "
                  "plan's stream); up to three plan sets in rotation (how many - or none: layer after layer - is settled by a short untimed trial) so "
                  "uploads of a step overlap downloads of the steps before; every step's outputs are waited for "
                  "inside the timed region" if args.impl == "ours" else
                  "pinned host buffers; per layer H2D, reference call, D2H on the default stream; one sync per step"}
    if args.impl == "ours":
        e2e["plan_sets_in_rotation"] = depth_box[0]
    if args.impl == "ours":
        for slot in plans:
            for p in slot:
                p.close()
        status = api.last_device_status(args.variant)
        if status != 0:
            raise RuntimeError(f"device status word = {status}: a bounded wait ran out; results invalid")

    cb = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.impl == "ours":
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
                       "us_per_layer": ms_per_step * 1e3 / len(LAYERS)},
            "e2e": e2e, "gpu_launches": 2 * len(LAYERS) * args.steps, "clocks": clocks,
        }
        if args.impl == "reference":
            line["impl"] = "reference"
            line["cpu_baseline"] = {"value": value, "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                    "sample": "the reference has no CPU implementation: its own CUDA kernels "
                                              "(oracle/_ref, built for sm_100a) were timed on the GPU"}
        else:
            line["roofline"] = roof
            line["cpu_baseline"] = cb
            line["layers"] = per_layer
            line["tensor_core"] = tensor_core
            line["cudnn"] = cudnn
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
