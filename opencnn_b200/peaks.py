"""Runs the measurement aids of csrc/peaks.cu and prints their tables:

    python -m opencnn_b200.peaks

* FP32 FMA rate (the roofline denominator of the fp32 path), with operands that barely change and
  with operands that keep changing;
* whether instructions mixed into a stream of packed FMAs cost issue slots;
* how long one SM waits for a 32 / 64 KB TMA load out of L2 with one to three loads in flight;
* SM cycles per tcgen05.mma (M = 128) in a long chain, by operand layout, N and issuing threads; the
  commit -> wait round trip; whether MMA operand reads and TMA writes share an SM's shared-memory bandwidth.
"""
import ctypes
import sys

from .build import build_peaks


def load():
    lib = ctypes.CDLL(build_peaks())
    d = ctypes.POINTER(ctypes.c_double)
    lib.opencnn_peaks_fp32_tflops.argtypes = [ctypes.c_int, ctypes.c_int, d]
    lib.opencnn_peaks_fp32_tflops_busy.argtypes = [ctypes.c_int, ctypes.c_int, d]
    lib.opencnn_peaks_issue_probe.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, d]
    lib.opencnn_peaks_tma_latency.argtypes = [ctypes.c_int] * 5 + [d]
    lib.opencnn_peaks_mma_rate.argtypes = [ctypes.c_int] * 6 + [d]
    lib.opencnn_peaks_mma_round_trip.argtypes = [ctypes.c_int] * 5 + [d]
    lib.opencnn_peaks_smem_share.argtypes = [ctypes.c_int] * 3 + [d, d]
    return lib


def _call(fn, *args):
    out = ctypes.c_double(0.0)
    err = fn(*args, ctypes.byref(out))
    if err != 0:
        raise RuntimeError(f"{fn.__name__}{args} returned cudaError {err}")
    return out.value


def issue_probe(lib, iters=20000):
    """{(extra, kind): ms} for the loop of 64 packed FMAs + extra instructions (kind 0 xor, 1 mov, 2 add.f32)."""
    cases = [(0, 0), (8, 0), (16, 0), (32, 0), (64, 0), (16, 1), (32, 1), (16, 2), (32, 2)]
    return {c: _call(lib.opencnn_peaks_issue_probe, c[0], c[1], iters) for c in cases}


def tma_latency(lib, grid, iters=400):
    """{(bytes, tiled, depth): cycles per load}."""
    return {(b, t, d): _call(lib.opencnn_peaks_tma_latency, b, t, d, iters, grid)
            for b in (65536, 32768) for t in (1, 0) for d in (1, 2, 3)}


MMA_LAYOUTS = ["MN-major, as the fused kernels hold them", "K-major, no swizzle", "K-major, 32-byte swizzle",
               "K-major, 128-byte swizzle"]


def mma_rate(lib, grid, iters=2000):
    """{(kind, n, layout, issuers): cycles per MMA}; kind 0 BF16 (K = 16), 1 TF32 (K = 8).  All layouts with one
    issuing thread; the layout of the fused kernels also with two and four."""
    cases = [(k, n, l, 1) for k in (0, 1) for l in range(4) for n in (32, 64, 128, 256)]
    cases += [(k, n, 0, i) for k in (0, 1) for i in (2, 4) for n in (32, 64, 128)]
    return {c: _call(lib.opencnn_peaks_mma_rate, c[0], c[1], c[2], c[3], iters, grid) for c in cases}


def mma_round_trip(lib, grid, iters=2000):
    """{(kind, issuers): cycles from the first MMA of a group of 16 / issuers (N = 32) to the wake-up after its commit}."""
    return {(k, i): _call(lib.opencnn_peaks_mma_round_trip, k, 32, i, iters, grid) for k in (0, 1) for i in (1, 2, 4)}


def smem_share(lib, grid, groups=2000, loads=1600):
    """MMA operand reads (80 KB per group of 16 MMAs) and TMA writes (64 KB per load) alone and together:
    {"mma alone" | "tma alone" | "together": (mma cycles, tma cycles)}."""
    out = {}
    for name, g, l in (("mma alone", groups, 0), ("tma alone", 0, loads), ("together", groups, loads)):
        a, b = ctypes.c_double(0.0), ctypes.c_double(0.0)
        err = lib.opencnn_peaks_smem_share(g, l, grid, ctypes.byref(a), ctypes.byref(b))
        if err != 0:
            raise RuntimeError(f"opencnn_peaks_smem_share({g}, {l}, {grid}) returned {err}")
        out[name] = (a.value, b.value)
    return out


def main() -> int:
    import torch
    if not torch.cuda.is_available():
        print("needs a CUDA device", file=sys.stderr)
        return 1
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    lib = load()
    print(f"FP32 pipe, fma.rn.f32x2: {_call(lib.opencnn_peaks_fp32_tflops, 20000, 3):.1f} TFLOP/s (operands that barely change), "
          f"{_call(lib.opencnn_peaks_fp32_tflops_busy, 20000, 3):.1f} TFLOP/s (operands that keep changing)")
    kinds = ["xor", "mov", "add.f32"]
    base = None
    for (extra, kind), ms in issue_probe(lib).items():
        base = base or ms
        print(f"64 packed FMAs + {extra:2d} {kinds[kind]:8s}: {ms:.3f} ms  ({ms / base:.2f} x the plain loop)")
    for grid in (1, sms):
        for (b, t, d), cyc in tma_latency(lib, grid).items():
            print(f"{grid:3d} SMs  {b // 1024} KB {'tiled box ' if t else 'linear    '} {d} in flight: {cyc:6.0f} cycles per load, {b / cyc:5.1f} B/clk")
    for (k, n, l, i), cyc in mma_rate(lib, sms).items():
        macs = 128 * n * (16 if k == 0 else 8)
        print(f"tcgen05.mma {'BF16' if k == 0 else 'TF32'} 128x{n:<3d} {MMA_LAYOUTS[l]:40s} {i} issuing thread(s): "
              f"{cyc:6.1f} cycles per MMA, {macs / cyc:6.0f} MAC/clk")
    for (k, i), cyc in mma_round_trip(lib, sms).items():
        print(f"{'BF16' if k == 0 else 'TF32'} {16 // i:2d} MMAs 128x32 per thread, {i} thread(s), commit + wait after each group: "
              f"{cyc:6.0f} cycles per group")
    groups, loads = 2000, 1600
    for grid in (1, sms):
        for name, (a, b) in smem_share(lib, grid, groups, loads).items():
            mma = f"MMA operand reads {groups * 80 * 1024 / a:6.1f} B/clk" if a else "no MMAs"
            tma = f"TMA writes {loads * 65536 / b:6.1f} B/clk" if b else "no loads"
            print(f"{grid:3d} SMs  {name:10s}: {mma:32s} {tma}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
