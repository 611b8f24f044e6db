"""Command line compatible with the reference's benchmark binary `wgrad`
(argv: src/openCNN_winograd.cu:246-255; output line: :257, :118-125, :445-467;
sweep script bench/bench.sh).

    python -m opencnn_b200.wgrad N C H W K C 3 3 [--variant OPTSTS64] [--precision fp32]

Prints, like the reference, `in_n,in_c,in_h,filt_k,filt_h,<ms>,<TFLOPS>,<ms>,<TFLOPS>` where the
first pair is this library (1 warm-up + 100 calls between two CUDA events, filter transform
included in every call) and the second pair is cuDNN through torch (fp32, TF32 disabled), both
with the reference's flop formula 2*N*C*(H+2)*(W+2)*K*9 / 2.25.  `--header` prints the column
names of bench/bench.sh:1 first.  The result is compared with cuDNN's like the reference does
(src/openCNN_winograd.cu:177-201) but with a relative bound instead of |diff| <= 1.
"""
from __future__ import annotations

import argparse
import sys


def api_kernels():
    from .api import TC_KERNELS
    return TC_KERNELS


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("dims", nargs="*", type=int, help="N C H W K C R S (defaults 128 256 14 14 256 256 3 3)")
    ap.add_argument("--variant", default="OPTSTS64")
    ap.add_argument("--precision", default="fp32", choices=["fp32", "tf32", "bf16"])
    ap.add_argument("--tc-kernel", default="auto", choices=sorted(api_kernels()),
                    help="with --precision tf32/bf16: which tensor-core kernel runs (default: the library's own choice)")
    ap.add_argument("--header", action="store_true")
    ap.add_argument("--iterations", type=int, default=100)
    args = ap.parse_args(argv)
    d = list(args.dims) + [128, 256, 14, 14, 256, 256, 3, 3][len(args.dims):]
    N, C, H, W, K, C2, R, S = d[:8]
    if C2 != C or R != 3 or S != 3:
        print("Configuration not supported yet", file=sys.stderr)
        return 1

    import torch
    import torch.nn.functional as F

    from . import api

    if not torch.cuda.is_available():
        print("wgrad needs a CUDA device: the operator has no CPU path", file=sys.stderr)
        return 1
    if args.header:
        print("in_n,in_c,in_h,filt_k,filt_w,openCNN_sec,openCNN_flops,cuDNN_sec,cuDNN_flops")
    x = torch.rand(N, C, H, W, device="cuda")                       # U(0,1] like the reference's curand_uniform
    w = torch.rand(K, C, 3, 3, device="cuda")
    xc, wc = torch.empty((C, H, W, N), device="cuda"), torch.empty((C, 3, 3, K), device="cuda")
    y, ws = torch.empty((K, H, W, N), device="cuda"), torch.empty((C, 4, 4, K), device="cuda")
    if api.nchw_to_chwn(x, xc, N, C, H, W, variant=args.variant) or api.kcrs_to_crsk(w, wc, K, C, variant=args.variant):
        print("layout conversion failed", file=sys.stderr)
        return 1

    def ours():
        if args.tc_kernel == "auto" or args.precision == "fp32":
            return api.conv3x3(xc, wc, y, ws, N, C, H, W, K, precision=args.precision, variant=args.variant)
        err = api.filter_transform(wc, ws, C, K, precision=args.precision, variant=args.variant)
        return err or api.winograd_forward_kernel(xc, ws, y, N, C, H, W, K, precision=args.precision,
                                                  kernel=args.tc_kernel, variant=args.variant)

    err = ours()
    if err != 0:
        print(f"Error occurred: cudaError {err}", file=sys.stderr)
        return 1
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.iterations):
        ours()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.iterations
    flops = 2.0 * N * C * (H + 2) * (W + 2) * K * 9
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cudnn.benchmark = True
    ref = F.conv2d(x, w, padding=1)
    torch.cuda.synchronize()
    a.record()
    for _ in range(args.iterations):
        F.conv2d(x, w, padding=1)
    b.record()
    torch.cuda.synchronize()
    ms2 = a.elapsed_time(b) / args.iterations
    print(f"{N},{C},{H},{K},3,{ms:.3f},{flops / (2.25 * ms * 1e9):.2f},{ms2:.3f},{flops / (2.25 * ms2 * 1e9):.2f}")
    print("********************************************")
    out = torch.empty((N, K, H, W), device="cuda")
    api.khwn_to_nkhw(y, out, N, K, H, W, variant=args.variant)
    torch.cuda.synchronize()
    diff = (out - ref).abs()
    tol = {"fp32": 1e-4, "tf32": 4e-3, "bf16": 3e-2}[args.precision] * float(ref.abs().max())
    bad = int((diff > tol).sum())
    print(f"[max_error: {float(diff.max()):f}][error_cnt: {bad}] of {N * H * W * K}")
    return 0 if bad == 0 and api.last_device_status(args.variant) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
