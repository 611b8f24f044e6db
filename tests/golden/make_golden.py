"""Generates the golden fixtures ref_*.npz from the REFERENCE's own kernels.

Run on a machine with a B200 and with oracle/_ref/libref_<VARIANT>.so present (built by
oracle/Makefile from the reference checkout):

    python tests/golden/make_golden.py [output_dir]

For each small case it uploads seeded tensors, runs the reference operator (filter transform FX
+ Winograd_kernel) in all four staging variants, checks that the variants agree bit for bit,
and stores input, filter, the transformed-filter workspace and the output.  The fixtures pin the
CPU oracle (tests/test_oracle_cpu.py) to the real reference.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from conftest import Oracle, RefLib, _oracle_path, ref_lib_path  # noqa: E402

# name, N, C, K, H=W, kind.  The reference supports square images only.
CASES = [("u_n32_c8_k64_w7", 32, 8, 64, 7, "uniform"),      # minimum tile sizes, odd width
         ("u_n32_c16_k64_w8", 32, 16, 64, 8, "uniform"),
         ("u_n64_c8_k128_w6", 64, 8, 128, 6, "uniform"),    # two image blocks, two filter blocks
         ("i_n32_c8_k64_w5", 32, 8, 64, 5, "int")]


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden")
    os.makedirs(out_dir, exist_ok=True)
    oracle = Oracle(_oracle_path())
    refs = {v: RefLib(ref_lib_path(v)) for v in ("BASE", "OPTSTS64", "OPTSTS64_CMP", "OPTLDS64")}
    for name, N, C, K, HW, kind in CASES:
        if kind == "int":
            x, g = oracle.input_int(N, C, HW, HW), oracle.filter_int(C, K)
        else:
            x, g = oracle.input_chwn(N, C, HW, HW), oracle.filter_crsk(C, K)
        dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
        outs, wss = {}, {}
        for v, ref in refs.items():
            dy = torch.full((K, HW, HW, N), float("nan"), device="cuda")
            dws = torch.zeros((C, 4, 4, K), device="cuda")
            err = ref.forward(dx, dg, dy, dws, N, C, HW, K)
            torch.cuda.synchronize()
            assert err == 0, (v, err)
            outs[v], wss[v] = dy.cpu().numpy(), dws.cpu().numpy()
        base = outs["OPTSTS64"]
        for v in refs:
            same = np.array_equal(outs[v], base) and np.array_equal(wss[v], wss["OPTSTS64"])
            print(f"{name}: {v} identical to OPTSTS64: {same}")
            assert same
        truth = oracle.direct_f64(x, g)
        print(f"{name}: reference max |err| vs fp64 direct = {np.abs(base - truth).max():.3e}; "
              f"oracle bit-exact: {np.array_equal(oracle.forward(x, g), base)}")
        np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"), input_chwn=x, filter_crsk=g,
                            workspace=wss["OPTSTS64"], output_khwn=base,
                            shape=np.array([N, C, K, HW, HW], np.int32))


if __name__ == "__main__":
    main()
