"""Runs the shared-memory LDS / STS probes (csrc/smem_probe.cu) and prints the table that the
reference's bench/smem/{LDS,STS}/main.cu print for Turing: clocks per instruction and bytes per
clock, for plain, broadcast and conflicting patterns and for the access patterns this library's
kernels (and the reference's optSTS64 staging) actually use.

    python -m opencnn_b200.smem_probe
"""
import ctypes
import sys

from .build import build_smem_probe

OPS = ["LDS.32", "LDS.64", "LDS.128", "STS.32", "STS.64", "STS.128"]
WIDTH = [4, 8, 16, 4, 8, 16]
PATTERNS = ["contiguous", "same address", "stride 2 (2-way conflict)", "library STS.64 staging deposit",
            "reference optSTS64 deposit", "library main-loop image-pair load", "library main-loop filter load",
            "reference opt3 (256 B, lanes 8-15/16-23 swapped)", "reference sts64_2bank_conflict",
            "reference sts64_broadcast", "reference sts128, lanes with lane%16 <= 8"]
# which (op, pattern) pairs make sense
CASES = [(o, p) for o in range(6) for p in (0, 1, 2)] + [(4, 3), (4, 4), (2, 5), (2, 6), (1, 7), (4, 7), (4, 8), (4, 9),
                                                         (5, 10)]
# lanes that take part (for bytes per clock)
ACTIVE = {10: 18}


def measure(lib, op: int, pattern: int) -> float:
    """Clocks per warp instruction of one (instruction, pattern) pair."""
    out = ctypes.c_double(0.0)
    err = lib.opencnn_smem_probe(op, pattern, ctypes.byref(out))
    if err != 0:
        raise RuntimeError(f"opencnn_smem_probe({op}, {pattern}) returned cudaError {err}")
    return out.value


def load():
    lib = ctypes.CDLL(build_smem_probe())
    lib.opencnn_smem_probe.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    return lib


def main() -> int:
    lib = load()
    print(f"{'instruction':9s} {'pattern':48s} {'clk/instr':>10s} {'bytes/clk':>10s}")
    for op, pat in CASES:
        try:
            clk = measure(lib, op, pat)
        except RuntimeError as exc:
            print(exc, file=sys.stderr)
            return 1
        print(f"{OPS[op]:9s} {PATTERNS[pat]:48s} {clk:10.2f} {ACTIVE.get(pat, 32) * WIDTH[op] / clk:10.1f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
