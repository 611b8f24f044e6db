"""Builds the CUDA libraries in-tree: one shared object per output-staging variant.

    python -m opencnn_b200.build            # all four variants
    python -m opencnn_b200.build OPTSTS64   # one

The variant is a compile-time -D, as in the reference (Makefile:3,8): BASE, OPTSTS64 (default),
OPTSTS64_CMP, OPTLDS64.  Output: opencnn_b200/lib/libopencnn_b200_<VARIANT>.so.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

VARIANTS = ("BASE", "OPTSTS64", "OPTSTS64_CMP", "OPTLDS64")
HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def lib_path(variant: str) -> str:
    return os.path.join(LIBDIR, f"libopencnn_b200_{variant}.so")


def _sources() -> list[str]:
    out = []
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
    out.append(os.path.join(os.path.dirname(HERE), "include", "opencnn_b200.h"))
    return out


def _stale(target: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in _sources())


def nvcc() -> str:
    exe = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build the opencnn_b200 CUDA libraries")
    return exe


def build_variant(variant: str, force: bool = False, verbose: bool = False) -> str:
    if variant not in VARIANTS:
        raise ValueError(f"unknown variant {variant!r}; expected one of {VARIANTS}")
    os.makedirs(LIBDIR, exist_ok=True)
    target = lib_path(variant)
    if not force and not _stale(target):
        return target
    cmd = [nvcc(), *ARCH, "-O3", "-lineinfo", "-std=c++17", f"-D{variant}", "-Xcompiler", "-fPIC", "-shared",
           "-o", target, os.path.join(CSRC, "abi.cu")]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {variant}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return target


def peaks_lib_path() -> str:
    return os.path.join(LIBDIR, "libopencnn_b200_peaks.so")


def build_peaks(force: bool = False) -> str:
    """The FP32-pipe peak probe used by bench.py (csrc/peaks.cu); not part of the operator."""
    os.makedirs(LIBDIR, exist_ok=True)
    target, src = peaks_lib_path(), os.path.join(CSRC, "peaks.cu")
    if force or not os.path.exists(target) or os.path.getmtime(src) > os.path.getmtime(target):
        cmd = [nvcc(), *ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", target, src]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for peaks.cu:\n{res.stdout}\n{res.stderr}")
    return target


def smem_probe_lib_path() -> str:
    return os.path.join(LIBDIR, "libopencnn_b200_smem_probe.so")


def build_smem_probe(force: bool = False) -> str:
    """The LDS/STS issue-rate probes (csrc/smem_probe.cu); not part of the operator."""
    os.makedirs(LIBDIR, exist_ok=True)
    target, src = smem_probe_lib_path(), os.path.join(CSRC, "smem_probe.cu")
    if force or not os.path.exists(target) or os.path.getmtime(src) > os.path.getmtime(target):
        cmd = [nvcc(), *ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", target, src]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for smem_probe.cu:\n{res.stdout}\n{res.stderr}")
    return target


def cudnn_probe_path() -> str:
    return os.path.join(LIBDIR, "cudnn_probe")


def build_cudnn_probe(force: bool = False) -> str | None:
    """The cuDNN legacy-API timing program (csrc/cudnn_probe.cu), a baseline for bench.py; not part of
    the operator.  Returns None where cuDNN's headers or library are not installed."""
    os.makedirs(LIBDIR, exist_ok=True)
    target, src = cudnn_probe_path(), os.path.join(CSRC, "cudnn_probe.cu")
    if force or not os.path.exists(target) or os.path.getmtime(src) > os.path.getmtime(target):
        cmd = [nvcc(), *ARCH, "-O2", "-std=c++17", "-o", target, src, "-lcudnn"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            return None
    return target


def build_all(force: bool = False, verbose: bool = False) -> list[str]:
    with ThreadPoolExecutor(max_workers=6) as ex:
        peaks = ex.submit(build_peaks, force)
        probe = ex.submit(build_smem_probe, force)
        cudnn = ex.submit(build_cudnn_probe, force)
        libs = list(ex.map(lambda v: build_variant(v, force, verbose), VARIANTS))
        cudnn.result()                   # optional: absent where cuDNN is not installed
        return libs + [peaks.result(), probe.result()]


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("-")]
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    for v in (args or VARIANTS):
        print(build_variant(v, force=force, verbose=verbose))
