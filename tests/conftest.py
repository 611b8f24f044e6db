import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


class Oracle:
    """ctypes view of oracle/liboracle.so (the CPU restatement; test infrastructure only)."""

    def __init__(self, path):
        L = ctypes.CDLL(path)
        f, d = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double)
        i64 = ctypes.POINTER(ctypes.c_int64)
        ci, u64 = ctypes.c_int, ctypes.c_uint64
        L.oc_fill_input_chwn.argtypes = [f, ci, ci, ci, ci, ctypes.c_long, u64]
        L.oc_fill_filter_crsk.argtypes = [f, ci, ci, ctypes.c_double, u64]
        L.oc_fill_input_int.argtypes = [f, ci, ci, ci, ci, u64]
        L.oc_fill_filter_int.argtypes = [f, ci, ci, u64]
        L.oc_direct_f64.argtypes = [f, f, d, ci, ci, ci, ci, ci]
        L.oc_direct_f64_sampled.argtypes = [f, f, i64, ctypes.c_int64, d, ci, ci, ci, ci, ci]
        L.oc_direct_f32_omp.argtypes = [f, f, f, ci, ci, ci, ci, ci]
        L.oc_filter_transform.argtypes = [f, f, ci, ci]
        L.oc_winograd_f32.argtypes = [f, f, f, ci, ci, ci, ci, ci]
        L.oc_convolution_forward.argtypes = [f, f, f, f, ci, ci, ci, ci, ci]
        L.oc_winograd_tc_model.argtypes = [f, f, f, ci, ci, ci, ci, ci, ci]
        L.oc_round_tf32.argtypes = [f, ctypes.c_size_t]
        L.oc_round_bf16.argtypes = [f, ctypes.c_size_t]
        L.oc_num_threads.restype = ci
        self.L = L

    @staticmethod
    def _p(a):
        t = {np.dtype(np.float32): ctypes.c_float, np.dtype(np.float64): ctypes.c_double,
             np.dtype(np.int64): ctypes.c_int64}[a.dtype]
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data_as(ctypes.POINTER(t))

    def input_chwn(self, N, C, H, W, seed=0, n_offset=0):
        x = np.empty((C, H, W, N), np.float32)
        self.L.oc_fill_input_chwn(self._p(x), N, C, H, W, n_offset, seed)
        return x

    def filter_crsk(self, C, K, sigma=0.05, seed=0):
        g = np.empty((C, 3, 3, K), np.float32)
        self.L.oc_fill_filter_crsk(self._p(g), C, K, sigma, seed)
        return g

    def input_int(self, N, C, H, W, seed=1):
        x = np.empty((C, H, W, N), np.float32)
        self.L.oc_fill_input_int(self._p(x), N, C, H, W, seed)
        return x

    def filter_int(self, C, K, seed=1):
        g = np.empty((C, 3, 3, K), np.float32)
        self.L.oc_fill_filter_int(self._p(g), C, K, seed)
        return g

    def direct_f64(self, x, g):
        C, H, W, N = x.shape
        K = g.shape[3]
        y = np.empty((K, H, W, N), np.float64)
        self.L.oc_direct_f64(self._p(x), self._p(g), self._p(y), N, C, K, H, W)
        return y

    def direct_f64_sampled(self, x, g, idx):
        C, H, W, N = x.shape
        K = g.shape[3]
        idx = np.ascontiguousarray(idx, np.int64)
        out = np.empty(idx.shape[0], np.float64)
        self.L.oc_direct_f64_sampled(self._p(x), self._p(g), self._p(idx), idx.shape[0], self._p(out), N, C, K, H, W)
        return out

    def direct_f32(self, x, g):
        C, H, W, N = x.shape
        K = g.shape[3]
        y = np.empty((K, H, W, N), np.float32)
        self.L.oc_direct_f32_omp(self._p(x), self._p(g), self._p(y), N, C, K, H, W)
        return y

    def filter_transform(self, g):
        C, _, _, K = g.shape
        U = np.empty((C, 4, 4, K), np.float32)
        self.L.oc_filter_transform(self._p(g), self._p(U), C, K)
        return U

    def winograd_f32(self, x, U):
        C, H, W, N = x.shape
        K = U.shape[3]
        y = np.empty((K, H, W, N), np.float32)
        self.L.oc_winograd_f32(self._p(x), self._p(U), self._p(y), N, C, K, H, W)
        return y

    def forward(self, x, g):
        return self.winograd_f32(x, self.filter_transform(g))

    def tc_model(self, x, g, precision):
        """Model of the tensor-core path (operands rounded after the fp32 transforms)."""
        C, H, W, N = x.shape
        K = g.shape[3]
        y = np.empty((K, H, W, N), np.float32)
        self.L.oc_winograd_tc_model(self._p(x), self._p(g), self._p(y), N, C, K, H, W, {"tf32": 1, "bf16": 2}[precision])
        return y

    def round_tf32(self, a):
        a = np.ascontiguousarray(a, np.float32).copy()
        self.L.oc_round_tf32(self._p(a), a.size)
        return a

    def round_bf16(self, a):
        a = np.ascontiguousarray(a, np.float32).copy()
        self.L.oc_round_bf16(self._p(a), a.size)
        return a


def _oracle_path():
    path = os.path.join(ROOT, "oracle", "liboracle.so")
    src = os.path.join(ROOT, "oracle", "oracle.c")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), path], check=True, capture_output=True)
    return path


@pytest.fixture(scope="session")
def oracle():
    return Oracle(_oracle_path())


@pytest.fixture(scope="session")
def libs():
    """Builds (if stale) and loads the four variant libraries."""
    from opencnn_b200 import _lib, build
    build.build_all()
    return {v: _lib.load(v) for v in build.VARIANTS}


class RefLib:
    """The reference's own kernels (oracle/_ref/libref_<VARIANT>.so), GPU only."""

    def __init__(self, path):
        L = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        L.ref_upload_tables.restype = ci
        L.ref_convolutionForward.restype = ci
        L.ref_convolutionForward.argtypes = [vp, ci, ci, vp, ci, ci, ci, ci, vp, vp, ctypes.c_uint] + [ci] * 11
        L.ref_time_calls.restype = ctypes.c_float
        L.ref_time_calls.argtypes = [vp, ci, vp, ci, ci, ci, vp, vp, ci]
        L.ref_variant_name.restype = ctypes.c_char_p
        self.L = L
        self._tables = False

    def forward(self, x, g, y, ws, N, C, HW, K):
        if not self._tables:
            assert self.L.ref_upload_tables() == 0
            self._tables = True
        td = (HW + 1) // 2
        return self.L.ref_convolutionForward(x.data_ptr(), HW, HW, g.data_ptr(), HW, HW, N, K, y.data_ptr(),
                                             ws.data_ptr(), 0, td, N, 4, td * 4, C, K, C, 3, 3, 4, 2)


def ref_lib_path(variant):
    return os.path.join(ROOT, "oracle", "_ref", f"libref_{variant}.so")


@pytest.fixture(scope="session")
def ref_libs():
    out = {}
    for v in ("BASE", "OPTSTS64", "OPTSTS64_CMP", "OPTLDS64"):
        p = ref_lib_path(v)
        if os.path.exists(p):
            out[v] = RefLib(p)
    return out


def wait_probe_lib_path():
    """Builds (if stale) the test-only bounded-wait probe, tests/wait_probe.cu."""
    here = os.path.dirname(os.path.abspath(__file__))
    src = os.path.join(here, "wait_probe.cu")
    out = os.path.join(here, "_build", "libwait_probe.so")
    deps = [src, os.path.join(ROOT, "opencnn_b200", "csrc", "ptx.cuh")]
    if not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps):
        from opencnn_b200 import build
        os.makedirs(os.path.dirname(out), exist_ok=True)
        subprocess.run([build.nvcc(), *build.ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
                        "-o", out, src], check=True, capture_output=True)
    return out
