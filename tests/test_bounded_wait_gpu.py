"""The give-up path of the kernels' bounded waits (opencnn_b200/csrc/ptx.cuh), which a healthy run
never takes: a test-only kernel (tests/wait_probe.cu) waits on an mbarrier on which, by a host flag,
nobody arrives.  The wait must run out after its limit, set the status word, let the other waiter
of the CTA fall through, and the kernel must return with the context intact - checked by running
the real operator afterwards and comparing it with the oracle bit for bit."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from conftest import wait_probe_lib_path  # noqa: E402
from opencnn_b200 import api  # noqa: E402

pytestmark = pytest.mark.gpu
LIMIT_NS = 2_000_000          # 2 ms per wait


@pytest.fixture(scope="module")
def probe():
    lib = ctypes.CDLL(wait_probe_lib_path())
    lib.wait_probe_run.argtypes = [ctypes.c_int, ctypes.c_ulonglong, ctypes.POINTER(ctypes.c_longlong)]
    lib.wait_probe_last_status.restype = ctypes.c_int
    return lib


def _run(lib, skip_arrive):
    out = (ctypes.c_longlong * 8)()
    assert lib.wait_probe_run(int(skip_arrive), LIMIT_NS, out) == 0
    keys = ("issuer_ok", "waiter_ok", "waiter_second_ok", "drain_ok", "drain_timeout_ok", "issuer_wait_ns",
            "waiter_second_ns", "drain_timeout_ns")
    return dict(zip(keys, list(out)))


def test_healthy_wait_leaves_status_clear(probe):
    r = _run(probe, skip_arrive=False)
    assert r["issuer_ok"] == 1 and r["waiter_ok"] == 1
    assert r["drain_ok"] == 1
    assert r["drain_timeout_ok"] == 1 and r["drain_timeout_ns"] >= LIMIT_NS       # the drain's own limit
    assert probe.wait_probe_last_status() == 0


def test_wait_that_runs_out_sets_status_and_returns(oracle, libs, probe):
    r = _run(probe, skip_arrive=True)
    assert r["issuer_ok"] == 0, "nobody arrived: the wait must give up"
    assert LIMIT_NS <= r["issuer_wait_ns"] < 50 * LIMIT_NS
    assert r["waiter_ok"] == 0, "the second waiter must come back through the CTA's dead word"
    assert r["waiter_second_ok"] == 0 and r["waiter_second_ns"] < LIMIT_NS, "later waits return at once"
    assert r["drain_ok"] == 1 and r["drain_timeout_ok"] == 1
    assert probe.wait_probe_last_status() == 1          # kStatusWaitTimeout
    assert probe.wait_probe_last_status() == 0          # reading resets it
    # the context is intact: the operator runs and is bit-exact
    N, C, K, H, W = 32, 16, 64, 6, 6
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    dy = torch.full((K, H, W, N), float("nan"), device="cuda")
    dws = torch.empty((C, 4, 4, K), device="cuda")
    assert api.conv3x3(torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda(), dy, dws, N, C, H, W, K) == 0
    assert api.last_device_status() == 0
    assert np.array_equal(dy.cpu().numpy(), oracle.forward(x, g))
