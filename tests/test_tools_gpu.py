"""The two measurement tools either side of the operator, run on the GPU: the shared-memory
LDS / STS probes (counterpart of the reference's bench/smem microbenchmarks) and the command line
compatible with the reference's `wgrad` binary (argv src/openCNN_winograd.cu:246-255, CSV line
:257, header bench/bench.sh:1)."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")

from opencnn_b200 import smem_probe  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LDS32, LDS64, LDS128, STS32, STS64, STS128 = range(6)


def test_smem_probe_conflict_free_patterns_sit_at_the_floor_and_conflicts_cost_double():
    lib = smem_probe.load()
    t = {case: smem_probe.measure(lib, *case) for case in smem_probe.CASES}
    floor = t[(LDS32, 0)]                          # what a lone warp can issue at all
    assert 3.0 < floor < 8.0
    # 32- and 64-bit loads without conflicts: at the issue floor
    for case in [(LDS32, 1), (LDS64, 0), (LDS64, 1), (STS32, 0)]:
        assert t[case] <= 1.15 * floor, (case, t[case], floor)
    # conflict-free 64-bit stores: one rate for contiguous, this library's deposit and the reference's
    # optSTS64 deposit
    for case in [(STS64, 3), (STS64, 4)]:
        assert abs(t[case] - t[(STS64, 0)]) <= 0.1 * t[(STS64, 0)], (case, t[case], t[(STS64, 0)])
    # the reference's opt3 permutation (its optLDS64 read-back): 256 contiguous bytes, so at best conflict-free;
    # if the hardware serves 64-bit accesses strictly per half-warp it is a two-way conflict - never worse
    assert 0.9 * t[(LDS64, 0)] <= t[(LDS64, 7)] <= 1.15 * t[(LDS64, 2)]
    assert 0.9 * t[(STS64, 0)] <= t[(STS64, 7)] <= 1.15 * t[(STS64, 2)]
    # this library's broadcast-heavy main-loop loads cost no more than a same-address LDS.128
    for case in [(LDS128, 5), (LDS128, 6)]:
        assert t[case] <= 1.1 * t[(LDS128, 1)], (case, t[case])
    # two-way conflicts: twice the data cycles of the conflict-free access of the same width (a 64-bit warp
    # access is 2 data cycles, 4 with the conflict; the issue floor hides part of it, so compare with 128-bit)
    assert 0.85 * t[(LDS128, 0)] <= t[(LDS64, 2)] <= 1.15 * t[(LDS128, 0)]
    assert 0.85 * t[(LDS128, 0)] <= t[(STS64, 2)] <= 1.15 * t[(LDS128, 0)]
    assert 0.85 * t[(STS64, 2)] <= t[(STS64, 8)] <= 1.15 * t[(STS64, 2)], "the reference's 2-way pattern"
    assert 1.8 <= t[(LDS128, 2)] / t[(LDS128, 0)] <= 2.2
    assert t[(STS64, 8)] >= 1.25 * t[(STS64, 0)]
    # same-address stores are not slower than contiguous ones; 18 active lanes of STS.128 not slower than 32
    assert t[(STS64, 9)] <= 1.1 * t[(STS64, 0)]
    assert t[(STS128, 10)] <= 1.1 * t[(STS128, 0)]


def test_wgrad_command_line_prints_the_reference_csv():
    cmd = [sys.executable, "-m", "opencnn_b200.wgrad", "32", "64", "56", "56", "64", "64", "3", "3", "--header",
           "--iterations", "20"]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = res.stdout.strip().splitlines()
    assert lines[0] == "in_n,in_c,in_h,filt_k,filt_w,openCNN_sec,openCNN_flops,cuDNN_sec,cuDNN_flops"
    cols = lines[1].split(",")
    assert len(cols) == 9 and cols[:5] == ["32", "64", "56", "64", "3"]
    ms, tf, ms2, tf2 = (float(c) for c in cols[5:])
    assert 0 < ms < 100 and 0 < ms2 < 100 and tf > 0 and tf2 > 0
    assert "[error_cnt: 0]" in lines[-1]
    # a configuration outside the operator's domain is refused like the reference does (exit code 1, message)
    bad = subprocess.run([sys.executable, "-m", "opencnn_b200.wgrad", "32", "64", "56", "56", "64", "64", "5", "5"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "not supported" in bad.stderr


def test_peak_probes_relations():
    """The measurement aids of csrc/peaks.cu: moves mixed into a packed-FMA stream are free, scalar adds are not;
    a second TMA load in flight nearly halves the time per load."""
    from opencnn_b200 import peaks
    lib = peaks.load()
    t = peaks.issue_probe(lib, iters=5000)
    plain = t[(0, 0)]
    assert t[(16, 1)] <= 1.05 * plain and t[(32, 0)] <= 1.06 * plain, t
    assert t[(32, 2)] >= 1.10 * plain, t
    assert t[(64, 0)] >= 1.3 * plain, t
    lat = peaks.tma_latency(lib, grid=8, iters=200)
    for b in (65536, 32768):
        assert 300 < lat[(b, 1, 1)] < 5000, lat
        assert lat[(b, 1, 2)] <= 0.75 * lat[(b, 1, 1)], lat


def test_mma_rate_probe_is_sane():
    """The tcgen05.mma issue-rate probe: a chain of MMAs can never beat the tensor pipe (4096 BF16 / 2048 TF32
    multiply-adds per clock and SM), and a wider MMA takes longer than a narrow one."""
    from opencnn_b200 import peaks
    lib = peaks.load()
    r = peaks.mma_rate(lib, grid=8, iters=500)
    for (kind, n, layout, issuers), cyc in r.items():
        macs = 128 * n * (16 if kind == 0 else 8)
        assert 1.0 < cyc < 5000.0, r
        assert macs / cyc <= 1.05 * (4096 if kind == 0 else 2048), ((kind, n, layout, issuers), cyc)
    for kind in (0, 1):
        for layout in range(4):
            assert r[(kind, 256, layout, 1)] > r[(kind, 32, layout, 1)], r
    trip = peaks.mma_round_trip(lib, grid=8, iters=300)
    for (kind, issuers), cyc in trip.items():
        # a group that is committed and waited for cannot be faster than its MMAs in the pipe
        assert cyc >= 0.95 * (16 // issuers) * r[(kind, 32, 0, 1 if issuers == 1 else issuers)] and cyc < 20000.0, trip
