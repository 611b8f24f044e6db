"""The tcgen05 / TMEM path (TF32 and BF16 operands, fp32 accumulate) through the C ABI.

Two checks per case: (1) against the CPU model of exactly that computation (fp32 transforms,
operands rounded once, exact contraction) with a tight tolerance, which catches layout and
indexing errors; (2) against the fp64 direct convolution with the tolerance the arithmetic
allows, which is the accuracy claim of the path.  Inputs and filters are themselves rounded to
the operand type first (the tensor-core benchmark configuration prescribes operands rounded once
from the seeded fp32 tensors)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from opencnn_b200 import api  # noqa: E402

pytestmark = pytest.mark.gpu

# TF32 problems with >= 64 K-steps per tile (C >= 512) and >= 64 images take the CTA-pair kernel - the last five
# here, also with an odd number of 32-image blocks and with K not a multiple of 128; everything else, and all of
# BF16, the single-CTA kernel.
SHAPES = [(32, 16, 128, 8, 8), (32, 8, 64, 7, 7), (64, 40, 192, 5, 9), (32, 64, 64, 14, 14), (96, 32, 256, 6, 6),
          (64, 512, 128, 4, 4), (96, 512, 192, 3, 5), (128, 520, 64, 2, 2), (64, 1024, 128, 3, 3), (96, 1040, 192, 2, 3)]
MODEL_REL = 2e-4                     # device vs model: fp32 accumulation order inside the tensor core
TRUTH_REL = {"tf32": 4e-3, "bf16": 3e-2}   # device vs fp64 truth, relative to rms(truth)


def run_tc(x, g, precision):
    C, H, W, N = x.shape
    K = g.shape[3]
    dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    dy = torch.full((K, H, W, N), float("nan"), device="cuda")
    dws = torch.empty((C, 4, 4, K), device="cuda")
    err = api.conv3x3(dx, dg, dy, dws, N, C, H, W, K, precision=precision,
                      stream=torch.cuda.current_stream().cuda_stream)
    assert err == 0, f"cudaError {err}"
    assert api.last_device_status() == 0
    return dy.cpu().numpy()


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
@pytest.mark.parametrize("shape", SHAPES)
def test_tensor_core_path(oracle, libs, precision, shape):
    N, C, K, H, W = shape
    rnd = oracle.round_tf32 if precision == "tf32" else oracle.round_bf16
    x = rnd(oracle.input_chwn(N, C, H, W)).reshape(C, H, W, N)
    g = rnd(oracle.filter_crsk(C, K)).reshape(C, 3, 3, K)
    y = run_tc(x, g, precision)
    assert np.isfinite(y).all()
    model = oracle.tc_model(x, g, precision)
    rms = float(np.sqrt(np.mean(model.astype(np.float64) ** 2)))
    worst = float(np.abs(y - model).max())
    assert worst <= MODEL_REL * max(rms, 1e-30), f"vs model: {worst / rms:.3e} of rms"
    truth = oracle.direct_f64(x, g)
    trms = float(np.sqrt(np.mean(truth ** 2)))
    tworst = float(np.abs(y - truth).max())
    assert tworst <= TRUTH_REL[precision] * trms, f"vs fp64: {tworst / trms:.3e} of rms"


# Ragged last image block (N % 8 == 0 on this path), single-CTA kernel and CTA-pair kernel (TF32, >= 64 K-steps, N >= 64).
RAGGED = [(40, 16, 128, 6, 6), (72, 32, 64, 5, 7), (8, 16, 128, 4, 4), (72, 512, 128, 4, 4), (104, 512, 128, 3, 3),
          (72, 1024, 128, 2, 2),
          (32, 3, 64, 6, 6), (40, 21, 128, 5, 5), (64, 515, 128, 3, 3)]   # and channel counts that are not a multiple of 8


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
@pytest.mark.parametrize("shape", RAGGED)
def test_ragged_batch_on_tensor_cores(oracle, libs, precision, shape):
    N, C, K, H, W = shape
    rnd = oracle.round_tf32 if precision == "tf32" else oracle.round_bf16
    x = rnd(oracle.input_chwn(N, C, H, W)).reshape(C, H, W, N)
    g = rnd(oracle.filter_crsk(C, K)).reshape(C, 3, 3, K)
    y = run_tc(x, g, precision)
    assert np.isfinite(y).all()
    model = oracle.tc_model(x, g, precision)
    rms = float(np.sqrt(np.mean(model.astype(np.float64) ** 2)))
    worst = float(np.abs(y - model).max())
    assert worst <= MODEL_REL * max(rms, 1e-30), f"vs model: {worst / rms:.3e} of rms"
    dx = torch.zeros((C, H, W, N + 4), device="cuda")
    assert api.conv3x3(dx, torch.from_numpy(g).cuda(), torch.empty((K, H, W, N + 4), device="cuda"),
                       torch.empty((C, 4, 4, K), device="cuda"), N + 4, C, H, W, K, precision=precision) != 0, \
        "N % 8 != 0 must be refused on the tensor-core path"


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
def test_integer_tensors_are_exact_on_tensor_cores(oracle, libs, precision):
    """Small integers are exact in both operand types and in the fp32 accumulator."""
    N, C, K, H, W = 32, 16, 128, 6, 6
    x, g = oracle.input_int(N, C, H, W), oracle.filter_int(C, K)
    y = run_tc(x, g, precision)
    assert np.array_equal(y.astype(np.float64), oracle.direct_f64(x, g))


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
def test_tensor_core_results_are_repeatable(libs, precision):
    """Same bits run after run, also from the CTA-pair kernel that deep TF32 problems take (its two partial
    results are added by an L2 reduction, but two addends commute)."""
    for (N, C, K, H, W) in [(64, 64, 64, 9, 9), (64, 1024, 128, 3, 3)]:
        x = torch.rand((C, H, W, N), device="cuda") * 2 - 1
        g = torch.randn((C, 3, 3, K), device="cuda") * 0.05
        ws = torch.empty((C, 4, 4, K), device="cuda")
        first = torch.empty((K, H, W, N), device="cuda")
        again = torch.empty_like(first)
        assert api.conv3x3(x, g, first, ws, N, C, H, W, K, precision=precision) == 0
        for _ in range(3):
            assert api.conv3x3(x, g, again, ws, N, C, H, W, K, precision=precision) == 0
            torch.cuda.synchronize()
            assert torch.equal(first, again)
    assert api.last_device_status() == 0


# The benchmark shapes at full size (the N=128 layer sweep and the two wide stress layers): error of both
# operand types against 10^5 sampled fp64 outputs, relative to rms(truth).  The N=64 C=K=1024 layer takes the
# CTA-pair kernel in TF32.
FULL = [(128, 64, 64, 56), (128, 128, 128, 28), (128, 256, 256, 14), (128, 512, 512, 7), (64, 1024, 1024, 14),
        (256, 32, 64, 112)]


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
@pytest.mark.parametrize("shape", FULL)
def test_tensor_core_error_at_benchmark_sizes(oracle, libs, precision, shape):
    N, C, K, HW = shape
    rnd = oracle.round_tf32 if precision == "tf32" else oracle.round_bf16
    x = rnd(oracle.input_chwn(N, C, HW, HW)).reshape(C, HW, HW, N)
    g = rnd(oracle.filter_crsk(C, K)).reshape(C, 3, 3, K)
    dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    dy = torch.full((K, HW, HW, N), float("nan"), device="cuda")
    dws = torch.empty((C, 4, 4, K), device="cuda")
    assert api.conv3x3(dx, dg, dy, dws, N, C, HW, HW, K, precision=precision) == 0
    assert api.last_device_status() == 0
    assert bool(torch.isfinite(dy).all().item()), "an output was not written"
    idx = np.random.default_rng(11).integers(0, dy.numel(), 100000)
    truth = oracle.direct_f64_sampled(x, g, idx)
    got = dy.view(-1)[torch.from_numpy(idx).cuda()].cpu().numpy()
    trms = float(np.sqrt(np.mean(truth ** 2)))
    worst = float(np.abs(got - truth).max())
    assert worst <= TRUTH_REL[precision] * trms, f"vs fp64: {worst / trms:.3e} of rms"
    # a second run gives the same bits
    dy2 = torch.empty_like(dy)
    assert api.conv3x3(dx, dg, dy2, dws, N, C, HW, HW, K, precision=precision) == 0
    torch.cuda.synchronize()
    assert torch.equal(dy, dy2)


# Every tensor-core kernel on its own, chosen by the caller (opencnn_winograd_forward_kernel), whatever the
# library's own rule would take: small and deep problems, an odd number of 32-image blocks, a ragged last block,
# K not a multiple of 128, channel counts that are not a multiple of the K-step.
KERNEL_SHAPES = [(32, 16, 128, 8, 8), (64, 40, 192, 5, 9), (96, 32, 256, 6, 6), (64, 512, 128, 4, 4), (128, 64, 64, 14, 14),
                 (72, 48, 64, 5, 7), (104, 515, 128, 3, 3), (8, 16, 128, 4, 4), (160, 24, 320, 7, 7)]


@pytest.mark.parametrize("kernel", ["single", "pair_local"])
@pytest.mark.parametrize("precision", ["tf32", "bf16"])
def test_each_tensor_core_kernel(oracle, libs, precision, kernel):
    rnd = oracle.round_tf32 if precision == "tf32" else oracle.round_bf16
    for (N, C, K, H, W) in KERNEL_SHAPES:
        x = rnd(oracle.input_chwn(N, C, H, W)).reshape(C, H, W, N)
        g = rnd(oracle.filter_crsk(C, K)).reshape(C, 3, 3, K)
        dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
        dws = torch.empty((C, 4, 4, K), device="cuda")
        assert api.filter_transform(dg, dws, C, K, precision=precision) == 0
        outs = []
        for _ in range(2):
            dy = torch.full((K, H, W, N), float("nan"), device="cuda")
            assert api.winograd_forward_kernel(dx, dws, dy, N, C, H, W, K, precision=precision, kernel=kernel) == 0
            assert api.last_device_status() == 0, (kernel, precision, (N, C, K, H, W))
            outs.append(dy)
        assert torch.equal(outs[0], outs[1]), "not repeatable"
        y = outs[0].cpu().numpy()
        assert np.isfinite(y).all(), (kernel, precision, (N, C, K, H, W))
        model = oracle.tc_model(x, g, precision)
        rms = float(np.sqrt(np.mean(model.astype(np.float64) ** 2)))
        worst = float(np.abs(y - model).max())
        assert worst <= MODEL_REL * max(rms, 1e-30), f"{kernel} {precision} {(N, C, K, H, W)}: {worst / rms:.3e} of rms"
    bad = torch.zeros(16, device="cuda")
    assert api.winograd_forward_kernel(bad, bad, bad, 32, 8, 4, 4, 64, precision="fp32", kernel=kernel) != 0


# The stacked-blocks kernel (at most 64 filters): even and odd numbers of 32-image blocks, a ragged last block,
# channel counts that are not a multiple of the K-step, one K-step and many, more tiles than SMs (so that both
# stages of the filter ring are reused).
STACKED_SHAPES = [(64, 16, 64, 8, 8), (96, 40, 64, 5, 9), (128, 64, 64, 14, 14), (72, 3, 64, 6, 6), (32, 32, 64, 7, 7),
                  (200, 72, 64, 3, 5), (256, 32, 64, 12, 12), (256, 32, 64, 30, 30)]


@pytest.mark.parametrize("precision", ["tf32", "bf16"])
def test_stacked_blocks_kernel(oracle, libs, precision):
    rnd = oracle.round_tf32 if precision == "tf32" else oracle.round_bf16
    for (N, C, K, H, W) in STACKED_SHAPES:
        x = rnd(oracle.input_chwn(N, C, H, W)).reshape(C, H, W, N)
        g = rnd(oracle.filter_crsk(C, K)).reshape(C, 3, 3, K)
        dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
        dws = torch.empty((C, 4, 4, K), device="cuda")
        assert api.filter_transform(dg, dws, C, K, precision=precision) == 0
        outs = []
        for _ in range(2):
            dy = torch.full((K, H, W, N), float("nan"), device="cuda")
            assert api.winograd_forward_kernel(dx, dws, dy, N, C, H, W, K, precision=precision, kernel="stacked") == 0
            assert api.last_device_status() == 0, (N, C, K, H, W)
            outs.append(dy)
        assert torch.equal(outs[0], outs[1]), "not repeatable"
        # the single-CTA kernel issues the same products in the same order: the two must agree bit for bit
        single = torch.full((K, H, W, N), float("nan"), device="cuda")
        assert api.winograd_forward_kernel(dx, dws, single, N, C, H, W, K, precision=precision, kernel="single") == 0
        assert torch.equal(outs[0], single), (N, C, K, H, W)
        y = outs[0].cpu().numpy()
        assert np.isfinite(y).all(), (N, C, K, H, W)
        model = oracle.tc_model(x, g, precision)
        rms = float(np.sqrt(np.mean(model.astype(np.float64) ** 2)))
        worst = float(np.abs(y - model).max())
        assert worst <= MODEL_REL * max(rms, 1e-30), f"{(N, C, K, H, W)}: {worst / rms:.3e} of rms"
    # refused: more than 64 filters
    z = torch.zeros(1 << 16, device="cuda")
    assert api.winograd_forward_kernel(z, z, z, 64, 16, 4, 4, 128, precision=precision, kernel="stacked") != 0
