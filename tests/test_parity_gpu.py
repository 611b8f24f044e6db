"""Parity of the CUDA path, called through the C ABI, against the CPU oracle, the fp64 ground
truth, the golden fixtures and (when built) the reference's own kernels on the same device."""
import glob
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from opencnn_b200 import api, build  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# N, C, K, H, W: minimum tile sizes, odd and even extents, 1x1, rectangles, several blocks.
SMALL = [(32, 8, 64, 7, 7), (32, 16, 64, 8, 8), (64, 8, 128, 6, 6), (32, 8, 64, 1, 1), (32, 24, 64, 5, 9),
         (96, 8, 64, 3, 3), (32, 40, 192, 4, 2)]
REL = 1e-4   # the fp32 path's tolerance: |a - r| <= REL * max(|r|, floor)


def run(variant, x, g, via="legacy"):
    C, H, W, N = x.shape
    K = g.shape[3]
    dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    dy = torch.full((K, H, W, N), float("nan"), device="cuda")
    dws = torch.full((C, 4, 4, K), float("nan"), device="cuda")
    if via == "legacy":
        err = api.call_like_reference(dx, dg, dy, dws, N, C, H, W, K, variant=variant)
    else:
        err = api.conv3x3(dx, dg, dy, dws, N, C, H, W, K, stream=torch.cuda.current_stream().cuda_stream,
                          variant=variant)
    assert err == 0, f"cudaError {err}"
    assert api.last_device_status(variant) == 0
    return dy.cpu().numpy(), dws.cpu().numpy()


def within(y, truth, rel=REL, floor_frac=1.0):
    """|y - truth| <= rel * max(|truth|, floor_frac * rms(truth)) everywhere.

    Against the fp64 ground truth the floor is rms(truth): every output is a sum of 9*C products
    whose rounding noise scales with the size of the terms, not with the (possibly cancelled)
    result, and the reference's own kernels carry exactly the same noise.  Against the reference
    itself the floor is 1% of the rms, and the results are in fact bit-identical."""
    tau = floor_frac * float(np.sqrt(np.mean(truth.astype(np.float64) ** 2)))
    return bool(np.all(np.abs(y - truth) <= rel * np.maximum(np.abs(truth), tau)))


@pytest.mark.parametrize("variant", build.VARIANTS)
@pytest.mark.parametrize("shape", SMALL)
def test_matches_oracle_bit_for_bit(oracle, libs, variant, shape):
    N, C, K, H, W = shape
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    via = "legacy" if H == W else "stream"          # the legacy entry keeps the reference's tiles_dim argument
    y, ws = run(variant, x, g, via)
    assert np.array_equal(ws, oracle.filter_transform(g)), "filter transform"
    expect = oracle.forward(x, g)
    assert within(y, oracle.direct_f64(x, g)), "fp64 ground truth, 1e-4 relative"
    assert np.array_equal(y, expect), f"max |diff| {np.abs(y - expect).max()}"


# Batches that are not a multiple of 32 (an extension over the reference, which needs N % 32 == 0): the last
# image block is ragged.  Accepted by the opencnn_* entries for N % 4 == 0; the legacy entries still refuse.
RAGGED = [(36, 8, 64, 5, 5), (44, 16, 64, 6, 4), (100, 8, 128, 3, 3), (4, 8, 64, 4, 4), (60, 8, 64, 7, 7)]


@pytest.mark.parametrize("variant", build.VARIANTS)
@pytest.mark.parametrize("shape", RAGGED)
def test_ragged_batch_bit_for_bit(oracle, libs, variant, shape):
    N, C, K, H, W = shape
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    guard = 4096                                    # floats after the output that must stay untouched
    flat = torch.full((K * H * W * N + guard,), float("nan"), device="cuda")
    dy = flat[:K * H * W * N].view(K, H, W, N)
    dws = torch.empty((C, 4, 4, K), device="cuda")
    assert api.call_like_reference(dx, dg, dy, dws, N, C, H, W, K, variant=variant) != 0 or H != W, \
        "the legacy entry keeps N % 32 == 0"
    err = api.conv3x3(dx, dg, dy, dws, N, C, H, W, K, stream=torch.cuda.current_stream().cuda_stream, variant=variant)
    assert err == 0, f"cudaError {err}"
    assert api.last_device_status(variant) == 0
    got = flat.cpu().numpy()
    assert np.isnan(got[K * H * W * N:]).all(), "wrote past the end of the output"
    y = got[:K * H * W * N].reshape(K, H, W, N)
    expect = oracle.forward(x, g)
    assert np.array_equal(y, expect), f"max |diff| {np.nanmax(np.abs(y - expect))}"
    assert api.conv3x3(dx, dg, dy, dws, N + 2, C, H, W, K, variant=variant) != 0, "N % 4 != 0 must be refused"


# Channel counts that are not a multiple of 8 (e.g. the 3 channels of a first layer) and filter counts that are
# not a multiple of 64 (fp32 path: K % 4 == 0): further extensions over the reference.
ODD_CHANNELS = [(32, 3, 64, 8, 8), (32, 1, 64, 5, 5), (64, 12, 64, 7, 7), (36, 19, 128, 4, 6),
                (32, 8, 96, 6, 6), (32, 16, 4, 5, 5), (64, 8, 132, 3, 3), (44, 5, 68, 4, 4)]


@pytest.mark.parametrize("variant", build.VARIANTS)
@pytest.mark.parametrize("shape", ODD_CHANNELS)
def test_any_channel_count_bit_for_bit(oracle, libs, variant, shape):
    N, C, K, H, W = shape
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    dy = torch.full((K, H, W, N), float("nan"), device="cuda")
    dws = torch.full((C, 4, 4, K), float("nan"), device="cuda")
    if H == W and N % 32 == 0:
        assert api.call_like_reference(dx, dg, dy, dws, N, C, H, W, K, variant=variant) != 0, \
            "the legacy entry keeps C % 8 == 0"
    err = api.conv3x3(dx, dg, dy, dws, N, C, H, W, K, stream=torch.cuda.current_stream().cuda_stream, variant=variant)
    assert err == 0, f"cudaError {err}"
    assert api.last_device_status(variant) == 0
    assert np.array_equal(dws.cpu().numpy(), oracle.filter_transform(g)), "filter transform"
    y, expect = dy.cpu().numpy(), oracle.forward(x, g)
    assert within(y, oracle.direct_f64(x, g)), "fp64 ground truth, 1e-4 relative"
    assert np.array_equal(y, expect), f"max |diff| {np.nanmax(np.abs(y - expect))}"
    if K % 64:
        assert api.conv3x3(dx, dg, dy, dws, N, C, H, W, K, precision="tf32", variant=variant) != 0 or N % 8, \
            "the tensor-core path keeps K % 64 == 0"


@pytest.mark.parametrize("variant", build.VARIANTS)
def test_integer_known_answers_are_exact(oracle, libs, variant):
    for N, C, K, H, W in [(32, 8, 64, 5, 5), (64, 16, 64, 8, 8)]:
        x, g = oracle.input_int(N, C, H, W), oracle.filter_int(C, K)
        y, _ = run(variant, x, g)
        assert np.array_equal(y.astype(np.float64), oracle.direct_f64(x, g))


@pytest.mark.parametrize("variant", build.VARIANTS)
def test_golden_fixtures(libs, variant):
    files = sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz")))
    assert files
    for path in files:
        z = np.load(path)
        y, ws = run(variant, z["input_chwn"], z["filter_crsk"])
        assert np.array_equal(ws, z["workspace"]) and np.array_equal(y, z["output_khwn"]), path


@pytest.mark.parametrize("variant", build.VARIANTS)
def test_matches_reference_kernels_on_device(oracle, libs, ref_libs, variant):
    """Same seeded tensors through the reference's own kernels (same staging variant) and ours."""
    if variant not in ref_libs:
        pytest.skip("oracle/_ref not built")
    for N, C, K, HW in [(32, 8, 64, 7), (64, 64, 64, 14), (32, 128, 128, 28)]:
        x, g = oracle.input_chwn(N, C, HW, HW), oracle.filter_crsk(C, K)
        dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
        ry = torch.full((K, HW, HW, N), float("nan"), device="cuda")
        rws = torch.zeros((C, 4, 4, K), device="cuda")
        assert ref_libs[variant].forward(dx, dg, ry, rws, N, C, HW, K) == 0
        torch.cuda.synchronize()
        y, ws = run(variant, x, g)
        r = ry.cpu().numpy()
        assert within(y, r, floor_frac=1e-2), "1e-4 relative against the reference"
        assert np.array_equal(ws, rws.cpu().numpy())
        assert np.array_equal(y, r), f"not bit-identical: max |diff| {np.abs(y - r).max()}"


def test_full_size_first_config(oracle, libs):
    """N=32, C=64, K=64, 56x56 (the reference bench's first shape): all variants agree, the result
    is within tolerance of fp64 on 10^5 sampled outputs, equals the oracle, and is homogeneous
    under an exact power-of-two scaling of the input."""
    N, C, K, H, W = 32, 64, 64, 56, 56
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    outs = {v: run(v, x, g)[0] for v in build.VARIANTS}
    base = outs["OPTSTS64"]
    for v in build.VARIANTS:
        assert np.array_equal(outs[v], base), v
    idx = np.random.default_rng(0).integers(0, base.size, 100000)
    truth = oracle.direct_f64_sampled(x, g, idx)
    assert within(base.ravel()[idx], truth)
    assert np.array_equal(base, oracle.forward(x, g))
    y4, _ = run("OPTSTS64", x * np.float32(4.0), g)
    assert np.array_equal(y4, base * np.float32(4.0))


def test_layer_sweep_shapes_sampled(oracle, libs):
    """The N=128 ResNet-style layers: sampled fp64 check and agreement between two variants."""
    for N, C, K, HW in [(128, 128, 128, 28), (128, 256, 256, 14), (128, 512, 512, 7)]:
        x, g = oracle.input_chwn(N, C, HW, HW), oracle.filter_crsk(C, K)
        a, _ = run("OPTSTS64", x, g)
        b, _ = run("OPTLDS64", x, g)
        assert np.array_equal(a, b)
        idx = np.random.default_rng(1).integers(0, a.size, 100000)
        assert within(a.ravel()[idx], oracle.direct_f64_sampled(x, g, idx))


def test_split_entries_and_repeat_calls(oracle, libs):
    """Filter transform once, fused kernel twice on a side stream: same result as the one-call entry."""
    N, C, K, H, W = 64, 32, 128, 10, 10
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    expect, _ = run("OPTSTS64", x, g)
    s = torch.cuda.Stream()
    dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    dws = torch.empty((C, 4, 4, K), device="cuda")
    dy = torch.empty((K, H, W, N), device="cuda")
    torch.cuda.synchronize()
    assert api.filter_transform(dg, dws, C, K, stream=s.cuda_stream) == 0
    for _ in range(2):
        dy.fill_(float("nan"))
        torch.cuda.synchronize()
        assert api.winograd_forward(dx, dws, dy, N, C, H, W, K, stream=s.cuda_stream) == 0
        s.synchronize()
        assert np.array_equal(dy.cpu().numpy(), expect)


def test_host_buffer_plan(oracle, libs):
    N, C, K, H, W = 32, 16, 64, 12, 12
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    hx, hg = torch.from_numpy(x).pin_memory(), torch.from_numpy(g).pin_memory()
    hy = torch.empty((K, H, W, N)).pin_memory()
    plan = api.HostPlan(N, C, H, W, K)
    for _ in range(2):
        hy.fill_(float("nan"))
        assert plan.run(hx.data_ptr(), hg.data_ptr(), hy.data_ptr()) == 0
        assert np.array_equal(hy.numpy(), oracle.forward(x, g))
    plan.close()
