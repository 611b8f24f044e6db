"""opencnn_convolutionForward_noalloc: the operator for callers that may not allocate device
memory (an application that hands out all device memory from its own pool, a plugin that gets
only its tensors, a process on a fixed memory budget).  Its workspace is a 4 MiB array inside
the library, so this checks, through the C ABI, that it gives exactly what the ordinary entry
point gives with a caller-allocated workspace - on two calls in a row with different data,
because the built-in array keeps whatever the previous call left in it - and that problems too
large for the array are refused.  Collected last on purpose: it must pass after every other
test has used the library, and also alone in a fresh process."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from opencnn_b200 import api, build  # noqa: E402

pytestmark = pytest.mark.gpu


def _reference_entry(variant, dx, dg, N, C, H, W, K):
    dy = torch.full((K, H, W, N), float("nan"), device="cuda")
    dws = torch.empty((C, 4, 4, K), device="cuda")
    assert api.conv3x3(dx, dg, dy, dws, N, C, H, W, K, variant=variant) == 0
    torch.cuda.synchronize()
    return dy


@pytest.mark.parametrize("variant", build.VARIANTS)
def test_noalloc_matches_ordinary_entry_on_two_calls(oracle, libs, variant):
    # second problem is smaller in C*K than the first: stale workspace contents beyond it must not matter
    for seed, (N, C, K, H, W) in enumerate([(64, 64, 128, 12, 12), (32, 16, 64, 7, 9)]):
        x, g = oracle.input_chwn(N, C, H, W, seed=seed), oracle.filter_crsk(C, K, seed=seed)
        dx, dg = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
        expect = _reference_entry(variant, dx, dg, N, C, H, W, K)
        dy = torch.full((K, H, W, N), float("nan"), device="cuda")
        # Free device memory as the driver reports it (cudaMemGetInfo): unlike torch's own counters
        # it would also show a cudaMalloc made inside the library.  The first call per variant and
        # device does the one-time set-up (module load, address look-up), so the measured call is
        # the one after it; nothing else allocates in between.
        if seed == 0:
            assert api.conv3x3_noalloc(dx, dg, dy, N, C, H, W, K, variant=variant) == 0
            torch.cuda.synchronize()
            dy.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert api.conv3x3_noalloc(dx, dg, dy, N, C, H, W, K, variant=variant) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert api.last_device_status(variant) == 0
        assert torch.equal(dy, expect), f"max |diff| {(dy - expect).abs().max().item()}"
        assert np.array_equal(dy.cpu().numpy(), oracle.forward(x, g))


def test_noalloc_refuses_problems_beyond_its_workspace(libs, capfd):
    N, C, K, H, W = 32, 512, 256, 4, 4            # C*K = 131072 > 65536
    assert C * K > api.NOALLOC_MAX_CK
    dx = torch.zeros((C, H, W, N), device="cuda")
    dg = torch.zeros((C, 3, 3, K), device="cuda")
    dy = torch.zeros((K, H, W, N), device="cuda")
    assert api.conv3x3_noalloc(dx, dg, dy, N, C, H, W, K) == api.cudaErrorInvalidValue
    assert "OPENCNN_NOALLOC_MAX_CK" in capfd.readouterr().err
    # the largest problem that fits is accepted
    C = K = 256
    dx = torch.zeros((C, H, W, N), device="cuda")
    dg = torch.zeros((C, 3, 3, K), device="cuda")
    dy = torch.full((K, H, W, N), float("nan"), device="cuda")
    assert api.conv3x3_noalloc(dx, dg, dy, N, C, H, W, K) == 0
    torch.cuda.synchronize()
    assert torch.count_nonzero(dy).item() == 0
