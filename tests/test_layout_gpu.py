"""Layout adapters (NCHW -> CHWN, KCRS -> CRSK, KHWN -> NKHW) against torch permutes, and the
whole NCHW-in / NCHW-out chain against torch's own convolution in fp64."""
import pytest

torch = pytest.importorskip("torch")

from opencnn_b200 import api  # noqa: E402

pytestmark = pytest.mark.gpu


# both extents multiples of 4 (the 128-bit kernel, with partial tiles), an odd batch and an odd C*H*W (the
# element-wise kernel), and the benchmark's largest tensor
@pytest.mark.parametrize("shape", [(32, 8, 7, 7), (64, 24, 5, 9), (33, 3, 17, 2), (32, 3, 7, 7), (68, 4, 9, 13), (128, 64, 56, 56)])
def test_nchw_to_chwn_and_back(libs, shape):
    N, C, H, W = shape
    x = torch.randn(N, C, H, W, device="cuda")
    chwn = torch.full((C, H, W, N), float("nan"), device="cuda")
    assert api.nchw_to_chwn(x, chwn, N, C, H, W) == 0
    torch.cuda.synchronize()
    assert torch.equal(chwn, x.permute(1, 2, 3, 0).contiguous())
    back = torch.full((N, C, H, W), float("nan"), device="cuda")        # KHWN -> NKHW with K := C
    assert api.khwn_to_nkhw(chwn, back, N, C, H, W) == 0
    torch.cuda.synchronize()
    assert torch.equal(back, x)


@pytest.mark.parametrize("kc", [(192, 40), (64, 3), (130, 7)])
def test_kcrs_to_crsk(libs, kc):
    K, C = kc
    w = torch.randn(K, C, 3, 3, device="cuda")
    crsk = torch.empty((C, 3, 3, K), device="cuda")
    assert api.kcrs_to_crsk(w, crsk, K, C) == 0
    torch.cuda.synchronize()
    assert torch.equal(crsk, w.permute(1, 2, 3, 0).contiguous())


def test_nchw_chain_matches_fp64_convolution(libs):
    N, C, K, H, W = 32, 16, 64, 10, 10
    x = torch.rand(N, C, H, W, device="cuda") * 2 - 1
    w = torch.randn(K, C, 3, 3, device="cuda") * 0.05
    xc, wc = torch.empty((C, H, W, N), device="cuda"), torch.empty((C, 3, 3, K), device="cuda")
    yk, ws = torch.empty((K, H, W, N), device="cuda"), torch.empty((C, 4, 4, K), device="cuda")
    y = torch.empty((N, K, H, W), device="cuda")
    assert api.nchw_to_chwn(x, xc, N, C, H, W) == 0 and api.kcrs_to_crsk(w, wc, K, C) == 0
    assert api.call_like_reference(xc, wc, yk, ws, N, C, H, W, K) == 0
    assert api.khwn_to_nkhw(yk, y, N, K, H, W) == 0
    torch.cuda.synchronize()
    truth = torch.nn.functional.conv2d(x.double(), w.double(), padding=1)
    rms = truth.pow(2).mean().sqrt()
    assert (y.double() - truth).abs().max() <= 1e-4 * rms       # the fp32 path's tolerance against fp64
