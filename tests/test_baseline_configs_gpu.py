"""Parity at the full sizes of the benchmark configurations: the N=128 layer sweep, the two wide
stress layers (N=64 C=K=1024 14x14: 128 chunks per tile, the deepest FMA chains; N=256 C=32 K=64
112x112: 25 088 tiles, the largest tile index and output offsets) and the N=1024 stack shapes with
their per-GPU shards.  Every staging variant is compared on the device, bit for bit, with the
reference's own kernels of the same variant (oracle/_ref, grid (in_n/32, tiles, filt_k/64) as in
src/convolutionForward_32x64x8.cu:281; shapes of bench/bench.sh:3-21) - workspace and output -
and one variant per shape with 10^5 sampled fp64 outputs.  Nothing is copied to the host except
the operands of the sampled check."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from opencnn_b200 import api, build  # noqa: E402

pytestmark = pytest.mark.gpu
REL = 1e-4

# name -> N, C, K, H=W
SHAPES = {
    "sweep_56": (128, 64, 64, 56), "sweep_28": (128, 128, 128, 28), "sweep_14": (128, 256, 256, 14),
    "sweep_7": (128, 512, 512, 7),
    "layer_a": (64, 1024, 1024, 14), "layer_b": (256, 32, 64, 112),
    "stack_56_n1024": (1024, 64, 64, 56), "stack_7_n1024": (1024, 512, 512, 7),
    "shard_28_n512": (512, 128, 128, 28), "shard_14_n256": (256, 256, 256, 14),
}


def _tensors(N, C, K, HW, seed):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    x = torch.rand((C, HW, HW, N), device="cuda", generator=gen) * 2 - 1
    g = torch.randn((C, 3, 3, K), device="cuda", generator=gen) * 0.05
    return x, g


@pytest.mark.parametrize("name", list(SHAPES))
def test_bit_identical_to_reference_kernels_at_full_size(oracle, libs, ref_libs, name):
    if set(build.VARIANTS) - set(ref_libs):
        pytest.skip("oracle/_ref not built")
    N, C, K, HW = SHAPES[name]
    x, g = _tensors(N, C, K, HW, seed=len(name))
    ours = torch.empty((K, HW, HW, N), device="cuda")
    theirs = torch.empty_like(ours)
    ws, rws = torch.empty((C, 4, 4, K), device="cuda"), torch.empty((C, 4, 4, K), device="cuda")
    first = None
    for variant in build.VARIANTS:
        ours.fill_(float("nan")); theirs.fill_(float("nan")); ws.fill_(float("nan")); rws.fill_(0)
        assert ref_libs[variant].forward(x, g, theirs, rws, N, C, HW, K) == 0
        assert api.call_like_reference(x, g, ours, ws, N, C, HW, HW, K, variant=variant) == 0
        assert api.last_device_status(variant) == 0
        assert torch.equal(ws, rws), f"{variant}: filter transform differs"
        diff = int((ours != theirs).sum().item())             # NaN != NaN: unwritten outputs count
        assert diff == 0, f"{variant}: {diff} of {ours.numel()} outputs differ from the reference kernel's"
        if first is None:
            first = ours.clone()
        else:
            assert torch.equal(ours, first), f"{variant} differs from {build.VARIANTS[0]}"
    # ground truth on 10^5 sampled outputs: |y - t| <= 1e-4 * max(|t|, rms(t))
    hx, hg = x.cpu().numpy(), g.cpu().numpy()
    idx = np.random.default_rng(7).integers(0, first.numel(), 100000)
    truth = oracle.direct_f64_sampled(hx, hg, idx)
    got = first.view(-1)[torch.from_numpy(idx).cuda()].cpu().numpy()
    tau = float(np.sqrt(np.mean(truth ** 2)))
    assert np.all(np.abs(got - truth) <= REL * np.maximum(np.abs(truth), tau)), \
        f"worst {np.max(np.abs(got - truth) / np.maximum(np.abs(truth), tau)):.2e}"


def test_split_and_one_call_entries_agree_on_the_deepest_layer(libs):
    """Layer A through the cached-filter entries on a side stream equals the one-call entry."""
    N, C, K, HW = SHAPES["layer_a"]
    x, g = _tensors(N, C, K, HW, seed=3)
    a, b = torch.empty((K, HW, HW, N), device="cuda"), torch.full((K, HW, HW, N), float("nan"), device="cuda")
    ws = torch.empty((C, 4, 4, K), device="cuda")
    assert api.call_like_reference(x, g, a, ws, N, C, HW, HW, K) == 0
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    ws2 = torch.empty_like(ws)
    assert api.filter_transform(g, ws2, C, K, stream=s.cuda_stream) == 0
    assert api.winograd_forward(x, ws2, b, N, C, HW, HW, K, stream=s.cuda_stream) == 0
    s.synchronize()
    assert torch.equal(a, b) and api.last_device_status() == 0
