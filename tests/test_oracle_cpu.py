"""The CPU oracle against exact-arithmetic known answers, the fp64 ground truth and the golden
fixtures produced by the reference's own kernels."""
import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SMALL = [(32, 8, 64, 7, 7), (32, 16, 64, 8, 8), (64, 8, 128, 5, 5), (32, 8, 64, 1, 1), (32, 8, 64, 2, 3)]


def test_generators_are_deterministic_and_sliceable(oracle):
    a = oracle.input_chwn(64, 8, 5, 5, seed=0)
    lo = oracle.input_chwn(32, 8, 5, 5, seed=0, n_offset=0)
    hi = oracle.input_chwn(32, 8, 5, 5, seed=0, n_offset=32)
    assert np.array_equal(a[..., :32], lo) and np.array_equal(a[..., 32:], hi)
    assert not np.array_equal(a, oracle.input_chwn(64, 8, 5, 5, seed=1))
    assert a.min() > -1.0 and a.max() < 1.0 and abs(float(a.mean())) < 0.02
    g = oracle.filter_crsk(64, 64, sigma=0.05, seed=0)
    assert abs(float(g.std()) - 0.05) < 0.002 and abs(float(g.mean())) < 0.002


@pytest.mark.parametrize("shape", SMALL)
def test_integer_tensors_are_exact(oracle, shape):
    N, C, K, H, W = shape
    x, g = oracle.input_int(N, C, H, W), oracle.filter_int(C, K)
    truth = oracle.direct_f64(x, g)
    assert np.array_equal(oracle.forward(x, g).astype(np.float64), truth)
    assert np.array_equal(oracle.direct_f32(x, g).astype(np.float64), truth)


@pytest.mark.parametrize("shape", SMALL)
def test_winograd_model_matches_fp64_direct(oracle, shape):
    N, C, K, H, W = shape
    x, g = oracle.input_chwn(N, C, H, W), oracle.filter_crsk(C, K)
    truth = oracle.direct_f64(x, g)
    y = oracle.forward(x, g)
    tau = 1e-2 * float(np.sqrt(np.mean(truth ** 2)))
    assert np.all(np.abs(y - truth) <= 1e-4 * np.maximum(np.abs(truth), tau))


def test_filter_transform_is_G_g_Gt(oracle):
    g = oracle.filter_crsk(8, 64)
    U = oracle.filter_transform(g).astype(np.float64)
    G = np.array([[1, 0, 0], [0.5, 0.5, 0.5], [0.5, -0.5, 0.5], [0, 0, 1]])
    expect = np.einsum("ir,crsk,js->cijk", G, g.astype(np.float64), G)
    assert np.allclose(U, expect, rtol=0, atol=1e-7)
    gi = oracle.filter_int(8, 64)
    assert np.array_equal(oracle.filter_transform(gi).astype(np.float64),
                          np.einsum("ir,crsk,js->cijk", G, gi.astype(np.float64), G))


def test_sampled_truth_matches_full(oracle):
    x, g = oracle.input_chwn(32, 8, 7, 7), oracle.filter_crsk(8, 64)
    truth = oracle.direct_f64(x, g).ravel()
    idx = np.random.default_rng(0).integers(0, truth.size, 2000)
    assert np.array_equal(oracle.direct_f64_sampled(x, g, idx), truth[idx])


def test_operand_rounding(oracle):
    a = np.array([1.0, 1.0 + 2 ** -11, 1.0 + 2 ** -10 + 2 ** -11, -3.14159, 1e-30, 65504.0], np.float32)
    t = oracle.round_tf32(a)
    assert np.all((t.view(np.uint32) & 0x1FFF) == 0)
    assert t[1] == 1.0 and t[2] == np.float32(1.0 + 2 ** -9)      # ties to even
    b = oracle.round_bf16(a)
    assert np.all((b.view(np.uint32) & 0xFFFF) == 0)
    assert np.all(np.abs(b - a) <= np.abs(a) * 2 ** -8)


def golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz")))


def test_golden_fixtures_exist():
    assert golden_files(), "tests/golden holds no reference fixtures (see tests/golden/make_golden.py)"


@pytest.mark.parametrize("path", golden_files() or [None])
def test_oracle_reproduces_reference_kernels_bit_for_bit(oracle, path):
    """Pins the oracle: the fixtures are outputs of the reference's own kernels on a B200."""
    if path is None:
        pytest.skip("no fixtures")
    z = np.load(path)
    x, g = z["input_chwn"], z["filter_crsk"]
    assert np.array_equal(oracle.filter_transform(g), z["workspace"]), "filter transform differs from FX"
    assert np.array_equal(oracle.forward(x, g), z["output_khwn"]), "fused model differs from Winograd_kernel"
