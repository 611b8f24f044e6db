"""The C-ABI libraries load and export what include/opencnn_b200.h declares; argument errors
are reported before any CUDA work (no GPU needed)."""
import ctypes
import os
import re

import pytest

from opencnn_b200 import _lib, api, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "opencnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(names))


def test_header_lists_the_expected_entry_points():
    names = header_functions()
    assert "convolutionForward" in names and "convolutionForward_32x64x8" in names
    assert set(names) == set(_lib.SIGNATURES), (names, sorted(_lib.SIGNATURES))


def test_python_enums_match_the_header():
    """The precision and tensor-core kernel codes of the Python mirror are the header's enumerators."""
    text = open(os.path.join(ROOT, "include", "opencnn_b200.h")).read()
    enums = {m.group(1): int(m.group(2)) for m in re.finditer(r"\b(OPENCNN_[A-Z0-9_]+)\s*=\s*(\d+)", text)}
    assert enums["OPENCNN_FP32"] == api.PRECISIONS["fp32"] and enums["OPENCNN_TF32"] == api.PRECISIONS["tf32"]
    assert enums["OPENCNN_BF16"] == api.PRECISIONS["bf16"]
    header_kernels = {"auto": "OPENCNN_TC_AUTO", "single": "OPENCNN_TC_SINGLE_CTA", "pair_local": "OPENCNN_TC_PAIR_LOCAL",
                      "stacked": "OPENCNN_TC_STACKED_BLOCKS"}
    assert set(api.TC_KERNELS) == set(header_kernels)
    for name, enumerator in header_kernels.items():
        assert api.TC_KERNELS[name] == enums[enumerator], name


@pytest.mark.parametrize("variant", build.VARIANTS)
def test_library_exports_every_declared_symbol(libs, variant):
    lib = libs[variant]
    for name in header_functions():
        assert hasattr(lib, name), f"{variant}: missing symbol {name}"
    assert lib.opencnn_variant_name().decode() == variant


def test_workspace_bytes(libs):
    lib = libs["OPTSTS64"]
    assert lib.opencnn_workspace_bytes(64, 64) == 64 * 16 * 64 * 4
    assert lib.opencnn_workspace_bytes(1024, 1024) == 1024 * 16 * 1024 * 4
    assert lib.opencnn_workspace_bytes(0, 64) == 0


def test_missing_library_raises(monkeypatch):
    monkeypatch.setattr(_lib, "lib_path", lambda v: "/nonexistent/libopencnn_b200.so")
    monkeypatch.setattr(_lib, "_cache", {})
    with pytest.raises(_lib.LibraryMissing):
        _lib.load("OPTSTS64")


def _call(variant, N=32, C=8, H=8, W=8, K=64, ptr=0x1000, **over):
    a = dict(k=ptr, in_h=H, in_w=W, w=ptr, out_h=H, out_w=W, out_n=N, out_c=K, C=ptr, Ww=ptr, n=0,
             tiles_dim=(W + 1) // 2, in_n=N, tile_size=4, elems_dim=0, in_c=C, filt_k=K, filt_c=C, filt_h=3,
             filt_w=3, alpha=4, m=2)
    a.update(over)
    return api.convolutionForward(*a.values(), variant=variant)


@pytest.mark.parametrize("variant", build.VARIANTS)
def test_argument_errors_are_reported(libs, variant):
    inval = api.cudaErrorInvalidValue
    assert _call(variant, in_n=48, out_n=48) == inval          # N % 32
    assert _call(variant, filt_k=96, out_c=96) == inval        # K % 64
    assert _call(variant, in_c=12, filt_c=12) == inval         # C % 8
    assert _call(variant, filt_h=5) == inval                   # 3x3 only
    assert _call(variant, m=4) == inval                        # F(2x2,3x3) only
    assert _call(variant, tiles_dim=3) == inval                # inconsistent tiling
    assert _call(variant, out_c=128) == inval                  # out_c != filt_k
    assert _call(variant, k=0) == inval                        # null input
    assert _call(variant, C=0x1004) == inval                   # misaligned output
    assert _call(variant, in_n=0, out_n=0) == inval


def test_unknown_variant_rejected():
    with pytest.raises(ValueError):
        _lib.load("OPTSTS32")


def test_tensor_core_output_must_be_32_byte_aligned(libs):
    """The TF32 / BF16 kernels store 32 bytes per thread: a 16-byte-aligned output that is not 32-byte aligned
    is refused before anything is launched (no GPU needed); fp32 accepts it."""
    lib = libs["OPTSTS64"]
    inval = api.cudaErrorInvalidValue
    N, C, H, W, K = 32, 8, 8, 8, 64
    for prec in (api.PRECISIONS["tf32"], api.PRECISIONS["bf16"]):
        assert lib.opencnn_convolutionForward_stream(0x1000, 0x1000, 0x1010, 0x1000, N, C, H, W, K, prec, None) == inval
        assert lib.opencnn_winograd_forward(0x1000, 0x1000, 0x1010, N, C, H, W, K, prec, None) == inval
    # 8-byte-aligned pointers are refused everywhere
    assert lib.opencnn_convolutionForward_stream(0x1000, 0x1000, 0x1008, 0x1000, N, C, H, W, K, 0, None) == inval
