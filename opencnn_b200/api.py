"""Host-side mirror of the reference's operator interface, over the C ABI.

`convolutionForward` has the argument list of the reference's dispatcher
(src/openCNN_winograd.cu:204-209) and is called the way its main() calls it (:429-440).  Device
buffers may be given as integers (device addresses) or as objects with `data_ptr()` (torch
tensors).  Layouts: input CHWN, filter CRSK, output KHWN, workspace [C][4][4][K], all fp32.
"""
from __future__ import annotations

import ctypes

from . import _lib

cudaSuccess = 0
cudaErrorInvalidValue = 1
PRECISIONS = {"fp32": 0, "tf32": 1, "bf16": 2}


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    raise TypeError(f"expected a device address or a tensor, got {type(x).__name__}")


def tiles_dim(in_w: int) -> int:
    """ceil(ceil((in_w+2)/2) - 1), the reference's tile count per row (src/openCNN_winograd.cu:286-288)."""
    return (in_w + 1) // 2


def convolutionForward(k, in_h, in_w, w, out_h, out_w, out_n, out_c, C, Ww, n, tiles_dim, in_n, tile_size,
                       elems_dim, in_c, filt_k, filt_c, filt_h, filt_w, alpha, m, *, variant="OPTSTS64") -> int:
    """Filter transform + fused Winograd kernel on the default stream; returns a cudaError_t code."""
    lib = _lib.load(variant)
    return lib.convolutionForward(_ptr(k), in_h, in_w, _ptr(w), out_h, out_w, out_n, out_c, _ptr(C), _ptr(Ww),
                                  int(n) & 0xFFFFFFFF, tiles_dim, in_n, tile_size, elems_dim, in_c, filt_k, filt_c,
                                  filt_h, filt_w, alpha, m)


def convolutionForward_32x64x8(k, in_h, in_w, w, out_h, out_w, out_n, out_c, C, Ww, n, tiles_dim, in_n, tile_size,
                               in_c, filt_k, filt_c, filt_h, filt_w, alpha, m, *, variant="OPTSTS64") -> int:
    """The reference's launcher (src/convolutionForward_32x64x8.cu:264-284)."""
    lib = _lib.load(variant)
    return lib.convolutionForward_32x64x8(_ptr(k), in_h, in_w, _ptr(w), out_h, out_w, out_n, out_c, _ptr(C),
                                          _ptr(Ww), int(n) & 0xFFFFFFFF, tiles_dim, in_n, tile_size, in_c, filt_k,
                                          filt_c, filt_h, filt_w, alpha, m)


def conv3x3(input_chwn, filter_crsk, output_khwn, workspace, N, C, H, W, K, *, precision="fp32", stream=0,
            variant="OPTSTS64") -> int:
    """Same operator with explicit sizes, arithmetic and stream (opencnn_convolutionForward_stream)."""
    lib = _lib.load(variant)
    return lib.opencnn_convolutionForward_stream(_ptr(input_chwn), _ptr(filter_crsk), _ptr(output_khwn),
                                                 _ptr(workspace), N, C, H, W, K, PRECISIONS[precision], stream)


NOALLOC_MAX_CK = 65536


def conv3x3_noalloc(input_chwn, filter_crsk, output_khwn, N, C, H, W, K, *, stream=0, variant="OPTSTS64") -> int:
    """The operator without a caller-supplied workspace (opencnn_convolutionForward_noalloc): the
    transformed filter goes to a 4 MiB array built into the library, so the call allocates nothing.
    Needs C*K <= NOALLOC_MAX_CK; calls that may overlap on the GPU must be ordered by the caller."""
    lib = _lib.load(variant)
    return lib.opencnn_convolutionForward_noalloc(_ptr(input_chwn), _ptr(filter_crsk), _ptr(output_khwn), N, C, H,
                                                  W, K, stream)


def call_like_reference(x, g, y, ws, N, C, H, W, K, *, variant="OPTSTS64") -> int:
    """Fills in the reference main()'s derived arguments (src/openCNN_winograd.cu:280-298, :429-431)."""
    td = tiles_dim(W)
    return convolutionForward(x, H, W, g, H, W, N, K, y, ws, K * N * H * W, td, N, 4, td * 4, C, K, C, 3, 3, 4, 2,
                              variant=variant)


def filter_transform(filter_crsk, workspace, C, K, *, precision="fp32", stream=0, variant="OPTSTS64") -> int:
    return _lib.load(variant).opencnn_filter_transform_p(_ptr(filter_crsk), _ptr(workspace), C, K,
                                                         PRECISIONS[precision], stream)


def winograd_forward(input_chwn, workspace, output_khwn, N, C, H, W, K, *, precision="fp32", stream=0,
                     variant="OPTSTS64") -> int:
    return _lib.load(variant).opencnn_winograd_forward(_ptr(input_chwn), _ptr(workspace), _ptr(output_khwn), N, C,
                                                       H, W, K, PRECISIONS[precision], stream)


TC_KERNELS = {"auto": 0, "single": 1, "pair_local": 2, "stacked": 3}


def winograd_forward_kernel(input_chwn, workspace, output_khwn, N, C, H, W, K, *, precision, kernel, stream=0,
                            variant="OPTSTS64") -> int:
    """The tensor-core fused kernel with an explicit choice of kernel (opencnn_winograd_forward_kernel)."""
    return _lib.load(variant).opencnn_winograd_forward_kernel(_ptr(input_chwn), _ptr(workspace), _ptr(output_khwn), N,
                                                              C, H, W, K, PRECISIONS[precision], TC_KERNELS[kernel],
                                                              stream)


def nchw_to_chwn(src, dst, N, C, H, W, *, stream=0, variant="OPTSTS64") -> int:
    return _lib.load(variant).opencnn_nchw_to_chwn(_ptr(src), _ptr(dst), N, C, H, W, stream)


def kcrs_to_crsk(src, dst, K, C, *, stream=0, variant="OPTSTS64") -> int:
    return _lib.load(variant).opencnn_kcrs_to_crsk(_ptr(src), _ptr(dst), K, C, stream)


def khwn_to_nkhw(src, dst, N, K, H, W, *, stream=0, variant="OPTSTS64") -> int:
    return _lib.load(variant).opencnn_khwn_to_nkhw(_ptr(src), _ptr(dst), N, K, H, W, stream)


def workspace_bytes(C, K, *, variant="OPTSTS64") -> int:
    return int(_lib.load(variant).opencnn_workspace_bytes(C, K))


def variant_name(variant="OPTSTS64") -> str:
    return _lib.load(variant).opencnn_variant_name().decode()


def last_device_status(variant="OPTSTS64") -> int:
    return int(_lib.load(variant).opencnn_last_device_status())


class HostPlan:
    """Host-buffer front end (opencnn_host_plan_*): numpy arrays in, numpy array out."""

    def __init__(self, N, C, H, W, K, *, precision="fp32", variant="OPTSTS64"):
        self._lib = _lib.load(variant)
        self._h = ctypes.c_void_p()
        err = self._lib.opencnn_host_plan_create(ctypes.byref(self._h), N, C, H, W, K, PRECISIONS[precision])
        if err != cudaSuccess:
            raise RuntimeError(f"opencnn_host_plan_create failed with cudaError {err}")

    def run(self, input_host_ptr: int, filter_host_ptr: int, output_host_ptr: int) -> int:
        return self._lib.opencnn_host_plan_run(self._h, input_host_ptr, filter_host_ptr, output_host_ptr)

    def run_async(self, input_host_ptr: int, filter_host_ptr: int, output_host_ptr: int) -> int:
        return self._lib.opencnn_host_plan_run_async(self._h, input_host_ptr, filter_host_ptr, output_host_ptr)

    def copy_async(self, input_host_ptr: int, filter_host_ptr: int, output_host_ptr: int) -> int:
        """The copies of run_async without the kernels (the end-to-end floor of a step)."""
        return self._lib.opencnn_host_plan_copy_async(self._h, input_host_ptr, filter_host_ptr, output_host_ptr)

    def wait(self) -> int:
        return self._lib.opencnn_host_plan_wait(self._h)

    def close(self):
        if self._h:
            self._lib.opencnn_host_plan_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
