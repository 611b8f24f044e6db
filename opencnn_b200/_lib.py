"""ctypes bindings of the C ABI declared in include/opencnn_b200.h.

There is no fallback of any kind: if the shared library of the requested variant has not been
built, loading raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_uint, c_void_p, POINTER

from .build import VARIANTS, lib_path

_f = POINTER(c_float)

# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "convolutionForward_32x64x8": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                           c_void_p, c_uint] + [c_int] * 10),
    "convolutionForward": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                   c_void_p, c_uint] + [c_int] * 11),
    "opencnn_convolutionForward_stream": (c_int, [c_void_p] * 4 + [c_int] * 6 + [c_void_p]),
    "opencnn_filter_transform": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "opencnn_filter_transform_p": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "opencnn_winograd_forward": (c_int, [c_void_p] * 3 + [c_int] * 6 + [c_void_p]),
    "opencnn_winograd_forward_kernel": (c_int, [c_void_p] * 3 + [c_int] * 7 + [c_void_p]),
    "opencnn_convolutionForward_noalloc": (c_int, [c_void_p] * 3 + [c_int] * 5 + [c_void_p]),
    "opencnn_nchw_to_chwn": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "opencnn_kcrs_to_crsk": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "opencnn_khwn_to_nkhw": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "opencnn_workspace_bytes": (c_size_t, [c_int, c_int]),
    "opencnn_variant_name": (c_char_p, []),
    "opencnn_last_device_status": (c_int, []),
    "opencnn_host_plan_create": (c_int, [POINTER(c_void_p)] + [c_int] * 6),
    "opencnn_host_plan_run": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "opencnn_host_plan_run_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "opencnn_host_plan_copy_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "opencnn_host_plan_wait": (c_int, [c_void_p]),
    "opencnn_host_plan_destroy": (c_int, [c_void_p]),
}

_cache: dict[str, ctypes.CDLL] = {}


class LibraryMissing(RuntimeError):
    pass


def load(variant: str = "OPTSTS64") -> ctypes.CDLL:
    """Loads libopencnn_b200_<variant>.so (built by opencnn_b200.build) and types its symbols."""
    if variant not in VARIANTS:
        raise ValueError(f"unknown variant {variant!r}; expected one of {VARIANTS}")
    if variant in _cache:
        return _cache[variant]
    path = lib_path(variant)
    if not os.path.exists(path):
        raise LibraryMissing(f"{path} not found: build it with `python -m opencnn_b200.build` "
                             "(there is no non-CUDA fallback)")
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _cache[variant] = lib
    return lib
