"""ctypes binding of libcomfy_kitchen_b200.so (the C ABI in include/comfy_kitchen_b200.h).

The reference binds its kernels with nanobind + DLPack
(comfy_kitchen/backends/cuda/dlpack_bindings.cpp); here the same entry points are
plain ``extern "C"`` functions taking device pointers, so the binding is a table of
argument types.  There is no fallback: if the library is missing or was built
for another architecture, importing the CUDA backend raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_bool, c_char_p, c_float, c_int, c_int64, c_void_p

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_ROOT, "lib", "libcomfy_kitchen_b200.so")

P, I64, I, F, B = c_void_p, c_int64, c_int, c_float, c_bool

# name -> argument types; every function returns int (0 = ok) unless listed in _RESTYPES
SIGNATURES: dict[str, list] = {
    "ck_abi_version": [],
    "ck_check_device": [],
    "ck_gemm_device_status": [],
    "ck_norm_device_status": [],
    "ck_set_option": [c_char_p, I],
    "ck_tp_device_status": [],
    "launch_tp_reduce_rows_kernel": [P, P, P, I, I, P, P, I64, I64, I64, I64, I64, I, I, P],
    "launch_tp_gather_kernel": [P, P, I, I, I64, I64, I64, I64, I, P],
    "launch_tp_exchange_noalloc_kernel": [P, P, P, P, I64, I64, I64, I, I, P],
    "launch_tp_exchange_kernel": [P, P, P, P, P, I, I, P, P, I64, I64, I64, I, I, P],
    "launch_quantize_fp8_kernel": [P, P, P, I64, I, I, P],
    "launch_dequantize_fp8_kernel": [P, P, P, I64, I, I, P],
    "launch_quantize_nvfp4_kernel": [P, P, P, P, I64, I64, I64, I64, F, I, B, P],
    "launch_dequantize_nvfp4_kernel": [P, P, P, P, I64, I64, I, B, P],
    "launch_quantize_mxfp8_kernel": [P, P, P, I64, I64, I64, I64, I, P],
    "launch_dequantize_mxfp8_kernel": [P, P, P, I64, I64, I, P],
    "launch_cublas_gemm_blockwise_fp4_kernel": [P, P, P, P, P, P, I64, I64, I64, P, I, P, B, P],
    "launch_scaled_mm_nvfp4_kernel": [P, P, P, P, P, P, I, I64, I64, I64, P, I, P],
    "launch_scaled_mm_nvfp4_residual_kernel": [P, P, P, P, P, P, I, P, P, I64, I64, I64, P, I, P],
    "launch_scaled_mm_nvfp4_scatter_kernel": [P, P, P, P, P, P, I, I64, P, I, I64, I64, I64, P, I, P],
    "launch_scaled_mm_mxfp8_kernel": [P, P, P, P, P, P, I, I64, I64, I64, I, P],
    "launch_apply_rope_kernel": [P, P, P, P, P] + [I64] * 17 + [I, I, B, P],
    "launch_stochastic_rounding_fp8_kernel": [P, P, P, I64, I, I, P],
    "launch_quantize_nvfp4_gather_kernel": [P, I64, I64, I64, I64, I, P, I64, I64, I64, I64, I, P, P, P, I64, I, B, P],
    "launch_qk_norm_rope_kernel": [P, I64, P, P, P, P, P, P, I64, I64, I64, I64, F, I, P],
    "launch_adaln_kernel": [P, P, P, P, I64, I64, I64, I64, F, I, P],
    "launch_rmsnorm_kernel": [P, P, P, I64, I64, F, I, P],
    "launch_adaln_quantize_nvfp4_kernel": [P, P, P, P, P, P, I64, I64, I64, I64, F, I, B, I, P],
    "launch_adaln_quantize_nvfp4_rows_kernel": [P, P, P, P, P, P, I64, I64, I64, I64, F, I, B, I, I64, I64, P],
    "launch_adaln_quantize_mxfp8_kernel": [P, P, P, P, P, I64, I64, I64, I64, F, I, I, P],
}
_RESTYPES = {"ck_last_error": c_char_p, "ck_tp_pad_bytes": c_int64}

_lib = None


class NativeLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NativeLibraryError(
            f"{LIB_PATH} not found: build it with `python comfy-kitchen_b200/build.py` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.ck_tp_pad_bytes.argtypes = []
    lib.ck_tp_pad_bytes.restype = c_int64
    lib.ck_last_error.argtypes = []
    lib.ck_last_error.restype = c_char_p
    _lib = lib
    return lib


def call(name: str, *args) -> None:
    """Invoke an entry point; raise RuntimeError with the library's message on failure."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.ck_last_error().decode(errors="replace")
        raise RuntimeError(f"{name} failed (status {rc}): {msg}")
