"""ctypes view of the reference's own W8A8 CUDA operators, built by build_reference_ops.py.

TEST AND BENCHMARK INFRASTRUCTURE ONLY: the product never loads this.  The operators have C++
linkage in the reference (src/world_cuda_ops.cuh:20-56, 120-138, 315-328), so they are looked
up by their Itanium-mangled names.  Arguments are torch CUDA tensors; every operator runs on the
stream the reference uses (its default stream) and returns the reference's 0 / 1 status."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libworld_cuda_ops_ref.so"

_SYMBOLS = {
    "gemm_i8_i32": ("_Z19wm_cuda_gemm_i8_i32PKaS0_Piiii", [c_void_p] * 3 + [c_int] * 3),
    "gemm_i8_i32_can_implement": ("_Z33wm_cuda_gemm_i8_i32_can_implementPKaS0_Piiii", [c_void_p] * 3 + [c_int] * 3),
    "quantize_rows_f32_i8": ("_Z28wm_cuda_quantize_rows_f32_i8PKfPaPfii", [c_void_p] * 3 + [c_int] * 2),
    "rms_norm_quantize_rows_i8": ("_Z33wm_cuda_rms_norm_quantize_rows_i8PKfS0_S0_PaPfiif",
                                  [c_void_p] * 5 + [c_int] * 2 + [c_float]),
    "dequant_silu_quantize_rows_i8": ("_Z37wm_cuda_dequant_silu_quantize_rows_i8PKiPKfS2_S2_PaPfii",
                                      [c_void_p] * 6 + [c_int] * 2),
    "dequant_gated_residual_f32": ("_Z34wm_cuda_dequant_gated_residual_f32PKiPKfS2_S2_S2_Pfii",
                                   [c_void_p] * 6 + [c_int] * 2),
    "dequant_add_residual_f32": ("_Z32wm_cuda_dequant_add_residual_f32PKiPKfS2_S2_Pfii", [c_void_p] * 5 + [c_int] * 2),
    "qkv_fused_rms_rope_i32_dequant": ("_Z38wm_cuda_qkv_fused_rms_rope_i32_dequantPKiPKfS2_PfS3_S3_PKlS5_S5_S2_S2_iiiiiif",
                                       [c_void_p] * 11 + [c_int] * 6 + [c_float]),
}

_lib = None


def available() -> bool:
    return LIB_PATH.is_file()


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(f"{LIB_PATH} is not built (python oracle/build_reference_ops.py)")
        _lib = ctypes.CDLL(str(LIB_PATH))
        for short, (mangled, argtypes) in _SYMBOLS.items():
            fn = getattr(_lib, mangled)
            fn.restype = c_int
            fn.argtypes = argtypes
            setattr(_lib, short, fn)
    return _lib


def _p(t):
    return None if t is None else t.data_ptr()


def call(name: str, *args) -> None:
    """Calls operator `name` with tensors / scalars in the reference's argument order."""
    rc = getattr(lib(), name)(*[_p(a) if hasattr(a, "data_ptr") else a for a in args])
    if rc != 0:
        raise RuntimeError(f"reference operator {name} returned {rc}")
