"""CPU-only checks of the boundary: the library loads, exports every symbol the C header
declares, the reference-named operators are defined with the reference's exact types, and
the host-side weight packer agrees with the oracle."""
import re
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

import os

ROOT = Path(__file__).resolve().parent.parent
# the reference checkout: $WORLDMODEL_REFERENCE_DIR, else a directory named `reference` beside this repository
REFERENCE_HEADER = Path(os.environ.get("WORLDMODEL_REFERENCE_DIR") or ROOT.parent / "reference") / "src" / "world_cuda_ops.cuh"


def declared_symbols():
    text = (ROOT / "include" / "b200_w8a8.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_w8a8_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.lib()
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/b200_w8a8.h but not exported"
    assert set(names) == set(pkg.exported_symbols())
    assert lib.b200_w8a8_abi_version() == 1


def test_dropin_operators_are_defined_with_cxx_linkage(pkg):
    nm = shutil.which("nm")
    if nm is None:
        pytest.skip("nm not available")
    out = subprocess.run([nm, "-D", "--defined-only", "-C", str(pkg.LIB_PATH)], capture_output=True, text=True).stdout
    for op in ["wm_cuda_quantize_rows_f32_i8(float const*, signed char*, float*, int, int)",
               "wm_cuda_rms_norm_quantize_rows_i8(float const*, float const*, float const*, signed char*, float*, int, int, float)",
               "wm_cuda_dequant_silu_quantize_rows_i8(int const*, float const*, float const*, float const*, signed char*, float*, int, int)",
               "wm_cuda_dequant_gated_residual_f32(int const*, float const*, float const*, float const*, float const*, float*, int, int)",
               "wm_cuda_dequant_add_residual_f32(int const*, float const*, float const*, float const*, float*, int, int)",
               "wm_cuda_qkv_fused_rms_rope_i32_dequant(",
               "wm_cuda_gemm_i8_i32_can_implement(signed char const*, signed char const*, int*, int, int, int)",
               "wm_cuda_gemm_i8_i32(signed char const*, signed char const*, int*, int, int, int)"]:
        assert op in out, f"missing drop-in operator {op}"


@pytest.mark.skipif(not REFERENCE_HEADER.exists(), reason="reference checkout not present")
def test_restated_header_has_the_reference_types(tmp_path):
    """Compiles one translation unit that sees BOTH headers; a mismatching redeclaration of
    any of the eight operators is a compile error, and the static_asserts pin the types."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src = tmp_path / "both.cu"
    ops = ["wm_cuda_quantize_rows_f32_i8", "wm_cuda_rms_norm_quantize_rows_i8",
           "wm_cuda_dequant_silu_quantize_rows_i8", "wm_cuda_dequant_gated_residual_f32",
           "wm_cuda_dequant_add_residual_f32", "wm_cuda_qkv_fused_rms_rope_i32_dequant",
           "wm_cuda_gemm_i8_i32_can_implement", "wm_cuda_gemm_i8_i32"]
    body = ['#include "world_cuda_ops.cuh"', '#include "world_cuda_ops_w8a8.cuh"', "#include <type_traits>"]
    body += [f"static_assert(std::is_function<decltype({op})>::value, \"{op}\");" for op in ops]
    body.append("int main() { return 0; }")
    src.write_text("\n".join(body) + "\n")
    r = subprocess.run([nvcc, "-std=c++17", "-c", str(src), "-o", str(tmp_path / "both.o"),
                        f"-I{REFERENCE_HEADER.parent}", f"-I{ROOT / 'include'}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


@pytest.mark.parametrize("layout", [0, 1])
def test_pack_weight_host_matches_oracle(pkg, ref, layout):
    g = torch.Generator().manual_seed(7)
    n, k = 72, 256
    w = torch.randn(n, k, generator=g) * 0.02
    w[3] = 0.0
    w[5, 17] *= -30.0
    packed, scales = pkg.pack_weight(w, layout=layout, threads=3)
    q_ref, s_ref = ref.quantize_weight(w)
    assert np.array_equal(scales.numpy().view(np.uint32), s_ref.numpy().view(np.uint32))
    if layout == pkg.W_ROW_MAJOR:
        got = packed.view(n, k)
    else:
        got = packed.view(k // 128, n, 128).permute(1, 0, 2).reshape(n, k)
    assert torch.equal(got, q_ref)
    assert scales[3].item() == 1.0 and int(got[3].abs().max()) == 0


def test_pack_weight_host_rejects_bad_input(pkg):
    w = torch.randn(8, 128)
    w[2, 5] = float("nan")
    with pytest.raises(pkg.W8A8Error, match="not finite"):
        pkg.pack_weight(w, layout=pkg.W_ROW_MAJOR)
    with pytest.raises(pkg.W8A8Error):
        pkg.pack_weight(torch.randn(8, 96), layout=pkg.W_SLAB128)  # K % 128 != 0


def test_argument_validation_needs_no_gpu(pkg):
    lib = pkg.lib()
    # null pointers and bad shapes are rejected on the host before anything is launched
    assert lib.b200_w8a8_gemm_i8_i32_can_implement(None, None, 0, None, 128, 128, 128) == 1
    assert lib.b200_w8a8_gemm_i8_i32_can_implement(4096, 8192, 0, 16384, 128, 100, 128) == 1  # K % 32
    assert b"K must be divisible by 32" in lib.b200_w8a8_last_error()
    assert lib.b200_w8a8_gemm_i8_i32_can_implement(4096, 8192, 0, 16384, 128, 128, 128) == 0
    assert lib.b200_w8a8_gemm_i8_i32_can_implement(4096, 8192, 1, 16384, 128, 96, 128) == 1  # slab needs K%128
    assert lib.b200_w8a8_gemm_i8_i32_can_implement(4097, 8192, 0, 16384, 128, 128, 128) == 1  # alignment
    assert lib.b200_w8a8_quantize_rows(None, 0, 8, None, 8, None, 1, 8, None) == 1


def test_reference_operator_library_exports_the_eight_w8a8_operators():
    """oracle/_ref/ holds the reference's own operator file compiled in place (test infrastructure);
    when it was built, every W8A8 operator must resolve under its C++-mangled name."""
    import sys
    sys.path.insert(0, str(ROOT / "oracle"))
    import ref_cuda_ops as rk
    if not rk.available():
        pytest.skip("the reference operator library is not built on this machine")
    lib = rk.lib()
    for short in ("gemm_i8_i32", "gemm_i8_i32_can_implement", "quantize_rows_f32_i8", "rms_norm_quantize_rows_i8",
                  "dequant_silu_quantize_rows_i8", "dequant_gated_residual_f32", "dequant_add_residual_f32",
                  "qkv_fused_rms_rope_i32_dequant"):
        assert callable(getattr(lib, short))


def test_ctypes_prototypes_match_the_header_parameter_by_parameter(pkg):
    """ctypes does not complain about a call with one argument too many or too few, so the Python prototype table
    is checked against the C declarations: same number of parameters, each of the same class (pointer, 32-bit
    integer, 64-bit integer / size, float, double)."""
    import ctypes
    text = (ROOT / "include" / "b200_w8a8.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    decls = re.findall(r"\b(b200_w8a8_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S)
    assert len(decls) >= 50

    def c_kind(param):
        p = " ".join(param.split())
        if p in ("void", ""):
            return None
        if "*" in p:
            return "ptr"
        if "int64_t" in p or "size_t" in p or "unsigned long long" in p:
            return "i64"
        if "double" in p:
            return "f64"
        if "float" in p:
            return "f32"
        assert re.search(r"\bint\b", p), f"unclassified parameter `{p}`"
        return "i32"

    def py_kind(t):
        if t in (ctypes.c_int64, ctypes.c_size_t, ctypes.c_ulonglong, ctypes.c_uint64):
            return "i64"
        if t is ctypes.c_int:
            return "i32"
        if t is ctypes.c_float:
            return "f32"
        if t is ctypes.c_double:
            return "f64"
        return "ptr"  # c_void_p, c_char_p, POINTER(...)

    for name, params in decls:
        want = [k for k in (c_kind(x) for x in params.split(",")) if k is not None]
        got = [py_kind(t) for t in pkg._PROTOTYPES[name][1]]
        assert want == got, f"{name}: header {want}, Python table {got}"
