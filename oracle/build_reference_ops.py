"""Compiles the reference's own CUDA operator file, where it lies, into oracle/_ref/.

TEST AND BENCHMARK INFRASTRUCTURE ONLY.  Nothing of the product loads this library; it is the
"reference kernels on the same GPU" comparator and the strongest pin of the parity tests.

Recipe: nvcc on `<reference>/src/world_cuda_ops.cu` alone (the file that defines the eight W8A8
operators of src/world_cuda_ops.cuh:20-56, 120-138, 315-328 next to the reference's other
operators), with the reference's own flags (`--use_fast_math --expt-relaxed-constexpr`,
CMakeLists.txt:47-48) and its CUTLASS 2.x-API Sm80 kernel (src/world_cuda_ops.cu:529-548)
compiled for sm_100a.  The reference fetches CUTLASS 3.5.1 at configure time
(CMakeLists.txt:52-84); that tree is absent here, so a CUTLASS header tree that some Python
package vendors is used instead.  It is a third-party dependency that is not part of the
reference checkout, so this library can be missing (the tests that need it skip, the bench
entry reports it as unavailable) and never gates correctness.  The memory-efficient attention
path of the file is compiled out by its own `__has_include("kernel_forward.h")` guard.

No reference source is copied: the compiler reads the file in place and only the built
library is written, to oracle/_ref/ (git-ignored).

Usage:  python oracle/build_reference_ops.py [--reference DIR] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
LIB = OUT_DIR / "libworld_cuda_ops_ref.so"
# the reference checkout: $WORLDMODEL_REFERENCE_DIR, else a directory named `reference` beside this repository
DEFAULT_REFERENCE = Path(os.environ.get("WORLDMODEL_REFERENCE_DIR") or HERE.parent.parent / "reference")
CUTLASS_CANDIDATES = ("flashinfer/data/cutlass/include", "tilelang/3rdparty/cutlass/include",
                      "deep_gemm/include")


def find_cutlass() -> Path | None:
    roots = {sysconfig.get_paths().get("purelib"), sysconfig.get_paths().get("platlib")}
    for root in filter(None, roots):
        for rel in CUTLASS_CANDIDATES:
            inc = Path(root) / rel
            if (inc / "cutlass" / "gemm" / "device" / "gemm.h").is_file():
                return inc
    return None


def build(reference: Path = DEFAULT_REFERENCE, force: bool = False, verbose: bool = False) -> Path | None:
    """Returns the library path, or None when the reference or a CUTLASS header tree is absent."""
    src = reference / "src" / "world_cuda_ops.cu"
    if not src.is_file():
        return LIB if LIB.is_file() else None
    if LIB.is_file() and not force and LIB.stat().st_mtime >= src.stat().st_mtime:
        return LIB
    cutlass = find_cutlass()
    if cutlass is None:
        if verbose:
            sys.stderr.write("no CUTLASS header tree found: the reference operators are not built\n")
        return None
    nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    OUT_DIR.mkdir(exist_ok=True)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--use_fast_math",
           "--expt-relaxed-constexpr", "-w", "-Xcompiler", "-fPIC", "-shared",
           "-I", str(reference / "src"), "-I", str(cutlass), "-o", str(LIB), str(src)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        if verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout[-4000:] + r.stderr[-4000:])
        return None
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    lib = build(a.reference, a.force, verbose=True)
    print(lib if lib else "not built")
    sys.exit(0 if lib else 1)
