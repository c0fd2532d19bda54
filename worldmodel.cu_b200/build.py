"""Builds libb200_w8a8.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Usage:  python worldmodel.cu_b200/build.py [--force] [--verbose]
Objects go to worldmodel.cu_b200/build/, the library next to this file.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "build"
LIB = HERE / "libb200_w8a8.so"
INCLUDE = HERE.parent / "include"

SOURCES = [
    "capi.cu",
    "status.cu",
    "quant_rows.cu",
    "dequant_ops.cu",
    "gemm_i8_tcgen05.cu",
    "gemm_i8_rowq.cu",
    "gemm_i8_blocks128.cu",
    "mma_rate.cu",
    "pack_weights.cpp",
    "weight_file.cpp",
    "dropin.cu",
    "linear_stack.cu",
    "layer_driver.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-O3,-pthread",
    "--expt-relaxed-constexpr",
]


if os.environ.get("B200_TRACE"):  # tuning builds only: per-CTA timestamps inside the GEMM kernels
    NVCC_FLAGS.append("-DB200_TRACE")


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isfile(cand) or cand == "nvcc"):
            return cand
    raise RuntimeError("nvcc not found")


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def _deps() -> list:
    return [p for p in list(CSRC.glob("*")) + list(INCLUDE.glob("*")) if p.is_file()]


def needs_build() -> bool:
    return not LIB.exists() or LIB.stat().st_mtime < _newest(_deps() + [Path(__file__)])


def build(force: bool = False, verbose: bool = False) -> Path:
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    if not force and not needs_build():
        return LIB
    OUT.mkdir(exist_ok=True)
    cc = nvcc()

    def compile_one(src: Path) -> Path:
        obj = OUT / (src.stem + ".o")
        cmd = [cc, *NVCC_FLAGS, "-x", "cu" if src.suffix == ".cu" else "c++", "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    cmd = [cc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC,-pthread",
           "-o", str(LIB), *map(str, objs)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
