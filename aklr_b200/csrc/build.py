"""Builds libaklr_b200.so (sm_100a only) in-tree with nvcc.  No GPU is needed to build."""

from __future__ import annotations

import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
LIB = HERE.parent / "libaklr_b200.so"
SOURCES = ["abi.cu", "routing.cu", "quant.cu", "grouped_gemm.cu", "grouped_gemm_prefill.cu", "grouped_gemm_mx.cu", "combine.cu", "router_gemm.cu", "ep.cu", "no_alloc.cu"]
HEADERS = ["common.cuh", "kernels.h", "quant_rows.cuh", "../../include/aklr_b200.h"]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(found).exists():
        raise RuntimeError("nvcc not found: libaklr_b200.so cannot be built")
    return found


def is_stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    return any((HERE / f).stat().st_mtime > built for f in SOURCES + HEADERS + ["build.py"])


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not is_stale():
        return LIB
    cmd = [
        nvcc_path(),
        "-gencode",
        "arch=compute_100a,code=sm_100a",
        "-lineinfo",
        "-O3",
        "-std=c++17",
        "-shared",
        "-Xcompiler",
        "-fPIC",
        "-Xptxas",
        "-v",
        "-o",
        str(LIB),
    ] + [str(HERE / s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libaklr_b200.so")
    (HERE / "ptxas.log").write_text(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
