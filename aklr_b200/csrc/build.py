"""Builds libaklr_b200.so (sm_100a only) in-tree with nvcc.  No GPU is needed to build.

Every ``.cu`` file is compiled to an object under ``build/`` at the repository root (one nvcc
process per file, side by side) and the objects are linked into ``aklr_b200/libaklr_b200.so``.
The compiler's resource report (registers, spills, shared memory per kernel) goes to
``build/ptxas.log``.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
LIB = HERE.parent / "libaklr_b200.so"
OBJ_DIR = HERE.parent.parent / "build" / "obj"
SOURCES = [
    "abi.cu",
    "routing.cu",
    "quant.cu",
    "grouped_gemm.cu",
    "grouped_gemm_prefill.cu",
    "grouped_gemm_deep.cu",
    "grouped_gemm_mx.cu",
    "combine.cu",
    "router_gemm.cu",
    "weight_layout.cu",
    "ep.cu",
    "no_alloc.cu",
]
HEADERS = ["common.cuh", "kernels.h", "quant_rows.cuh", "../../include/aklr_b200.h"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(found).exists():
        raise RuntimeError("nvcc not found: libaklr_b200.so cannot be built")
    return found


STAMP = LIB.with_suffix(".so.stamp")  # digest of what the library was built from


def _newest_header() -> float:
    return max((HERE / f).stat().st_mtime for f in HEADERS + ["build.py"])


def source_digest() -> str:
    """Digest of every source, header and flag: a copy of the tree whose file times were not kept
    still recognises its own library."""
    h = hashlib.sha256(" ".join(FLAGS).encode())
    for f in SOURCES + HEADERS:
        h.update(f.encode())
        h.update((HERE / f).read_bytes())
    return h.hexdigest()


def is_stale() -> bool:
    if not LIB.exists() or not STAMP.exists():
        return True
    return STAMP.read_text().strip() != source_digest()


def _compile(nvcc: str, source: str, force: bool) -> tuple[str, int, str]:
    obj = OBJ_DIR / (source + ".o")
    src = HERE / source
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, _newest_header()):
        log = obj.with_suffix(".log")
        return source, 0, log.read_text() if log.exists() else ""
    proc = subprocess.run([nvcc, *FLAGS, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
    text = proc.stdout + proc.stderr
    if proc.returncode == 0:
        obj.with_suffix(".log").write_text(text)
    return source, proc.returncode, text


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not is_stale():
        return LIB
    nvcc = nvcc_path()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(lambda s: _compile(nvcc, s, force), SOURCES))
    failed = [r for r in results if r[1] != 0]
    if verbose or failed:
        for source, _, text in failed or results:
            sys.stderr.write(f"---- {source}\n{text}")
    if failed:
        raise RuntimeError("nvcc failed on " + ", ".join(r[0] for r in failed))
    (OBJ_DIR.parent / "ptxas.log").write_text("".join(f"---- {s}\n{t}" for s, _, t in results))
    link = [nvcc, "-shared", "-o", str(LIB)] + [str(OBJ_DIR / (s + ".o")) for s in SOURCES]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("linking libaklr_b200.so failed")
    STAMP.write_text(source_digest() + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
