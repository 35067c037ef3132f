"""Stand-alone measurements of the pieces a grouped GEMM is made of, on all 148 SMs of one B200: what the tensor
pipe, the TMA ring and the two together can do with nothing else in their way.  The kernels' own periods are read
against these numbers.

    python -m aklr_b200.csrc.probes            # builds the programs under build/probes and runs them

* ``tma_ring``: persistent CTAs that only run the operand ring of the token-major kernel (48 KB x 4 stages, or
  32 KB x 6), stages recycled the moment they fill: bytes per second from L2 / HBM into shared memory; the same
  with the MXFP4 kernel's packed e2m1 weight tiles, which the TMA unpacks on the way.
* ``mma_chain``: cycles per ``tcgen05.mma kind::f8f6f4`` (M 128, K 32) for N = 16 .. 256, with every MMA depending on
  the one before or rotating over 2 .. 8 accumulators.
* ``mma_beside_tma``: the MMA stream of a K-block (two deep) alone, a TMA ring alone, and both at once.
* ``mx_issue``: the MXFP4 kernel's issue stream alone: four block-scaled MMAs per K-block with 0 .. 4 ``tcgen05.cp`` of
  scale factors in front of them.
* ``mma_burst``: bursts of 1 .. 12 MMAs from an idle pipe: what one ``tcgen05.mma`` costs its issuing thread and how far
  the pipe lets the thread run ahead.
* ``mma_data``: the same N = 256 MMA stream on constant and on random operands, in cycles and in nanoseconds: the SM
  clock the part holds while its tensor pipes are busy depends on the data.

Every wait in them is bounded; they allocate at most 4 GB and run for a few seconds.
"""

from __future__ import annotations

import pathlib
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
ROOT = HERE.parents[2]
OUT = ROOT / "build" / "probes"
PROGRAMS = ("tma_ring", "mma_chain", "mma_beside_tma", "mx_issue", "mma_burst", "mma_data")


def build() -> list[pathlib.Path]:
    OUT.mkdir(parents=True, exist_ok=True)
    built = []
    for name in PROGRAMS:
        exe = OUT / name
        src = HERE / f"{name}.cu"
        if not exe.exists() or exe.stat().st_mtime < src.stat().st_mtime:
            subprocess.run(
                ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
                 f"-I{ROOT / 'include'}", "-o", str(exe), str(src)],
                check=True,
            )
        built.append(exe)
    return built


def main() -> int:
    for exe in build():
        print(f"== {exe.name}", flush=True)
        rc = subprocess.run([str(exe)], timeout=120).returncode
        if rc:
            return rc
    return 0
