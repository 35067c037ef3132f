"""Weight layouts the FP8 grouped GEMMs take besides the checkpoint's row-major one.

``b200_tiled``: ``[experts, rows, cols]`` stored as ``[experts, rows/128, cols/128, 128, 128]`` -- every
128-row x 128-byte tile a TMA load fetches is one contiguous 16 KB run of HBM.  A loader converts once, after
the checkpoint is on the device (``to_b200_tiled``), and the tensor carries the attribute ``is_b200_tiled``;
the ops read that attribute the way the reference's contracts read ``is_shuffled`` for its own engine-side
layout (aklr/plugins/sglang/models/deepseek_v2/contract.py:181-185, 310-318; layout types
aklr/core/contract/semantics/_layouts.py:103-121).  Block scales are per 128 x 128 tile in both layouts and do
not change.  Outputs are bit-identical to the row-major path: the tiles land in shared memory the same way.
"""

from __future__ import annotations

import torch

from aklr_b200 import _lib

TILE = 128


def is_b200_tiled(t) -> bool:
    return bool(getattr(t, "is_b200_tiled", False))


def to_b200_tiled(w: torch.Tensor) -> torch.Tensor:
    """A new tensor of ``w``'s shape and dtype (1-byte elements, CUDA, contiguous, rows and cols multiples of
    128) whose storage holds the tile-contiguous layout, marked ``is_b200_tiled``.  Index it only through the
    ops: as a plain tensor its elements are permuted."""
    if is_b200_tiled(w):
        return w
    if not (w.is_cuda and w.is_contiguous() and w.element_size() == 1 and w.dim() >= 2):
        raise ValueError("a contiguous CUDA tensor of 1-byte elements [..., rows, cols] is needed")
    rows, cols = w.shape[-2:]
    if rows % TILE or cols % TILE:
        raise ValueError(f"rows and cols must be multiples of {TILE}, got {rows} x {cols}")
    out = torch.empty_like(w)
    matrices = w.numel() // (rows * cols)
    _lib.check(
        _lib.load().aklr_tile_weights_fp8(w.data_ptr(), out.data_ptr(), matrices, rows, cols, torch.cuda.current_stream(w.device).cuda_stream)
    )
    out.is_b200_tiled = True
    return out


def from_b200_tiled(w: torch.Tensor) -> torch.Tensor:
    """The row-major tensor a tile-contiguous one was made from (torch ops; for export and tests)."""
    *lead, rows, cols = w.shape
    tiles = w.reshape(*lead, rows // TILE, cols // TILE, TILE, TILE)
    n = len(lead)
    return tiles.permute(*range(n), n, n + 2, n + 1, n + 3).reshape(*lead, rows, cols).contiguous()
