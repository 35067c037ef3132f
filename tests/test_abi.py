"""The C-ABI library: builds, loads, exports every symbol the header declares (no GPU needed)."""

from __future__ import annotations

import ctypes
import pathlib
import re

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from aklr_b200.csrc.build import build

    build()
    from aklr_b200 import _lib

    return _lib.load()


def declared_symbols() -> set[str]:
    text = (ROOT / "include" / "aklr_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(aklr_[a-z0-9_]+)\s*\(", text))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from aklr_b200 import _lib

    names = declared_symbols()
    assert names, "no declarations found in the header"
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert names == set(_lib.SIGNATURES), "the ctypes table and the header disagree"


def test_version_and_status_strings(lib):
    assert lib.aklr_abi_version() == 2
    assert lib.aklr_status_string(0) == b"ok"
    assert b"workspace" in lib.aklr_status_string(-2)


def test_workspace_layout_is_ordered_and_sized(lib):
    from aklr_b200._lib import MoeConfig, WorkspaceLayout

    cfg = MoeConfig(n_tokens=256, hidden=7168, inter=2048, n_routed=256, n_shared=1, topk=8, scoring=1,
                    num_expert_group=8, topk_group=4, renormalize=1, routed_scaling_factor=2.5)
    lay = WorkspaceLayout()
    assert lib.aklr_moe_fp8_workspace(ctypes.byref(cfg), ctypes.byref(lay)) == 0
    assert lay.block_m == 16 and lay.n_experts == 257
    assert lay.max_blocks == 256 * 9 // 16 + 257 and lay.capacity == lay.max_blocks * 16
    offsets = [lay.status, lay.num_blocks, lay.topk_ids, lay.topk_weights, lay.sorted_ids, lay.block_expert,
               lay.counts, lay.chunk_hist, lay.xq, lay.xs, lay.hq, lay.hs, lay.rows]
    assert offsets == sorted(offsets) and lay.total_bytes > lay.rows
    assert lay.xq % 1024 == 0 and lay.hq % 1024 == 0
    assert lay.total_bytes >= lay.rows + 256 * 9 * 7168 * 2


def test_automatic_block_size_follows_rows_per_expert(lib):
    """Small blocks (weight-major kernels) up to 28 routes per routed expert, never 64; 128-token blocks above."""
    from aklr_b200._lib import MoeConfig, WorkspaceLayout

    def picked(tokens, n_routed=256, topk=8):
        cfg = MoeConfig(n_tokens=tokens, hidden=7168, inter=2048, n_routed=n_routed, n_shared=1, topk=topk, scoring=1,
                        num_expert_group=8, topk_group=4, renormalize=1, routed_scaling_factor=2.5)
        lay = WorkspaceLayout()
        assert lib.aklr_moe_fp8_workspace(ctypes.byref(cfg), ctypes.byref(lay)) == 0
        return lay.block_m

    assert [picked(t) for t in (1, 8, 256, 320)] == [16, 16, 16, 16]
    assert [picked(t) for t in (352, 512, 704, 768, 895)] == [32, 32, 32, 32, 32]
    assert [picked(t) for t in (896, 1024, 4096, 16384)] == [128, 128, 128, 128]
    assert picked(64, n_routed=8, topk=2) == 32 and picked(128, n_routed=8, topk=2) == 128  # 16 and 32 routes per expert


def test_bad_shapes_are_refused_with_a_message(lib):
    from aklr_b200._lib import MoeConfig, WorkspaceLayout

    cfg = MoeConfig(n_tokens=4, hidden=100, inter=128, n_routed=8, topk=2)
    assert lib.aklr_moe_fp8_workspace(ctypes.byref(cfg), ctypes.byref(WorkspaceLayout())) == -4
    assert b"multiples of 128" in lib.aklr_last_error()
    cfg = MoeConfig(n_tokens=4, hidden=128, inter=128, n_routed=8, topk=2, block_m=48)
    assert lib.aklr_moe_fp8_workspace(ctypes.byref(cfg), ctypes.byref(WorkspaceLayout())) == -1


def test_max_blocks_bound(lib):
    assert lib.aklr_moe_align_max_blocks(9, 257, 16) == 9
    assert lib.aklr_moe_align_max_blocks(4096 * 9, 257, 128) == 288 + 257


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device refusal")
def test_compute_calls_fail_loudly_without_a_device():
    from aklr_b200 import moe

    x = torch.zeros((4, 128), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        moe.act_quant_fp8(x)
