"""The sort entry point that allocates nothing (collected last on purpose).

``aklr_moe_align_noalloc`` serves callers that cannot allocate device memory at the call site --
a frozen memory pool, a hook that only receives the engine's tensors, a language binding with no
allocator -- by keeping its histogram scratch in a 1 MiB array inside the library.  The test
calls it through the C ABI twice in a row on different inputs (the array keeps the first call's
contents) and checks every output against the existing ``aklr_moe_align`` bit for bit and against
the CPU oracle's sort, with and without an expert map, on the multi-pass and the one-CTA path.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sort(lib, entry, ids, n_experts, block_m, with_scratch, expert_map=None):
    from aklr_b200 import _lib

    device = ids.device
    n_routes = ids.numel()
    n_global = n_experts if expert_map is None else expert_map.numel()
    max_blocks = max(1, lib.aklr_moe_align_max_blocks(n_routes, n_experts, block_m))
    sorted_ids = torch.full((max_blocks * block_m,), -7, dtype=torch.int32, device=device)
    block_expert = torch.full((max_blocks,), -7, dtype=torch.int32, device=device)
    counts = torch.full((n_experts,), -7, dtype=torch.int32, device=device)
    num_blocks = torch.zeros(2, dtype=torch.int32, device=device)
    args = [ids.data_ptr(), None if expert_map is None else expert_map.data_ptr(), n_routes, n_experts, n_global, block_m,
            sorted_ids.data_ptr(), block_expert.data_ptr(), counts.data_ptr(), num_blocks.data_ptr()]
    if with_scratch:
        scratch = torch.empty(max(1, (n_routes + 1023) // 1024) * n_experts, dtype=torch.int32, device=device)
        args.append(scratch.data_ptr())
    args.append(torch.cuda.current_stream(device).cuda_stream)
    with torch.cuda.device(device):
        rc = entry(*args)
        if rc != 0:
            raise _lib.AklrError(rc, (lib.aklr_moe_align_noalloc_last_error() or lib.aklr_last_error()).decode())
        torch.cuda.synchronize(device)
    nb = int(num_blocks[0])
    return sorted_ids[: nb * block_m].cpu(), block_expert[:nb].cpu(), counts.cpu(), num_blocks.cpu()


def _routes(seed, n_tokens, n_experts, k, device):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(n_experts, generator=g)[:k] for _ in range(n_tokens)]).to(torch.int32).to(device)


def _check_against_both(lib, ids, n_experts, block_m, expert_map=None):
    from oracle import moe_oracle as orc

    want = _sort(lib, lib.aklr_moe_align, ids, n_experts, block_m, with_scratch=True, expert_map=expert_map)
    got = _sort(lib, lib.aklr_moe_align_noalloc, ids, n_experts, block_m, with_scratch=False, expert_map=expert_map)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    local = ids.cpu().long() if expert_map is None else expert_map.cpu().long()[ids.cpu().long()]
    ref_sorted, ref_blocks, ref_counts = orc.moe_align(local, n_experts, block_m)
    assert torch.equal(got[0], ref_sorted)
    assert torch.equal(got[1], ref_blocks)
    assert torch.equal(got[2].long(), ref_counts)
    assert got[3].tolist() == [ref_blocks.numel(), ref_blocks.numel() * block_m]


def test_noalloc_sort_matches_the_sort_with_caller_scratch_twice_in_a_row():
    from aklr_b200 import _lib

    lib = _lib.load()
    device = torch.device("cuda:0")
    launches = lib.aklr_kernel_launch_count()
    # both calls take the multi-pass path (> 4096 routes), the one that uses the scratch
    for seed, n_tokens, n_experts, k, block_m in [(1, 3000, 257, 9, 128), (2, 1500, 64, 6, 32)]:
        _check_against_both(lib, _routes(seed, n_tokens, n_experts, k, device), n_experts, block_m)
    assert lib.aklr_kernel_launch_count() - launches == 2 * (3 + 3)  # counted like aklr_moe_align's


def test_noalloc_sort_with_an_expert_map_and_on_the_one_cta_path():
    from aklr_b200 import _lib

    lib = _lib.load()
    device = torch.device("cuda:0")
    # a rank that holds every third of 96 global experts (the others' routes are dropped), > 4096 routes
    expert_map = torch.full((96,), -1, dtype=torch.int32)
    expert_map[::3] = torch.arange(32, dtype=torch.int32)
    _check_against_both(lib, _routes(3, 2000, 96, 4, device), 32, 64, expert_map.to(device))
    # <= 4096 routes: one CTA sorts, the scratch is not touched; still the same answer, twice
    for seed in (4, 5):
        _check_against_both(lib, _routes(seed, 300, 40, 5, device), 40, 16)


def test_noalloc_sort_keeps_one_scratch_address_per_device():
    """The array's device address differs per GPU: a second device, where there is one, gets its own."""
    from aklr_b200 import _lib

    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    lib = _lib.load()
    for index in (1, 0, 1):
        device = torch.device("cuda", index)
        _check_against_both(lib, _routes(10 + index, 2500, 128, 8, device), 128, 128)


def test_noalloc_sort_refuses_sizes_beyond_its_array():
    from aklr_b200 import _lib

    lib = _lib.load()
    device = torch.device("cuda:0")
    limit = lib.aklr_moe_align_noalloc_max_scratch_ints()
    assert limit == 262144
    n_experts = 1024
    n_routes = (limit // n_experts + 1) * 1024  # one chunk too many
    ids = torch.zeros(n_routes, dtype=torch.int32, device=device)
    with pytest.raises(_lib.AklrError, match="scratch ints"):
        _sort(lib, lib.aklr_moe_align_noalloc, ids, n_experts, 128, with_scratch=False)
