"""The sort entry point that allocates nothing (collected last on purpose).

``aklr_moe_align_noalloc`` serves callers that cannot allocate device memory at the call site --
a frozen memory pool, a hook that only receives the engine's tensors, a language binding with no
allocator -- by keeping its histogram scratch in a 1 MiB array inside the library.  The test
calls it through the C ABI twice in a row on different inputs (the array keeps the first call's
contents) and checks every output against the existing ``aklr_moe_align``, bit for bit.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sort(lib, entry, ids, n_experts, block_m, with_scratch):
    from aklr_b200 import _lib
    from aklr_b200.moe import _stream

    device = ids.device
    n_routes = ids.numel()
    max_blocks = max(1, lib.aklr_moe_align_max_blocks(n_routes, n_experts, block_m))
    sorted_ids = torch.full((max_blocks * block_m,), -7, dtype=torch.int32, device=device)
    block_expert = torch.full((max_blocks,), -7, dtype=torch.int32, device=device)
    counts = torch.full((n_experts,), -7, dtype=torch.int32, device=device)
    num_blocks = torch.zeros(2, dtype=torch.int32, device=device)
    args = [ids.data_ptr(), None, n_routes, n_experts, n_experts, block_m, sorted_ids.data_ptr(),
            block_expert.data_ptr(), counts.data_ptr(), num_blocks.data_ptr()]
    if with_scratch:
        scratch = torch.empty(max(1, (n_routes + 1023) // 1024) * n_experts, dtype=torch.int32, device=device)
        args.append(scratch.data_ptr())
    args.append(_stream())
    rc = entry(*args)
    if rc != 0:
        raise _lib.AklrError(rc, (lib.aklr_moe_align_noalloc_last_error() or lib.aklr_last_error()).decode())
    torch.cuda.synchronize()
    nb = int(num_blocks[0])
    return sorted_ids[: nb * block_m].cpu(), block_expert[:nb].cpu(), counts.cpu(), num_blocks.cpu()


def test_noalloc_sort_matches_the_sort_with_caller_scratch_twice_in_a_row():
    from aklr_b200 import _lib

    lib = _lib.load()
    device = torch.device("cuda:0")
    # both calls take the multi-pass path (> 4096 routes), the one that uses the scratch
    for seed, n_tokens, n_experts, k, block_m in [(1, 3000, 257, 9, 128), (2, 1500, 64, 6, 32)]:
        g = torch.Generator().manual_seed(seed)
        ids = torch.stack([torch.randperm(n_experts, generator=g)[:k] for _ in range(n_tokens)]).to(torch.int32).to(device)
        want = _sort(lib, lib.aklr_moe_align, ids, n_experts, block_m, with_scratch=True)
        got = _sort(lib, lib.aklr_moe_align_noalloc, ids, n_experts, block_m, with_scratch=False)
        for a, b in zip(got, want):
            assert torch.equal(a, b)


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
