"""Expert parallelism on the device: several ranks emulated phase by phase in one process on one
GPU (no kernel ever waits on another rank), against the single-GPU layer and the CPU oracle."""

from __future__ import annotations

import pytest
import torch

from aklr_b200 import workloads as wl
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu


def routing_of(cfg):
    from aklr_b200.moe import Routing

    return Routing(cfg.topk, cfg.scoring, cfg.n_shared, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor)


@pytest.mark.parametrize("world,tokens", [(2, (33, 7)), (4, (16, 1, 40, 5)), (8, (3,) * 8), (2, (600, 520))])
def test_emulated_ranks_match_single_gpu_and_oracle(world, tokens):
    from aklr_b200.ep import ExpertParallelMoE, run_in_process
    from aklr_b200.moe import fused_moe_fp8

    cfg = wl.CONFIGS["deepseek_small"]  # 64 routed experts + 1 shared
    d = torch.device("cuda:0")
    w1, s1, w2, s2 = (t.to(d) for t in wl.expert_weights(cfg, seed=70))
    bias = wl.router_inputs(cfg, 1, seed=71)[2].to(d)
    n_local = cfg.n_routed // world
    layers, inputs = [], []
    for r in range(world):
        mine = list(range(r * n_local, (r + 1) * n_local)) + [cfg.n_routed]
        layers.append(ExpertParallelMoE(routing_of(cfg), w1[mine].contiguous(), s1[mine].contiguous(), w2[mine].contiguous(), s2[mine].contiguous(), r, world))
        hidden, logits, _ = wl.router_inputs(cfg, tokens[r], seed=80 + r)
        inputs.append((hidden.to(d), logits.to(d), bias))
    outs = run_in_process(layers, inputs)
    torch.cuda.synchronize()
    for r in range(world):
        hidden, logits, _ = inputs[r]
        single = fused_moe_fp8(hidden, logits, bias, w1, s1, w2, s2, routing_of(cfg))
        ref = orc.deepseek_v2_fp8_moe(
            hidden.cpu(), None, bias.cpu(), w1.cpu(), s1.cpu(), w2.cpu(), s2.cpu(), cfg.topk, cfg.num_expert_group,
            cfg.topk_group, True, cfg.routed_scaling_factor, logits=logits.cpu().float(),
        )
        gates = orc.output_gates(outs[r].cpu(), ref)
        assert orc.gates_pass(gates), (r, gates)
        # one row per (token, rank): a rank's routes of a token are summed there and rounded to bf16 once more
        # than on one GPU, so the two agree closely, not bit for bit
        close = orc.output_gates(outs[r].cpu(), single.cpu().float())
        assert close["sqnr_db"] > 45.0, (r, close)


def test_a_token_sends_one_row_per_rank_it_reaches():
    """The plan counts (token, rank) pairs, not routes: with 8 groups of experts and 4 kept, at one group per
    rank a token reaches at most 4 of 8 ranks whatever its 8 routes are; the rows sent are exactly the distinct
    (token, rank) pairs of the routing, ordered by rank, and every pair's position is recorded."""
    from aklr_b200.ep import CudaKernels
    from aklr_b200.moe import route

    cfg = wl.CONFIGS["deepseek_small"]
    d = torch.device("cuda:0")
    world, n_local = 8, cfg.n_routed // 8
    _, logits, bias = wl.router_inputs(cfg, 300, seed=90)
    ids, _ = route(logits.to(d), bias.to(d), routing_of(cfg))
    ids = ids[:, : cfg.topk].contiguous()
    sorted_ids, counts, position, num_blocks = CudaKernels().plan(ids, n_local, world)
    torch.cuda.synchronize()
    ranks = ids.cpu().long() // n_local
    pairs = sorted({(t, int(r)) for t in range(300) for r in ranks[t].tolist()}, key=lambda p: (p[1], p[0]))
    assert int(num_blocks[1]) == len(pairs) <= 300 * 4
    assert counts.cpu().tolist() == [sum(1 for p in pairs if p[1] == r) for r in range(world)]
    sent = sorted_ids[: len(pairs)].cpu().long()
    assert [(int(rid) // cfg.topk, int(ranks.reshape(-1)[rid])) for rid in sent] == pairs
    assert (position.cpu() == -1).all()  # pack fills the positions in
