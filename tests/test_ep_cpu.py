"""Expert-parallel host logic on CPU: two gloo ranks (and an in-process group) against the
single-process oracle on the concatenated tokens."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from aklr_b200 import workloads as wl
from aklr_b200.ep import ExpertParallelMoE, run_in_process
from aklr_b200.moe import Routing
from oracle import moe_oracle as orc
from tests.ep_oracle_kernels import OracleKernels

CFG = wl.MoEConfig("ep_small", hidden=256, inter=128, n_routed=16, topk=4, scoring="sigmoid", n_shared=1,
                   num_expert_group=4, topk_group=2, renormalize=True, routed_scaling_factor=2.5)
TOKENS = (5, 9)  # ragged: ranks hold different token counts


def routing() -> Routing:
    return Routing(CFG.topk, CFG.scoring, CFG.n_shared, CFG.num_expert_group, CFG.topk_group, True, CFG.routed_scaling_factor)


def rank_inputs(rank: int):
    hidden, logits, bias = wl.router_inputs(CFG, TOKENS[rank], seed=50 + rank)
    bias = wl.router_inputs(CFG, 1, seed=50)[2]  # the layer's bias is one tensor for all ranks
    return hidden, logits, bias


def rank_layer(rank: int, world: int, weights) -> ExpertParallelMoE:
    w1, s1, w2, s2 = weights
    n_local = CFG.n_routed // world
    mine = list(range(rank * n_local, (rank + 1) * n_local)) + [CFG.n_routed]
    return ExpertParallelMoE(routing(), w1[mine], s1[mine], w2[mine], s2[mine], rank, world, kernels=OracleKernels())


def reference_output(weights, rank: int) -> torch.Tensor:
    hidden, logits, bias = rank_inputs(rank)
    return orc.deepseek_v2_fp8_moe(hidden, None, bias, *weights, CFG.topk, CFG.num_expert_group, CFG.topk_group, True,
                                   CFG.routed_scaling_factor, logits=logits.float())


def check(out: torch.Tensor, ref: torch.Tensor) -> None:
    gates = orc.output_gates(out, ref)
    assert orc.gates_pass(gates, min_sqnr_db=40.0), gates


def test_in_process_group_matches_the_oracle():
    weights = wl.expert_weights(CFG, seed=60)
    layers = [rank_layer(r, 2, weights) for r in range(2)]
    outs = run_in_process(layers, [rank_inputs(r) for r in range(2)])
    for r in range(2):
        assert outs[r].shape == (TOKENS[r], CFG.hidden)
        check(outs[r], reference_output(weights, r))


def _worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        weights = wl.expert_weights(CFG, seed=60)
        out = rank_layer(rank, world, weights).forward(*rank_inputs(rank))
        # the same step as three interleaved parts gives every token the same result
        split = rank_layer(rank, world, weights).forward(*rank_inputs(rank), micro_batches=3)
        assert torch.equal(split, out)
        gates = orc.output_gates(out, reference_output(weights, rank))
        results.put((rank, tuple(out.shape), gates))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_the_oracle():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    got = [results.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, shape, gates in got:
        assert shape == (TOKENS[rank], CFG.hidden)
        assert orc.gates_pass(gates, min_sqnr_db=40.0), (rank, gates)


def test_router_width_must_match_the_group():
    weights = wl.expert_weights(CFG, seed=60)
    layer = rank_layer(0, 2, weights)
    hidden, logits, bias = rank_inputs(0)
    with pytest.raises(ValueError, match="the group holds"):
        layer.prepare(hidden, logits[:, :8].contiguous(), bias[:8].contiguous())
