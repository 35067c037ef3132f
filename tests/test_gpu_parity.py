"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and the golden fixtures.

Gates: routing ids, per-expert counts and sorted order bit-exact; routing weights abs/rel 1e-4;
FP8 codes and scales of the activation quantiser bit-exact; layer output max relative error
<= 2e-2 (per row, relative to the row's largest reference magnitude), cosine >= 0.9995 and whole-
output SQNR >= 30 dB against the float32 oracle rounded to bf16.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from aklr_b200 import workloads as wl
from oracle import moe_oracle as orc
from tests.golden import cases

pytestmark = pytest.mark.gpu

WEIGHT_TOL = 1e-4


def dev():
    return torch.device("cuda:0")


def t(a) -> torch.Tensor:
    return torch.from_numpy(np.asarray(a))


def routing_of(cfg: wl.MoEConfig):
    from aklr_b200.moe import Routing

    return Routing(
        topk=cfg.topk,
        scoring=cfg.scoring,
        n_shared=cfg.n_shared,
        num_expert_group=cfg.num_expert_group,
        topk_group=cfg.topk_group,
        renormalize=cfg.renormalize,
        routed_scaling_factor=cfg.routed_scaling_factor,
    )


def assert_routing(ids, weights, ref_ids, ref_weights):
    assert torch.equal(ids.cpu().long(), ref_ids.long()), "routing ids differ from the oracle"
    torch.testing.assert_close(weights.cpu(), ref_weights.float(), atol=WEIGHT_TOL, rtol=WEIGHT_TOL)


# ------------------------------------------------------------------------------------------------
# routing
# ------------------------------------------------------------------------------------------------
def test_grouped_sigmoid_routing_matches_golden(golden):
    from aklr_b200.moe import Routing, route

    logits, bias = cases.route_ds()
    r = Routing(topk=8, scoring="sigmoid", num_expert_group=8, topk_group=4, renormalize=True, routed_scaling_factor=2.5)
    ids, w = route(logits.to(dev()), bias.to(dev()), r)
    assert_routing(ids, w, t(golden["route_ds.ids"]), t(golden["route_ds.weights"]))
    r = Routing(topk=8, scoring="sigmoid", num_expert_group=8, topk_group=4, renormalize=False, routed_scaling_factor=1.0)
    ids, w = route(logits.to(dev()), bias.to(dev()), r)
    assert_routing(ids, w, t(golden["route_ds_norenorm.ids"]), t(golden["route_ds_norenorm.weights"]))


def test_tied_logits_route_to_the_lower_expert(golden):
    from aklr_b200.moe import Routing, route

    tied = cases.route_tied()
    r = Routing(topk=8, scoring="sigmoid", num_expert_group=8, topk_group=4, renormalize=True, routed_scaling_factor=2.5)
    ids, w = route(tied.to(dev()), torch.zeros(256, dtype=torch.bfloat16, device=dev()), r)
    assert_routing(ids, w, t(golden["route_tied.ids"]), t(golden["route_tied.weights"]))
    ids, w = route(tied[:, :128].contiguous().to(dev()), None, Routing(topk=8))
    assert_routing(ids, w, t(golden["route_tied_softmax.ids"]), t(golden["route_tied_softmax.weights"]))
    # the reference's known answer (tests/ops/test_reference.py:91-108): 1024 experts, float32 logits
    logits = torch.zeros(1, 1024)
    logits[0, [583, 571, 368, 31]] = 1.0
    r = Routing(topk=3, scoring="sigmoid", renormalize=False)
    ids, _ = route(logits.to(dev()), torch.zeros(1024, device=dev()), r)
    assert ids.cpu().tolist() == [[31, 368, 571]]


def test_float32_logits_route_like_the_oracle_up_to_near_ties():
    """Float32 logits (MiniMax-M2's gate, biased_grouped_topk on float32) are scored 1 / (1 + expf(-x)) on the
    device, which may differ from torch's CPU sigmoid in the last bit.  Over 24 seeded batches (256 experts, top-8,
    bias near 8 as the model holds it): every pick that differs from the oracle's sits on a near-tie -- the two
    biased scores involved are within 4 ulp of each other in the oracle -- and weights agree to 1e-6."""
    from aklr_b200.moe import Routing, route

    mismatched_tokens, checked, worst_gap = 0, 0, 0.0
    for seed in range(24):
        g = torch.Generator().manual_seed(9000 + seed)
        n_tokens = (1, 7, 64, 300, 1024, 2048)[seed % 6]
        logits = torch.randn(n_tokens, 256, generator=g) * (0.5 + 0.25 * (seed % 5))
        bias = 8.0 + 0.02 * torch.randn(256, generator=g)
        ref_ids, ref_w = orc.sigmoid_bias_topk(logits, bias, 8)
        ids, w = route(logits.to(dev()), bias.to(dev()), Routing(topk=8, scoring="sigmoid", renormalize=True))
        ids, w = ids.cpu().long(), w.cpu()
        checked += n_tokens
        biased = logits.sigmoid() + bias
        for tok in (ids != ref_ids).any(dim=-1).nonzero().flatten().tolist():
            mismatched_tokens += 1
            ours, theirs = set(ids[tok].tolist()), set(ref_ids[tok].tolist())
            if ours == theirs:  # the same experts in another order: two picks within the margin swapped places
                moved = [e for e, r in zip(ids[tok].tolist(), ref_ids[tok].tolist()) if e != r]
            else:
                moved = sorted(ours ^ theirs)
            scores = biased[tok, moved]
            gap = (scores.max() - scores.min()).item()
            worst_gap = max(worst_gap, gap)
            assert gap <= 4 * 2.0**-20, (seed, tok, moved, gap)  # 4 ulp of a value in [8, 16)
        same = (ids == ref_ids).all(dim=-1)
        torch.testing.assert_close(w[same], ref_w[same], atol=1e-6, rtol=1e-6)
    assert mismatched_tokens <= checked // 200, (mismatched_tokens, checked, worst_gap)


def test_softmax_routing_matches_golden(golden):
    from aklr_b200.moe import Routing, route

    cfg, logits = cases.route_qwen3()
    ids, w = route(logits.to(dev()), None, Routing(topk=cfg.topk))
    assert_routing(ids, w, t(golden["route_qwen3.ids"]), t(golden["route_qwen3.weights"]))


def test_standalone_biased_grouped_topk_matches_golden(golden):
    from aklr_b200.moe import Routing, route

    logits, bias = cases.bgt()
    r = Routing(topk=8, scoring="sigmoid", renormalize=True, routed_scaling_factor=2.5)
    ids, w = route(logits.to(dev()), bias.to(dev()), r)
    assert_routing(ids, w, t(golden["bgt.ids"]), t(golden["bgt.weights"]))


@pytest.mark.parametrize("n_tokens", [1, 2, 3, 31, 33, 127, 129, 1000])
@pytest.mark.parametrize("name", ["deepseek_v3", "qwen3", "mixtral"])
def test_routing_matches_oracle_on_ragged_batches(name, n_tokens):
    from aklr_b200.moe import route

    cfg = wl.CONFIGS[name]
    _, logits, bias = wl.router_inputs(cfg, n_tokens, seed=n_tokens)
    if cfg.scoring == "sigmoid":
        ref_ids, ref_w = orc.grouped_sigmoid_topk(
            logits.float(), bias.float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, True, cfg.routed_scaling_factor
        )
        ref_ids, ref_w = orc.with_shared_slot(ref_ids, ref_w, cfg.n_routed)
    else:
        ref_ids, ref_w = orc.softmax_topk(logits.float(), cfg.topk)
    ids, w = route(logits.to(dev()), None if bias is None else bias.to(dev()), routing_of(cfg))
    assert_routing(ids, w, ref_ids, ref_w)


@pytest.mark.parametrize("n_tokens", [5, 2100])  # routed by counting (one CTA per token) / by warp reductions
@pytest.mark.parametrize(
    "shape",
    [
        dict(n_routed=40, topk=3),                                             # not a multiple of 32
        dict(n_routed=8, topk=8),                                              # every expert picked
        dict(n_routed=1024, topk=31, n_shared=1),                              # the widest table
        dict(n_routed=72, topk=5, n_shared=2, scoring="sigmoid", num_expert_group=4, topk_group=2,
             renormalize=True, routed_scaling_factor=1.5),                    # groups of 18, two shared slots
        dict(n_routed=96, topk=6, scoring="sigmoid", num_expert_group=3, topk_group=3, renormalize=False),  # all groups kept
        dict(n_routed=8, topk=3, scoring="sigmoid", num_expert_group=8, topk_group=8, renormalize=True),    # one expert per group, all kept
    ],
)
def test_routing_on_odd_shapes(shape, n_tokens):
    from aklr_b200.moe import route

    cfg = wl.MoEConfig("odd", hidden=128, inter=128, **shape)
    _, logits, bias = wl.router_inputs(cfg, n_tokens, seed=17 + n_tokens)
    if cfg.scoring == "sigmoid" and cfg.n_routed == cfg.num_expert_group:
        # one expert per group, every group kept: the standalone op's statement, which forms no group score
        ref_w, ref_ids = orc.biased_grouped_topk(logits.float(), bias.float(), cfg.topk, cfg.renormalize, cfg.routed_scaling_factor)
        ref_ids = ref_ids.long()
    elif cfg.scoring == "sigmoid":
        ref_ids, ref_w = orc.grouped_sigmoid_topk(
            logits.float(), bias.float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor
        )
    else:
        ref_ids, ref_w = orc.softmax_topk(logits.float(), cfg.topk)
    for k in range(cfg.n_shared):  # shared experts follow the routed ones at weight 1
        ref_ids = torch.cat([ref_ids, torch.full_like(ref_ids[:, :1], cfg.n_routed + k)], dim=-1)
        ref_w = torch.cat([ref_w, torch.ones_like(ref_w[:, :1])], dim=-1)
    ids, w = route(logits.to(dev()), None if bias is None else bias.to(dev()), routing_of(cfg))
    assert_routing(ids, w, ref_ids, ref_w)


# ------------------------------------------------------------------------------------------------
# sort
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize(
    "n_tokens,n_experts,k,block_m",
    [(1, 257, 9, 16), (7, 8, 2, 16), (64, 8, 2, 32), (256, 257, 9, 16), (455, 257, 9, 32), (456, 128, 8, 64), (3000, 257, 9, 128), (20000, 64, 6, 128)],
)
def test_moe_align_matches_oracle(n_tokens, n_experts, k, block_m):
    from aklr_b200.moe import moe_align

    g = torch.Generator().manual_seed(n_tokens)
    ids = torch.stack([torch.randperm(n_experts, generator=g)[:k] for _ in range(n_tokens)]).to(torch.int32)
    sorted_ids, block_expert, counts, nb = moe_align(ids.to(dev()), n_experts, block_m)
    ref_sorted, ref_blocks, ref_counts = orc.moe_align(ids, n_experts, block_m)
    assert torch.equal(counts.cpu().long(), ref_counts)
    assert nb == ref_blocks.numel()
    assert torch.equal(block_expert.cpu(), ref_blocks)
    assert torch.equal(sorted_ids.cpu(), ref_sorted)


def test_moe_align_with_an_expert_map_drops_other_ranks_routes():
    from aklr_b200.moe import moe_align

    g = torch.Generator().manual_seed(3)
    ids = torch.stack([torch.randperm(32, generator=g)[:4] for _ in range(300)]).to(torch.int32)
    expert_map = torch.full((32,), -1, dtype=torch.int32)
    expert_map[8:16] = torch.arange(8, dtype=torch.int32)  # this rank holds global experts 8..15
    sorted_ids, block_expert, counts, nb = moe_align(ids.to(dev()), 8, 16, expert_map.to(dev()))
    local = torch.where((ids >= 8) & (ids < 16), ids - 8, -1)
    ref_sorted, ref_blocks, ref_counts = orc.moe_align(local, 8, 16)
    assert torch.equal(counts.cpu().long(), ref_counts)
    assert torch.equal(block_expert.cpu(), ref_blocks)
    assert torch.equal(sorted_ids.cpu(), ref_sorted)


# ------------------------------------------------------------------------------------------------
# quantisers
# ------------------------------------------------------------------------------------------------
def test_activation_quant_is_bit_exact():
    from aklr_b200.moe import act_quant_fp8

    x = wl.normal(5, "x", (67, 1024), 1.0, dtype=torch.bfloat16)
    x[3] = 0
    x[5, :128] *= 1e-30
    x[7] *= 300.0
    q, s = act_quant_fp8(x.to(dev()))
    ref_q, ref_s = orc.fp8_group_quant(x.float())
    assert torch.equal(s.cpu(), ref_s)
    assert torch.equal(q.cpu().view(torch.uint8), ref_q.view(torch.uint8))


def test_standalone_quant_ops_match_golden(golden):
    from aklr_b200.moe import per_group_quant_fp8, per_group_quant_mxfp8

    x = cases.quant_x().to(dev())
    q, s = per_group_quant_fp8(x)
    assert torch.equal(q.cpu().float(), t(golden["quant_fp8.q"]))
    assert torch.equal(s.cpu(), t(golden["quant_fp8.s"]))
    q, s = per_group_quant_mxfp8(x)
    assert torch.equal(q.cpu().float(), t(golden["quant_mxfp8.q"]))
    assert torch.equal(s.cpu(), t(golden["quant_mxfp8.s"]))


def test_router_gemm_rounds_like_the_oracle():
    from aklr_b200.moe import router_logits

    cfg, a = cases.tiny_layer()
    got = router_logits(a["hidden_states"].to(dev()), a["router_weight"].to(dev())).cpu().float()
    ref = orc.router_logits(a["hidden_states"], a["router_weight"])
    # float32 sums in another order may land one bf16 step away
    step = ref.abs().clamp_min(1e-3) * 2.0**-7
    assert ((got - ref).abs() <= step).all()
    assert (got == ref).float().mean() > 0.97


# ------------------------------------------------------------------------------------------------
# whole layer
# ------------------------------------------------------------------------------------------------
def run_layer(cfg, args, logits, block_m, variant=0):
    from aklr_b200.moe import fused_moe_fp8

    d = dev()
    bias = args.get("correction_bias")
    out, ws = fused_moe_fp8(
        args["hidden_states"].to(d),
        logits.to(torch.bfloat16).to(d),
        None if bias is None else bias.to(d),
        args["w1"].to(d),
        args["w1_scale"].to(d),
        args["w2"].to(d),
        args["w2_scale"].to(d),
        routing_of(cfg),
        block_m=block_m,
        return_workspace=True,
        variant=variant,
    )
    ws.check_status()
    return out, ws


def check_intermediates(cfg, args, ws, ref_ids):
    """Sorted order, counts, first quantisation bit-exact; second quantisation nearly so."""
    ids = ws.topk_ids().cpu()
    assert torch.equal(ids.long(), ref_ids)
    ref_sorted, ref_blocks, ref_counts = orc.moe_align(ids, cfg.n_experts, ws.layout.block_m)
    assert torch.equal(ws.counts().cpu().long(), ref_counts)
    assert torch.equal(ws.block_expert().cpu(), ref_blocks)
    assert torch.equal(ws.sorted_ids().cpu(), ref_sorted)
    xq, xs = ws.xq()
    rows = (ref_sorted >= 0).nonzero().flatten()
    tokens = ref_sorted[rows].long() // cfg.routes_per_token
    ref_q, ref_s = orc.fp8_group_quant(args["hidden_states"].float())
    assert torch.equal(xs.cpu()[rows], ref_s[tokens])
    assert torch.equal(xq.cpu().view(torch.uint8)[rows], ref_q.view(torch.uint8)[tokens])


@pytest.mark.parametrize("block_m", [16, 32, 64, 128, 0])
def test_tiny_layer_matches_golden(golden, block_m):
    cfg, a = cases.tiny_layer()
    out, ws = run_layer(cfg, a, t(golden["tiny.logits"]), block_m)
    check_intermediates(cfg, a, ws, t(golden["tiny.ids"]))
    gates = orc.output_gates(out.cpu(), t(golden["tiny.out"]))
    assert orc.gates_pass(gates), gates


@pytest.mark.parametrize("block_m", [16, 64, 0])
def test_deepseek_small_layer_matches_golden(golden, block_m):
    cfg, a = cases.ds_small_layer()
    out, ws = run_layer(cfg, a, t(golden["ds_small.logits"]), block_m)
    check_intermediates(cfg, a, ws, t(golden["ds_small.ids"]))
    gates = orc.output_gates(out.cpu(), t(golden["ds_small.out"]))
    assert orc.gates_pass(gates), gates


def test_layer_from_hidden_states_through_the_router_gemm(golden):
    """Router GEMM on the device: ids may differ from the oracle's only where two logits are
    one bf16 step apart; the output still has to pass the float gates."""
    from aklr_b200.moe import fused_moe_fp8, router_logits

    cfg, a = cases.tiny_layer()
    d = dev()
    logits = router_logits(a["hidden_states"].to(d), a["router_weight"].to(d))
    out = fused_moe_fp8(
        a["hidden_states"].to(d), logits, None, a["w1"].to(d), a["w1_scale"].to(d), a["w2"].to(d), a["w2_scale"].to(d), routing_of(cfg)
    )
    ref = orc.qwen3_moe_fp8_moe(
        a["hidden_states"], a["router_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], cfg.topk, logits=logits.cpu().float()
    )
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates


@pytest.mark.parametrize("n_tokens", [1, 2, 3, 31, 33, 129])
def test_ragged_token_counts(n_tokens):
    cfg = wl.CONFIGS["deepseek_small"]
    hidden, logits, bias = wl.router_inputs(cfg, n_tokens, seed=100 + n_tokens)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=9)
    a = dict(hidden_states=hidden, correction_bias=bias, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2)
    out, ws = run_layer(cfg, a, logits, 0)
    ref = orc.deepseek_v2_fp8_moe(
        hidden, None, bias, w1, s1, w2, s2, cfg.topk, cfg.num_expert_group, cfg.topk_group, True, 2.5, logits=logits.float()
    )
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates


def test_empty_batch_is_a_no_op():
    from aklr_b200.moe import fused_moe_fp8

    cfg = wl.CONFIGS["tiny"]
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=9)
    d = dev()
    out = fused_moe_fp8(
        torch.empty((0, cfg.hidden), dtype=torch.bfloat16, device=d),
        torch.empty((0, cfg.n_routed), dtype=torch.bfloat16, device=d),
        None, w1.to(d), s1.to(d), w2.to(d), s2.to(d), routing_of(cfg),
    )
    assert out.shape == (0, cfg.hidden)


def test_qwen3_shaped_layer_with_skewed_routing():
    cfg = wl.CONFIGS["qwen3"]
    n_tokens = 256
    hidden, logits, _ = wl.router_inputs(cfg, n_tokens, seed=21)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=22)
    a = dict(hidden_states=hidden, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2)
    out, ws = run_layer(cfg, a, logits, 0)
    ref_ids, _ = orc.softmax_topk(logits.float(), cfg.topk)
    check_intermediates(cfg, a, ws, ref_ids)
    ref = orc.qwen3_moe_fp8_moe(hidden, None, w1, s1, w2, s2, cfg.topk, logits=logits.float())
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates


def test_experts_only_entry_with_an_expert_map():
    """One rank's share under replicated-token expert parallelism: routes to experts the rank
    does not hold add nothing (aklr/ops/fused_moe/reference.py:78-84)."""
    from aklr_b200.moe import fused_experts_fp8

    cfg = wl.CONFIGS["tiny"]
    hidden, logits, _ = wl.router_inputs(cfg, 40, seed=31)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=32)
    ids, weights = orc.softmax_topk(logits.float(), cfg.topk)
    d = dev()
    lo, hi = 2, 6  # this rank holds global experts 2..5
    expert_map = torch.full((cfg.n_routed,), -1, dtype=torch.int32)
    expert_map[lo:hi] = torch.arange(hi - lo, dtype=torch.int32)
    out = fused_experts_fp8(
        hidden.to(d), ids.to(torch.int32).to(d), weights.to(d), w1[lo:hi].to(d), s1[lo:hi].to(d), w2[lo:hi].to(d), s2[lo:hi].to(d),
        expert_map=expert_map.to(d),
    )
    local = torch.where((ids >= lo) & (ids < hi), ids - lo, -1)
    ref = orc.fp8_experts(hidden, local, weights, w1[lo:hi], s1[lo:hi], w2[lo:hi], s2[lo:hi])
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates


class _LazyExperts:
    """Indexable like a weight tensor on the host, fetching one expert from the device at a time."""

    def __init__(self, device_tensor):
        self.t = device_tensor

    def __getitem__(self, e):
        return self.t[e].cpu()


@pytest.mark.parametrize("n_tokens", [64, 4096])
def test_deepseek_v3_full_width_on_sampled_tokens(n_tokens):
    """Full DeepSeek-V3 widths (11 GB of expert weights drawn on the device).  A token's output
    depends on that token alone, so the oracle checks a sample of tokens exactly as it would
    check all of them; ids and counts are checked for the whole batch."""
    from aklr_b200.moe import fused_moe_fp8

    cfg = wl.CONFIGS["deepseek_v3"]
    d = dev()
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=41, device=d)
    hidden, logits, bias = wl.router_inputs(cfg, n_tokens, seed=42)
    out, ws = fused_moe_fp8(hidden.to(d), logits.to(d), bias.to(d), w1, s1, w2, s2, routing_of(cfg), return_workspace=True)
    ws.check_status()
    ref_ids, ref_w = orc.grouped_sigmoid_topk(logits.float(), bias.float(), 8, 8, 4, True, 2.5)
    ref_ids, ref_w = orc.with_shared_slot(ref_ids, ref_w, cfg.n_routed)
    assert torch.equal(ws.topk_ids().cpu().long(), ref_ids)
    assert torch.equal(ws.counts().cpu().long(), torch.bincount(ref_ids.flatten(), minlength=cfg.n_experts))
    sample = torch.tensor([0, n_tokens // 3, n_tokens - 1])
    ref = orc.fp8_experts(
        hidden[sample], ref_ids[sample], ref_w[sample], _LazyExperts(w1), _LazyExperts(s1), _LazyExperts(w2), _LazyExperts(s2)
    )
    gates = orc.output_gates(out[sample.to(d)].cpu(), ref)
    assert orc.gates_pass(gates), gates
    # permuting the tokens permutes the output rows bit for bit
    perm = torch.randperm(n_tokens, generator=torch.Generator().manual_seed(1))
    out2 = fused_moe_fp8(hidden[perm].to(d), logits[perm].to(d), bias.to(d), w1, s1, w2, s2, routing_of(cfg))
    assert torch.equal(out2.cpu(), out.cpu()[perm])


@pytest.mark.parametrize("n_tokens", [16, 1024])
def test_mixtral_full_width_on_sampled_tokens(n_tokens):
    """Mixtral-8x7B widths (hidden 4096, intermediate 14336, 8 experts, top-2 softmax): the long
    reduction of the down projection (112 K-blocks) through the weight-major (16 tokens) and the
    token-major (1024 tokens) kernels, against the oracle on a sample of tokens."""
    from aklr_b200.moe import fused_moe_fp8

    cfg = wl.CONFIGS["mixtral"]
    d = dev()
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=51, device=d)
    hidden, logits, _ = wl.router_inputs(cfg, n_tokens, seed=52)
    out, ws = fused_moe_fp8(hidden.to(d), logits.to(d), None, w1, s1, w2, s2, routing_of(cfg), return_workspace=True)
    ws.check_status()
    ref_ids, ref_w = orc.softmax_topk(logits.float(), cfg.topk)
    assert torch.equal(ws.topk_ids().cpu().long(), ref_ids)
    assert torch.equal(ws.counts().cpu().long(), torch.bincount(ref_ids.flatten(), minlength=cfg.n_experts))
    sample = torch.tensor([0, n_tokens // 2, n_tokens - 1])
    ref = orc.fp8_experts(
        hidden[sample], ref_ids[sample], ref_w[sample], _LazyExperts(w1), _LazyExperts(s1), _LazyExperts(w2), _LazyExperts(s2)
    )
    gates = orc.output_gates(out[sample.to(d)].cpu(), ref)
    assert orc.gates_pass(gates), gates


def test_token_major_and_weight_major_kernels_agree(golden):
    """Full 128-token blocks run the token-major grouped GEMM; forcing the weight-major one on the
    same inputs must pass the same gates and agree closely."""
    from aklr_b200 import _lib

    cfg, a = cases.ds_small_layer()
    out_tm, ws = run_layer(cfg, a, t(golden["ds_small.logits"]), 128)
    check_intermediates(cfg, a, ws, t(golden["ds_small.ids"]))
    out_wm, _ = run_layer(cfg, a, t(golden["ds_small.logits"]), 128, variant=_lib.VARIANT_WEIGHT_MAJOR)
    for out in (out_tm, out_wm):
        gates = orc.output_gates(out.cpu(), t(golden["ds_small.out"]))
        assert orc.gates_pass(gates), gates
    close = orc.output_gates(out_tm.cpu(), out_wm.cpu().float())
    assert close["sqnr_db"] > 45.0, close


def test_cta_pair_kernels_match_the_single_cta_kernels(golden):
    """The CTA-pair (cta_group::2) grouped GEMMs take two token blocks of an expert per pair and read
    half of the weight tile from each CTA; per element the arithmetic is the single-CTA kernel's.
    Token counts are chosen so experts end up with one, two and three blocks (odd runs included)."""
    from aklr_b200 import _lib
    from aklr_b200.moe import fused_moe_fp8

    cfg, a = cases.ds_small_layer()
    out_single, ws = run_layer(cfg, a, t(golden["ds_small.logits"]), 128)
    out_pair, ws_pair = run_layer(cfg, a, t(golden["ds_small.logits"]), 128, variant=_lib.VARIANT_CTA_PAIRS)
    assert torch.equal(out_pair.cpu(), out_single.cpu())
    gates = orc.output_gates(out_pair.cpu(), t(golden["ds_small.out"]))
    assert orc.gates_pass(gates), gates

    # a batch large enough for several blocks per expert, against the same call without pairs
    cfg = wl.CONFIGS["deepseek_small"]
    d = dev()
    w1, s1, w2, s2 = (x.to(d) for x in wl.expert_weights(cfg, seed=5))
    hidden, logits, bias = (x.to(d) for x in wl.router_inputs(cfg, 1500, seed=6))
    outs = []
    for variant in (0, _lib.VARIANT_CTA_PAIRS):
        out, ws = fused_moe_fp8(hidden, logits, bias, w1, s1, w2, s2, routing_of(cfg), block_m=128, return_workspace=True, variant=variant)
        ws.check_status()
        outs.append(out.cpu())
        blocks = ws.num_blocks()
    assert blocks > cfg.n_routed  # some experts have more than one block
    assert torch.equal(outs[0], outs[1])


def test_padding_rows_of_128_token_blocks_carry_zero_codes():
    """The token-major GEMMs multiply a block's padding rows like any others; what they hold is never read back, but
    the tensor core's draw depends on it, so the gather and the gate_up epilogue write zero codes there.  Routed rows
    keep their codes (the output still passes against the same call on 16-token blocks, which has no such rows)."""
    from aklr_b200.moe import fused_moe_fp8

    cfg = wl.CONFIGS["deepseek_small"]
    d = dev()
    w1, s1, w2, s2 = (x.to(d) for x in wl.expert_weights(cfg, seed=5))
    hidden, logits, bias = (x.to(d) for x in wl.router_inputs(cfg, 700, seed=9))
    outs = {}
    for bm in (128, 16):
        # a call on other tokens first: the call under test then finds that call's codes where its padding falls
        ws = None
        for h, l in ((hidden.flip(0).contiguous(), logits.flip(0).contiguous()), (hidden, logits)):
            out, ws = fused_moe_fp8(h, l, bias, w1, s1, w2, s2, routing_of(cfg), block_m=bm, return_workspace=True, workspace=ws)
        ws.check_status()
        outs[bm] = out.float().cpu()
        if bm == 128:
            ids = ws.sorted_ids().cpu()
            padding = ids < 0
            assert padding.any() and (~padding).any()
            n = ids.numel()
            for name, (codes, _) in (("activations", ws.xq()), ("gated product", ws.hq())):
                as_bytes = codes[:n].view(torch.uint8).cpu()
                assert int(as_bytes[padding].max()) == 0, name
                assert int((as_bytes[~padding] != 0).sum()) > 0, name
    gates = orc.output_gates(outs[128], outs[16])
    assert orc.gates_pass(gates), gates


def test_deep_pipeline_kernels_match_the_two_buffer_kernels(golden):
    """128 x 128 tiles with four partials in flight: per element the same float32 operations in the same order
    as the 128 x 256 kernels, so outputs are bit-identical -- on the golden layer, on a batch with several blocks
    per expert, and on a width whose down projection has an odd K-block count (inter 640 -> 5)."""
    from aklr_b200 import _lib
    from aklr_b200.moe import Routing, fused_moe_fp8

    cfg, a = cases.ds_small_layer()
    out_ref, _ = run_layer(cfg, a, t(golden["ds_small.logits"]), 128)
    out_deep, ws = run_layer(cfg, a, t(golden["ds_small.logits"]), 128, variant=_lib.VARIANT_DEEP_PIPELINE)
    check_intermediates(cfg, a, ws, t(golden["ds_small.ids"]))
    assert torch.equal(out_deep.cpu(), out_ref.cpu())

    d = dev()
    shapes = [wl.CONFIGS["deepseek_small"], wl.MoEConfig("odd_k", hidden=768, inter=640, n_routed=8, topk=2)]
    for cfg, n_tokens in zip(shapes, (1500, 900)):
        w1, s1, w2, s2 = (x.to(d) for x in wl.expert_weights(cfg, seed=5))
        hidden, logits, bias = wl.router_inputs(cfg, n_tokens, seed=6)
        bias = bias.to(d) if cfg.scoring == "sigmoid" else None
        outs = []
        for variant in (0, _lib.VARIANT_DEEP_PIPELINE):
            out, ws = fused_moe_fp8(hidden.to(d), logits.to(d), bias, w1, s1, w2, s2, routing_of(cfg), block_m=128,
                                    return_workspace=True, variant=variant)
            ws.check_status()
            outs.append(out.cpu())
        assert ws.num_blocks() > cfg.n_routed
        assert torch.equal(outs[0], outs[1]), cfg.name


@pytest.mark.parametrize("name", ["deepseek_small", "qwen3", "eight_experts"])
@pytest.mark.parametrize("n_tokens", [1, 3, 8])
def test_decode_prologue_kernel_matches_the_separate_kernels(name, n_tokens):
    """One to eight tokens: routing and sort run as one kernel.  Everything it leaves in the workspace,
    and the layer output, equals bit for bit what the two kernels leave."""
    from aklr_b200 import _lib
    from aklr_b200.moe import fused_moe_fp8

    lib = _lib.load()
    # eight experts, top-2 softmax: Mixtral's routing shape, a team of 256 threads with 8 at work
    cfg = wl.CONFIGS.get(name) or wl.MoEConfig(name, hidden=256, inter=128, n_routed=8, topk=2)
    d = dev()
    w1, s1, w2, s2 = (x.to(d) for x in wl.expert_weights(cfg, seed=21))
    hidden, logits, bias = wl.router_inputs(cfg, n_tokens, seed=300 + n_tokens)
    bias_d = bias.to(d) if bias is not None and cfg.scoring == "sigmoid" else None
    got = []
    for variant in (0, _lib.VARIANT_SEPARATE_PROLOGUE):
        launches = lib.aklr_kernel_launch_count()
        out, ws = fused_moe_fp8(hidden.to(d), logits.to(d), bias_d, w1, s1, w2, s2, routing_of(cfg), return_workspace=True, variant=variant)
        ws.check_status()
        rows = ws.num_blocks() * ws.layout.block_m
        xq, xs = ws.xq()
        live = ws.sorted_ids()[:rows].cpu() >= 0
        got.append(dict(out=out.cpu(), ids=ws.topk_ids().cpu(), weights=ws.topk_weights().cpu(), counts=ws.counts().cpu(),
                        sorted=ws.sorted_ids()[:rows].cpu(), block_expert=ws.block_expert().cpu(),
                        xq=xq[:rows].cpu().view(torch.uint8)[live], xs=xs[:rows].cpu()[live],
                        launches=lib.aklr_kernel_launch_count() - launches))
    one, three = got
    assert one["launches"] == three["launches"] - 1
    for key in ("ids", "weights", "counts", "sorted", "block_expert", "xq", "xs", "out"):
        assert torch.equal(one[key], three[key]), key
    ref_ids = orc.grouped_sigmoid_topk(logits.float(), bias.float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, True, cfg.routed_scaling_factor)[0] \
        if cfg.scoring == "sigmoid" else orc.softmax_topk(logits.float(), cfg.topk)[0]
    assert torch.equal(one["ids"][:, : cfg.topk].long(), ref_ids)


def test_layer_call_is_cuda_graph_capturable():
    """No allocation, synchronisation or host read inside the call: it can be captured once a shape
    has run eagerly, and a replay on new input values gives what the eager call gives."""
    from aklr_b200.moe import Workspace, _config, fused_moe_fp8

    cfg = wl.CONFIGS["deepseek_small"]
    d = dev()
    w1, s1, w2, s2 = (x.to(d) for x in wl.expert_weights(cfg, seed=9))
    hidden, logits, bias = (x.to(d) for x in wl.router_inputs(cfg, 24, seed=1))
    routing = routing_of(cfg)
    ws = Workspace(_config(24, cfg.hidden, cfg.inter, cfg.n_routed, routing, logits, bias), d)
    out = torch.empty_like(hidden)
    fused_moe_fp8(hidden, logits, bias, w1, s1, w2, s2, routing, out=out, workspace=ws)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fused_moe_fp8(hidden, logits, bias, w1, s1, w2, s2, routing, out=out, workspace=ws)
    hidden2, logits2, _ = (x.to(d) for x in wl.router_inputs(cfg, 24, seed=2))
    hidden.copy_(hidden2)
    logits.copy_(logits2)
    graph.replay()
    torch.cuda.synchronize()
    replayed = out.clone()
    eager = fused_moe_fp8(hidden2, logits2, bias, w1, s1, w2, s2, routing)
    assert torch.equal(replayed, eager)
    ws.check_status()


@pytest.mark.parametrize("n_tokens,hidden,experts", [(300, 1024, 256), (64, 512, 40), (1000, 7168, 257), (5, 512, 64), (40, 256, 8)])
def test_router_gemm_paths_round_like_the_oracle(n_tokens, hidden, experts):
    """Tensor-core path (>= 64 tokens, ragged tiles, expert counts that are not tile multiples) and the
    warp-per-dot-product path for few tokens."""
    from aklr_b200.moe import router_logits

    x = wl.normal(1, "x", (n_tokens, hidden), 1.0, dtype=torch.bfloat16)
    w = wl.normal(2, "w", (experts, hidden), 0.05, dtype=torch.bfloat16)
    got = router_logits(x.to(dev()), w.to(dev())).cpu().float()
    ref = orc.router_logits(x, w)
    step = ref.abs().clamp_min(1e-2) * 2.0**-7
    assert ((got - ref).abs() <= step).all()
    assert (got == ref).float().mean() > 0.95


def test_tile_contiguous_weights_give_the_row_major_results():
    """The load-time converter against the torch statement of the layout, and the layer on tile-contiguous
    weights against the same call on row-major ones, bit for bit: decode blocks (weight-major kernel), full
    blocks (token-major kernel, whose down projection then takes its 256 rows as two tiles) and the 128 x 128-tile
    variant (64-row boxes inside a tile)."""
    from aklr_b200 import _lib, layouts
    from aklr_b200.moe import fused_experts_fp8, fused_moe_fp8

    d = dev()
    cfg = wl.CONFIGS["deepseek_small"]
    w1, s1, w2, s2 = (x.to(d) for x in wl.expert_weights(cfg, seed=11))
    t1, t2 = layouts.to_b200_tiled(w1), layouts.to_b200_tiled(w2)
    assert layouts.is_b200_tiled(t1) and t1.shape == w1.shape and t1.dtype == w1.dtype
    e, rows, cols = w1.shape
    expect = w1.view(torch.uint8).reshape(e, rows // 128, 128, cols // 128, 128).permute(0, 1, 3, 2, 4).contiguous()
    assert torch.equal(t1.view(torch.uint8).reshape(expect.shape), expect)
    assert torch.equal(layouts.from_b200_tiled(t1.view(torch.uint8)), w1.view(torch.uint8))
    assert layouts.to_b200_tiled(t1) is t1
    for n_tokens, variant in ((5, 0), (40, 0), (300, 0), (1500, 0), (1500, _lib.VARIANT_DEEP_PIPELINE)):
        hidden, logits, bias = (x.to(d) for x in wl.router_inputs(cfg, n_tokens, seed=12 + n_tokens))
        outs = []
        for a, b in ((w1, w2), (t1, t2)):
            out, ws = fused_moe_fp8(hidden, logits, bias, a, s1, b, s2, routing_of(cfg), return_workspace=True, variant=variant)
            ws.check_status()
            outs.append(out.cpu())
        assert torch.equal(outs[0], outs[1]), (n_tokens, variant, ws.layout.block_m)
    # routing given (the experts-only entry point), and a mixed pair is refused
    ids = torch.stack([torch.randperm(cfg.n_experts)[:4] for _ in range(64)]).to(torch.int32).to(d)
    wts = torch.rand(64, 4).to(d)
    x = wl.router_inputs(cfg, 64, seed=3)[0].to(d)
    assert torch.equal(fused_experts_fp8(x, ids, wts, t1, s1, t2, s2).cpu(), fused_experts_fp8(x, ids, wts, w1, s1, w2, s2).cpu())
    with pytest.raises(ValueError, match="same layout"):
        fused_experts_fp8(x, ids, wts, t1, s1, w2, s2)


def test_quantiser_division_shortcut_is_the_ieee_division():
    """The layer's quantiser computes x / scale as q + (x - q*scale) * (1/scale) with q = x * (1/scale).  Against
    __fdiv_rn over 64 M pairs: bf16 values of every magnitude over scales as the quantiser forms them (amax / 448),
    scales with an all-ones significand, the smallest scale it can use (FLT_MIN) and very large ones -- no bit differs."""
    import ctypes

    from aklr_b200 import _lib

    lib = _lib.load()
    d = dev()
    g = torch.Generator(device=d).manual_seed(77)
    n = 1 << 24
    total = 0
    for kind in range(4):
        amax = torch.randn(n, generator=g, device=d).abs() * torch.exp2(torch.randint(-40, 40, (n,), generator=g, device=d).float())
        scale = (amax.to(torch.bfloat16).float() / 448.0).clamp_min(torch.finfo(torch.float32).tiny)
        if kind == 1:  # all-ones significands
            scale = (scale.view(torch.int32) | 0x7FFFFF).view(torch.float32)
        elif kind == 2:  # the floor and its neighbourhood
            scale = torch.where(torch.rand(n, generator=g, device=d) < 0.5, torch.full_like(scale, torch.finfo(torch.float32).tiny), scale * 2.0**-100).clamp_min(torch.finfo(torch.float32).tiny)
        elif kind == 3:
            scale = scale * 2.0**80
        x = (torch.rand(n, generator=g, device=d) * 2 - 1) * scale * 448.0  # |x / scale| <= 448, as inside a group
        x = x.to(torch.bfloat16).float()
        bad = torch.zeros(1, dtype=torch.int32, device=d)
        _lib.check(lib.aklr_selftest_exact_divide(x.data_ptr(), scale.data_ptr(), n, bad.data_ptr(), torch.cuda.current_stream().cuda_stream))
        total += int(bad.item())
        assert int(bad.item()) == 0, (kind, int(bad.item()))
    assert total == 0
