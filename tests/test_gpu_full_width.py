"""Full-width parity at the token counts the benchmark configurations name.

The expert weights (up to 11 GB) are drawn on the device; routing ids and per-expert counts are
checked for the whole batch against the CPU oracle.  Outputs are checked in two ways, both against
the oracle with the layer's gates (max relative error per row <= 2e-2, cosine >= 0.9995, SQNR >= 30 dB):

* per ROUTE, on rows picked by their place in an expert's sorted run -- the first row, the last row of
  a full 128-row block, the first row of the next block, the first and last row of the padded tail
  block, the middle -- for the experts whose counts sit closest to 128 from below and from above, the
  least and the most loaded routed expert and the shared expert: the kernel's weighted per-route row
  (what the down projection wrote) against the oracle's contribution of that expert to that token;
* per TOKEN, on the token with the largest output magnitude, the first, the last and the tokens of
  the first picked routes: the combined output against the oracle over all of the token's experts.

A token's output depends on that token alone, so a sample is checked exactly as the whole batch would be.
"""

from __future__ import annotations

import pytest
import torch

from aklr_b200 import workloads as wl
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def routing_of(cfg):
    from aklr_b200.moe import Routing

    return Routing(cfg.topk, cfg.scoring, cfg.n_shared, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor)


class LazyExperts:
    """Indexable like a weight tensor on the host, fetching one expert from the device at a time."""

    def __init__(self, device_tensor):
        self.t = device_tensor

    def __getitem__(self, e):
        return self.t[e].cpu()


def oracle_routing(cfg, logits, bias):
    if cfg.scoring == "sigmoid":
        ids, w = orc.grouped_sigmoid_topk(
            logits.float(), bias.float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, cfg.renormalize, cfg.routed_scaling_factor
        )
        for k in range(cfg.n_shared):
            ids, w = orc.with_shared_slot(ids, w, cfg.n_routed + k)
        return ids, w
    return orc.softmax_topk(logits.float(), cfg.topk)


def places_in_run(count: int, block: int = 128) -> list[int]:
    """Rows of an expert's sorted run worth looking at: ends of the run, of its full blocks and of its tail."""
    last_block = (count - 1) // block * block
    want = {0, 1, count // 4, count // 2, 3 * count // 4, count - 2, count - 1, last_block, last_block - 1, last_block + 1}
    want |= {block - 1, block, 2 * block - 1, 2 * block, 31, 32, 63, 64}  # ends of blocks and of lane quarters
    return sorted(p for p in want if 0 <= p < count)


def experts_worth_a_look(counts: torch.Tensor, n_routed: int, block: int = 128) -> list[int]:
    routed = counts[:n_routed]
    chosen = []
    at_most = torch.where(routed <= block, routed, torch.full_like(routed, -1))
    if int(at_most.max()) > 0:
        chosen.append(int(at_most.argmax()))  # closest to a full block from below (exactly 128 when there is one)
    above = torch.where(routed > block, routed, torch.full_like(routed, 1 << 40))
    if int(above.min()) < (1 << 40):
        chosen.append(int(above.argmin()))  # one row or so into a second block
    live = torch.where(routed > 0, routed, torch.full_like(routed, 1 << 40))
    chosen += [int(live.argmin()), int(routed.argmax())]
    chosen += list(range(n_routed, counts.numel()))  # shared experts: every token
    seen, unique = set(), []
    for e in chosen:
        if e not in seen and int(counts[e]) > 0:
            seen.add(e)
            unique.append(e)
    return unique


def check_sampled(cfg, hidden, ref_ids, ref_w, out, route_rows, one_expert, whole_token, max_experts=5):
    """``one_expert(tokens, e, weights)`` and ``whole_token(tokens)`` are the oracle on a sample."""
    n_tokens, width = ref_ids.shape
    flat = ref_ids.flatten()
    counts = torch.bincount(flat, minlength=cfg.n_experts)
    picked_tokens, n_routes = [], 0
    for e in experts_worth_a_look(counts, cfg.n_routed)[:max_experts]:
        run = (flat == e).nonzero(as_tuple=True)[0]  # the expert's routes in sorted (= ascending) order
        rids = run[places_in_run(run.numel())]
        tokens = rids // width
        ref = one_expert(tokens, e, ref_w.flatten()[rids])
        got = route_rows[rids.to(route_rows.device)].cpu()
        gates = orc.output_gates(got, ref)
        assert orc.gates_pass(gates), (e, int(counts[e]), rids.tolist(), gates)
        picked_tokens += tokens[:2].tolist()
        n_routes += rids.numel()
    loudest = int(out.float().abs().amax(dim=1).argmax())
    if n_tokens <= 64:
        sample = torch.arange(n_tokens)  # a batch this small is checked whole
    else:
        sample = torch.tensor(sorted(set([0, n_tokens - 1, loudest] + picked_tokens[:5])))
    gates = orc.output_gates(out[sample.to(out.device)].cpu(), whole_token(sample))
    assert orc.gates_pass(gates), (sample.tolist(), gates)
    return n_routes, sample.numel()


FP8_CASES = [
    ("deepseek_v3", 16384),
    ("deepseek_v3", 4096),
    ("deepseek_v3", 1),  # nine blocks: the down projection runs on 64-channel tiles
    ("deepseek_v3", 2),
    ("mixtral", 4096),
    ("qwen3", 1),
    ("qwen3", 32),
    ("qwen3", 2048),
    ("qwen3", 8192),
]


@pytest.mark.parametrize("name,n_tokens", FP8_CASES)
def test_fp8_layer_at_benchmark_token_counts(name, n_tokens):
    from aklr_b200.moe import fused_moe_fp8

    cfg = wl.CONFIGS[name]
    d = dev()
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=61, device=d)
    hidden, logits, bias = wl.router_inputs(cfg, n_tokens, seed=62 + n_tokens)
    bias_d = None if bias is None else bias.to(d)
    out, ws = fused_moe_fp8(hidden.to(d), logits.to(d), bias_d, w1, s1, w2, s2, routing_of(cfg), return_workspace=True)
    ws.check_status()
    ref_ids, ref_w = oracle_routing(cfg, logits, bias)
    assert torch.equal(ws.topk_ids().cpu().long(), ref_ids)
    torch.testing.assert_close(ws.topk_weights().cpu(), ref_w.float(), atol=1e-4, rtol=1e-4)
    assert torch.equal(ws.counts().cpu().long(), torch.bincount(ref_ids.flatten(), minlength=cfg.n_experts))
    lazy = [LazyExperts(t) for t in (w1, s1, w2, s2)]

    def one_expert(tokens, e, weights):
        ids = torch.full((tokens.numel(), 1), e, dtype=torch.long)
        return orc.fp8_experts(hidden[tokens], ids, weights.reshape(-1, 1), *lazy)

    def whole_token(tokens):
        return orc.fp8_experts(hidden[tokens], ref_ids[tokens], ref_w[tokens], *lazy)

    n_routes, n_whole = check_sampled(cfg, hidden, ref_ids, ref_w, out, ws.route_rows(), one_expert, whole_token)
    assert n_routes + n_whole >= min(32, n_tokens)


def test_mxfp4_layer_at_deepseek_v3_widths_8192_tokens():
    """Configuration 5: DeepSeek-V3 routing and widths, MXFP4 expert weights, MXFP8 activations, 8192 tokens."""
    from aklr_b200.moe import fused_moe_mxfp4

    cfg = wl.CONFIGS["deepseek_v3"]
    n_tokens = 8192
    d = dev()
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed=71, device=d)
    hidden, logits, bias = wl.router_inputs(cfg, n_tokens, seed=72)
    out, ws = fused_moe_mxfp4(hidden.to(d), logits.to(d), bias.to(d), w1, s1, w2, s2, routing_of(cfg), return_workspace=True)
    ws.check_status()
    ref_ids, ref_w = oracle_routing(cfg, logits, bias)
    assert torch.equal(ws.topk_ids().cpu().long(), ref_ids)
    assert torch.equal(ws.counts().cpu().long(), torch.bincount(ref_ids.flatten(), minlength=cfg.n_experts))
    lazy = [LazyExperts(t) for t in (w1, s1, w2, s2)]

    def one_expert(tokens, e, weights):
        ids = torch.full((tokens.numel(), 1), e, dtype=torch.long)
        return orc.mx_experts(hidden[tokens], ids, weights.reshape(-1, 1), *lazy, act_bits=8)

    def whole_token(tokens):
        return orc.mx_experts(hidden[tokens], ref_ids[tokens], ref_w[tokens], *lazy, act_bits=8)

    n_routes, n_whole = check_sampled(cfg, hidden, ref_ids, ref_w, out, ws.route_rows(), one_expert, whole_token)
    assert n_routes + n_whole >= 32


@pytest.mark.parametrize("block_m", [0, 128, 64])
def test_experts_with_1_127_128_129_255_257_rows(block_m):
    """Routing crafted so that six experts receive exactly 1, 127, 128, 129, 255 and 257 rows (a seventh takes
    the rest): every row of the batch against the oracle, through the experts-only entry point."""
    from aklr_b200.moe import fused_experts_fp8

    cfg = wl.MoEConfig("crafted", hidden=512, inter=256, n_routed=7, topk=1)
    wanted = [1, 127, 128, 129, 255, 257]
    n_tokens = sum(wanted) + 40
    g = torch.Generator().manual_seed(5)
    assignment = torch.cat([torch.full((c,), e) for e, c in enumerate(wanted)] + [torch.full((40,), 6)])
    ids = assignment[torch.randperm(n_tokens, generator=g)].reshape(-1, 1).to(torch.int32)
    weights = torch.rand(n_tokens, 1, generator=g) + 0.5
    hidden = wl.normal(5, "hidden", (n_tokens, cfg.hidden), 1.0, dtype=torch.bfloat16)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=6)
    d = dev()
    out, ws = fused_experts_fp8(hidden.to(d), ids.to(d), weights.to(d), w1.to(d), s1.to(d), w2.to(d), s2.to(d),
                                block_m=block_m, return_workspace=True)
    ws.check_status()
    assert ws.counts().cpu().tolist() == wanted + [40]
    ref = orc.fp8_experts(hidden, ids.long(), weights, w1, s1, w2, s2)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates
    worst = ((out.cpu().float() - orc.bf16_round(ref)).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp_min(1e-30))
    assert float(worst.max()) <= 2e-2, (int(worst.argmax()), float(worst.max()))


def _layer_against_oracle(cfg, hidden, logits, bias, seed, max_experts=5):
    from aklr_b200.moe import fused_moe_fp8

    d = dev()
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=seed, device=d)
    bias_d = None if bias is None else bias.to(d)
    out, ws = fused_moe_fp8(hidden.to(d), logits.to(d), bias_d, w1, s1, w2, s2, routing_of(cfg), return_workspace=True)
    ws.check_status()
    ref_ids, ref_w = oracle_routing(cfg, logits, bias)
    assert torch.equal(ws.topk_ids().cpu().long(), ref_ids)
    counts = torch.bincount(ref_ids.flatten(), minlength=cfg.n_experts)
    assert torch.equal(ws.counts().cpu().long(), counts)
    # the sorted table: every expert's run holds exactly its routes, in ascending route order, padded with -1
    sorted_ids = ws.sorted_ids().cpu().long()
    live = sorted_ids[sorted_ids >= 0]
    assert live.numel() == ref_ids.numel()
    by_expert = ref_ids.flatten()[live]
    assert torch.equal(by_expert, by_expert.sort(stable=True).values)  # experts ascend along the table
    same = by_expert[1:] == by_expert[:-1]
    assert bool((live[1:][same] > live[:-1][same]).all())  # and routes ascend inside an expert
    lazy = [LazyExperts(t) for t in (w1, s1, w2, s2)]

    def one_expert(tokens, e, weights):
        ids = torch.full((tokens.numel(), 1), e, dtype=torch.long)
        return orc.fp8_experts(hidden[tokens], ids, weights.reshape(-1, 1), *lazy)

    def whole_token(tokens):
        return orc.fp8_experts(hidden[tokens], ref_ids[tokens], ref_w[tokens], *lazy)

    check_sampled(cfg, hidden, ref_ids, ref_w, out, ws.route_rows(), one_expert, whole_token, max_experts=max_experts)
    return counts


def test_largest_batch_the_ops_take():
    """65 536 tokens (the contracts' upper bound) at Qwen3 widths: 524 288 routes through the three-pass sort (512
    chunks), ids, counts and the sorted table bit for bit, outputs sampled by place in the runs."""
    cfg = wl.CONFIGS["qwen3"]
    hidden, logits, bias = wl.router_inputs(cfg, 65536, seed=71)
    counts = _layer_against_oracle(cfg, hidden, logits, bias, seed=72, max_experts=4)
    assert int(counts.sum()) == 65536 * cfg.topk


def test_every_token_on_the_same_experts():
    """Total imbalance: logits that send all 3000 tokens to the same eight experts (3000 rows each, 24 blocks) and
    leave 120 experts empty; and the mirror case, one expert with a single row among busy ones."""
    cfg = wl.CONFIGS["qwen3"]
    n_tokens = 3000
    hidden, logits, bias = wl.router_inputs(cfg, n_tokens, seed=73)
    logits = (logits.float() * 0.1)
    logits[:, [3, 17, 31, 45, 59, 73, 87, 101]] += 20.0
    logits[5, 120] += 40.0  # one token also picks expert 120: a run of one row
    logits = logits.to(torch.bfloat16)
    counts = _layer_against_oracle(cfg, hidden, logits, bias, seed=74, max_experts=6)
    assert int((counts > 0).sum()) == 9 and int(counts[120]) == 1 and int(counts.max()) == n_tokens


def test_a_thousand_experts():
    """1024 routed experts (the contracts' upper bound), top-8 softmax, 2000 tokens: most experts get 10-20 rows."""
    cfg = wl.MoEConfig("wide", hidden=512, inter=256, n_routed=1024, topk=8)
    hidden, logits, bias = wl.router_inputs(cfg, 2000, seed=75)
    counts = _layer_against_oracle(cfg, hidden, logits, bias, seed=76, max_experts=4)
    assert int((counts > 0).sum()) > 1000
