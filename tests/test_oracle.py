"""The CPU oracle against the reference's own outputs (golden fixtures) and its known-answer tests."""

from __future__ import annotations

import numpy as np
import torch

from oracle import moe_oracle as orc
from tests.golden import cases


def t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.asarray(a))


def check_inputs(prefix, args, golden_hashes):
    for k, v in args.items():
        if isinstance(v, torch.Tensor):
            assert orc.sha256_of(v) == golden_hashes[f"{prefix}.{k}"], f"seeded input {prefix}.{k} drifted"


def test_sigmoid_bits_are_the_fixture_writers(golden_hashes):
    every = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    assert orc.sha256_of(torch.sigmoid(every)) == golden_hashes["sigmoid_table_sha256"]


def test_tiny_layer_matches_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    cfg, a = cases.tiny_layer()
    check_inputs("tiny", a, golden_hashes)
    logits = orc.router_logits(a["hidden_states"], a["router_weight"])
    assert torch.equal(logits, t(golden["tiny.logits"]))
    ids, w = orc.softmax_topk(logits, cfg.topk)
    assert torch.equal(ids, t(golden["tiny.ids"]))
    assert torch.equal(w, t(golden["tiny.weights"]))
    out = orc.qwen3_moe_fp8_moe(
        a["hidden_states"], a["router_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], cfg.topk
    )
    assert torch.equal(out, t(golden["tiny.out"]))
    assert torch.equal(orc.fp8_input(a["hidden_states"].float()), t(golden["tiny.fp8_input"]))


def test_deepseek_small_layer_matches_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    cfg, a = cases.ds_small_layer()
    check_inputs("ds_small", a, golden_hashes)
    logits = orc.router_logits(a["hidden_states"], a["router_weight"])
    assert torch.equal(logits, t(golden["ds_small.logits"]))
    ids, w = orc.grouped_sigmoid_topk(
        logits, a["correction_bias"].float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, True, 2.5
    )
    ids, w = orc.with_shared_slot(ids, w, cfg.n_routed)
    assert torch.equal(ids, t(golden["ds_small.ids"]))
    assert torch.equal(w, t(golden["ds_small.weights"]))
    out = orc.deepseek_v2_fp8_moe(
        a["hidden_states"],
        a["router_weight"],
        a["correction_bias"],
        a["w1"],
        a["w1_scale"],
        a["w2"],
        a["w2_scale"],
        cfg.topk,
        cfg.num_expert_group,
        cfg.topk_group,
        True,
        2.5,
    )
    assert torch.equal(out, t(golden["ds_small.out"]))


def test_minimax_layer_matches_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    cfg, a = cases.minimax_layer()
    check_inputs("minimax", {k: v for k, v in a.items() if isinstance(v, torch.Tensor)}, golden_hashes)
    logits = a["hidden_states"].float() @ a["router_weight"].T
    ids, w = orc.sigmoid_bias_topk(logits, a["correction_bias"], cfg.topk)
    assert torch.equal(ids, t(golden["minimax.ids"])) and torch.equal(w, t(golden["minimax.weights"]))
    out = orc.minimax_m2_fp8_moe(
        a["hidden_states"], a["router_weight"], a["correction_bias"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"],
        cfg.topk, a["expert_offset"],
    )
    assert torch.equal(out, t(golden["minimax.out"]))
    assert (ids < a["expert_offset"]).any() and (ids >= a["expert_offset"] + cfg.n_routed).any()  # routes to other ranks exist


def test_qwen2_layer_matches_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    cfg, a = cases.qwen2_layer()
    check_inputs("qwen2", a, golden_hashes)
    ids, w = orc.softmax_topk(orc.router_logits(a["hidden_states"], a["router_weight"]).float(), cfg.topk)
    assert torch.equal(ids, t(golden["qwen2.ids"]).long()) and torch.equal(w, t(golden["qwen2.weights"]))
    out = orc.qwen2_moe_fp8_router_experts(
        a["hidden_states"], a["router_weight"], a["shared_gate_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], cfg.topk
    )
    assert torch.equal(out, t(golden["qwen2.out"]))
    out = orc.qwen2_moe_fp8_experts(
        a["hidden_states"], w, ids, a["shared_gate_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"]
    )
    assert torch.equal(out, t(golden["qwen2.experts_out"]))


def test_routing_matches_reference(golden, golden_hashes):
    logits, bias = cases.route_ds()
    assert orc.sha256_of(logits) == golden_hashes["route_ds.logits"]
    ids, w = orc.grouped_sigmoid_topk(logits.float(), bias.float(), 8, 8, 4, True, 2.5)
    assert torch.equal(ids, t(golden["route_ds.ids"])) and torch.equal(w, t(golden["route_ds.weights"]))
    ids, w = orc.grouped_sigmoid_topk(logits.float(), bias.float(), 8, 8, 4, False, 1.0)
    assert torch.equal(ids, t(golden["route_ds_norenorm.ids"]))
    assert torch.equal(w, t(golden["route_ds_norenorm.weights"]))
    tied = cases.route_tied()
    ids, w = orc.grouped_sigmoid_topk(tied.float(), torch.zeros(256), 8, 8, 4, True, 2.5)
    assert torch.equal(ids, t(golden["route_tied.ids"])) and torch.equal(w, t(golden["route_tied.weights"]))
    cfg, logits = cases.route_qwen3()
    ids, w = orc.softmax_topk(logits.float(), cfg.topk)
    assert torch.equal(ids, t(golden["route_qwen3.ids"])) and torch.equal(w, t(golden["route_qwen3.weights"]))
    ids, w = orc.softmax_topk(tied[:, :128].float(), 8)
    assert torch.equal(ids, t(golden["route_tied_softmax.ids"]))
    logits, bias = cases.bgt()
    w, ids = orc.biased_grouped_topk(logits, bias, 8, True, 2.5)
    assert torch.equal(ids, t(golden["bgt.ids"])) and torch.equal(w, t(golden["bgt.weights"]))


def test_ties_go_to_the_lower_expert():
    """Known answer of the reference's own test (tests/ops/test_reference.py:91-108)."""
    logits = torch.zeros(1, 1024)
    logits[0, [583, 571, 368, 31]] = 1.0
    _, ids = orc.biased_grouped_topk(logits, torch.zeros(1024), 3, False, 1.0)
    assert ids.tolist() == [[31, 368, 571]]


def test_quant_ops_match_reference(golden, golden_hashes):
    x = cases.quant_x()
    assert orc.sha256_of(x) == golden_hashes["quant.x"]
    q, s = orc.per_group_quant_fp8(x)
    assert torch.equal(q, t(golden["quant_fp8.q"])) and torch.equal(s, t(golden["quant_fp8.s"]))
    q, s = orc.per_group_quant_mxfp8(x)
    assert torch.equal(q, t(golden["quant_mxfp8.q"])) and torch.equal(s, t(golden["quant_mxfp8.s"]))
    assert torch.equal(orc.mxfp8_input(x.float()), t(golden["mxfp8_input"]))
    assert torch.equal(orc.mxfp4_input(x.float()), t(golden["mxfp4_input"]))


def test_mx_experts_match_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    a, group = cases.mega_group()
    check_inputs("mx_moe", a, golden_hashes)
    args = (a["hidden_states"], a["topk_ids"].long(), a["topk_weights"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"])
    assert torch.equal(orc.mx_experts(*args, act_bits=8), t(golden["mx_moe.out"]))
    assert torch.equal(orc.mx_experts(*args, act_bits=4), t(golden["mx_moe_a4.out"]))
    w1 = torch.cat([g["w1"] for g in group])
    s1 = torch.cat([g["w1_scale"] for g in group])
    w2 = torch.cat([g["w2"] for g in group])
    s2 = torch.cat([g["w2_scale"] for g in group])
    for r, g in enumerate(group):
        out = orc.mx_experts(
            g["hidden_states"], g["topk_ids"].long(), g["topk_weights"], w1, s1, w2, s2, swiglu_limit=10.0
        )
        assert torch.equal(out, t(golden[f"mega.rank{r}.out"]))


def test_mx_experts_variants_match_reference(golden, golden_hashes):
    """Activations, stage-1 weighting, the expert mask with rows not received: each against the
    reference's stored output, bit for bit."""
    torch.set_num_threads(1)
    for name, a, _, kw in cases.mx_variants():
        check_inputs(f"mx_moe_{name}", {k: v for k, v in a.items() if torch.is_tensor(v)}, golden_hashes)
        ids = a["topk_ids"].long()
        if "expert_mask" in a:  # a global id to its slot in w1, -1 off this rank
            held = a["expert_mask"].long()
            ids = torch.where(held[ids] == 1, (held.cumsum(0) - 1)[ids], -1)
        out = orc.mx_experts(a["hidden_states"], ids, a["topk_weights"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], **kw)
        assert torch.equal(out, t(golden[f"mx_moe_{name}.out"])), name


def test_deepseek_mxfp4_layer_matches_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    cfg, a = cases.ds_mx_layer()
    check_inputs("ds_mx", {k: v for k, v in a.items() if torch.is_tensor(v)}, golden_hashes)
    out = orc.deepseek_v2_mxfp4_moe(a["hidden_states"], a["router_weight"], a["correction_bias"], a["w1"], a["w1_scale"], a["w2"],
                                    a["w2_scale"], cfg.topk, True, 2.5)
    assert torch.equal(out, t(golden["ds_mx.out"]))


def test_minimax_mxfp4_layer_matches_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    cfg, a = cases.minimax_mx_layer()
    check_inputs("minimax_mx", {k: v for k, v in a.items() if torch.is_tensor(v)}, golden_hashes)
    out = orc.minimax_m2_mxfp4_moe(a["hidden_states"], a["router_weight"], a["correction_bias"], a["w1"], a["w1_scale"], a["w2"],
                                   a["w2_scale"], cfg.topk, a["expert_offset"])
    assert torch.equal(out, t(golden["minimax_mx.out"]))


def test_qwen2_mxfp4_layer_with_a_bf16_shared_expert_matches_reference(golden, golden_hashes):
    torch.set_num_threads(1)
    cfg, a = cases.qwen2_mx_layer()
    check_inputs("qwen2_mx", a, golden_hashes)
    out = orc.qwen2_moe_mxfp4_moe(a["hidden_states"], a["router_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"],
                                  a["shared_w1"], a["shared_w2"], a["shared_gate_weight"], cfg.topk)
    assert torch.equal(out, t(golden["qwen2_mx.out"]))
    # the shared expert carries about as much of the output as the routed ones, so dropping it fails any gate
    routed_only = orc.qwen2_moe_mxfp4_moe(a["hidden_states"], a["router_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"],
                                          a["shared_w1"], torch.zeros_like(a["shared_w2"]), a["shared_gate_weight"], cfg.topk)
    assert orc.sqnr_db(routed_only, out) < 6.0


def test_moe_align_is_a_stable_padded_sort():
    ids = torch.tensor([[2, 0], [2, 1], [0, 2], [-1, 2]])
    sorted_ids, block_expert, counts = orc.moe_align(ids, 4, 4)
    assert counts.tolist() == [2, 1, 4, 0]
    assert sorted_ids.tolist() == [1, 4, -1, -1, 3, -1, -1, -1, 0, 2, 5, 7]
    assert block_expert.tolist() == [0, 1, 2]


def test_reference_passes_its_own_gates(golden):
    ref = t(golden["tiny.out"])
    g = orc.output_gates(orc.bf16_round(ref).to(torch.bfloat16), ref)
    assert orc.gates_pass(g) and g["sqnr_db"] == float("inf")
