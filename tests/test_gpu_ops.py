"""The ops through their reference-shaped api functions (dispatch registry included) on the device."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from aklr_b200 import workloads as wl
from oracle import moe_oracle as orc
from tests.golden import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from aklr_b200 import ops as module

    torch.cuda.set_device(0)
    module.init()
    return module


def dev():
    return torch.device("cuda:0")


def to_dev(args):
    return {k: (v.to(dev()) if isinstance(v, torch.Tensor) else v) for k, v in args.items()}


def test_deepseek_v2_fp8_moe_op(ops, golden):
    cfg, a = cases.ds_small_layer()
    out = ops.deepseek_v2_fp8_moe(
        **to_dev(a), topk=cfg.topk, num_expert_group=cfg.num_expert_group, topk_group=cfg.topk_group,
        renormalize=True, scoring_func="sigmoid",
    )
    assert isinstance(out, torch.Tensor) and out.dtype == torch.bfloat16
    # the router GEMM runs on the device: compare against the oracle fed the device's logits
    from aklr_b200.moe import router_logits

    logits = router_logits(a["hidden_states"].to(dev()), a["router_weight"].to(dev())).cpu().float()
    ref = orc.deepseek_v2_fp8_moe(
        a["hidden_states"], None, a["correction_bias"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], cfg.topk,
        cfg.num_expert_group, cfg.topk_group, True, 2.5, logits=logits,
    )
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates


def test_ops_take_tile_contiguous_weights_by_their_attribute(ops):
    """A loader converts the experts once (aklr_b200.layouts.to_b200_tiled); the op reads the tensors' attribute, keys the
    call as another layout variant and returns the row-major call's output bit for bit.  One converted tensor
    with one row-major one is outside the contract."""
    from aklr_b200 import layouts

    cfg, a = cases.ds_small_layer()
    d = to_dev(a)
    kw = dict(topk=cfg.topk, num_expert_group=cfg.num_expert_group, topk_group=cfg.topk_group, renormalize=True,
              scoring_func="sigmoid")
    plain = ops.deepseek_v2_fp8_moe(**d, **kw)
    tiled = {**d, "w1": layouts.to_b200_tiled(d["w1"]), "w2": layouts.to_b200_tiled(d["w2"])}
    out = ops.deepseek_v2_fp8_moe(**tiled, **kw)
    assert isinstance(out, torch.Tensor) and torch.equal(out.cpu(), plain.cpu())
    assert ops.deepseek_v2_fp8_moe(**{**tiled, "w2": d["w2"]}, **kw) is ops.FallbackReason.OUT_OF_CONTRACT


def test_deepseek_v2_mxfp4_moe_op(ops, golden):
    """MXFP4 experts, ungrouped routing with a float32 bias, activations never quantised: against the reference's
    stored output (the kernels round the gated product to bf16, the reference does not: far inside the gates)."""
    cfg, a = cases.ds_mx_layer()
    args = {k: v for k, v in to_dev(a).items() if k != "routed_scaling_factor"}
    out = ops.deepseek_v2_mxfp4_moe(**args, topk=cfg.topk, num_expert_group=1, topk_group=1, renormalize=True,
                                    scoring_func="sigmoid", routed_scaling_factor=2.5)
    assert isinstance(out, torch.Tensor) and out.dtype == torch.bfloat16
    from aklr_b200.moe import router_logits

    logits = router_logits(a["hidden_states"].to(dev()), a["router_weight"].to(dev())).cpu().float()
    ref = orc.deepseek_v2_mxfp4_moe(a["hidden_states"], a["router_weight"], a["correction_bias"], a["w1"], a["w1_scale"], a["w2"],
                                    a["w2_scale"], cfg.topk, True, 2.5, logits=logits)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates, min_sqnr_db=40.0), gates
    stored = orc.output_gates(out.cpu(), torch.from_numpy(np.asarray(golden["ds_mx.out"])))
    assert stored["sqnr_db"] > 35.0, stored  # the host's router GEMM may round a logit the other way: a weight moves by a bf16 step
    # grouped routing and a bf16 bias are not this contract
    assert ops.deepseek_v2_mxfp4_moe(**args, topk=cfg.topk, num_expert_group=4, topk_group=2, renormalize=True,
                                     scoring_func="sigmoid", routed_scaling_factor=2.5) is ops.FallbackReason.OUT_OF_CONTRACT


def test_minimax_m2_mxfp4_moe_op(ops, golden):
    """MXFP4 experts under MiniMax-M2's routing (float32 gate, this rank holding experts 4..11 of 16), activations
    never quantised: against the reference's stored output, and at 600 tokens against the oracle on the device's logits."""
    from aklr_b200.moe import router_logits_f32

    cfg, a = cases.minimax_mx_layer()
    d = to_dev(a)
    out = ops.minimax_m2_mxfp4_moe(**d, topk=cfg.topk)
    assert isinstance(out, torch.Tensor) and out.dtype == torch.bfloat16
    gates = orc.output_gates(out.cpu(), torch.from_numpy(np.asarray(golden["minimax_mx.out"])))
    assert orc.gates_pass(gates, min_sqnr_db=40.0), gates
    hidden = torch.randn(600, cfg.hidden, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    big = {**d, "hidden_states": hidden.to(dev())}
    out = ops.minimax_m2_mxfp4_moe(**big, topk=cfg.topk)
    logits = router_logits_f32(big["hidden_states"], d["router_weight"]).cpu()
    ref = orc.minimax_m2_mxfp4_moe(hidden, a["router_weight"], a["correction_bias"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"],
                                   cfg.topk, a["expert_offset"], logits=logits)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates, min_sqnr_db=40.0), gates
    # FP8 weights are the other op's contract
    assert ops.minimax_m2_mxfp4_moe(**{**d, "w1": d["w1"].view(torch.float8_e4m3fn)}, topk=cfg.topk) is ops.FallbackReason.OUT_OF_CONTRACT


def test_qwen2_moe_mxfp4_moe_op(ops, golden):
    """The whole Qwen2-MoE block with MXFP4 routed experts and the shared expert apart in bf16: against the
    reference's stored output and, at 500 tokens, the oracle on the device's logits.  The reference's own floor
    for this op is 11 dB (aklr/plugins/sglang/models/qwen2_moe/contract.py:306); the shared expert's two GEMMs
    round to bf16 here and not in the reference, which leaves the output above 40 dB."""
    from aklr_b200.moe import router_logits

    cfg, a = cases.qwen2_mx_layer()
    d = to_dev(a)
    out = ops.qwen2_moe_mxfp4_moe(**d, topk=cfg.topk)
    assert isinstance(out, torch.Tensor) and out.dtype == torch.bfloat16
    stored = orc.output_gates(out.cpu(), torch.from_numpy(np.asarray(golden["qwen2_mx.out"])))
    assert stored["sqnr_db"] > 35.0 and stored["cosine"] > 0.9995, stored
    hidden = torch.randn(500, cfg.hidden, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    big = {**d, "hidden_states": hidden.to(dev())}
    out = ops.qwen2_moe_mxfp4_moe(**big, topk=cfg.topk)
    logits = router_logits(big["hidden_states"], d["router_weight"]).cpu().float()
    ref = orc.qwen2_moe_mxfp4_moe(hidden, a["router_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], a["shared_w1"],
                                  a["shared_w2"], a["shared_gate_weight"], cfg.topk, logits=logits)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates, min_sqnr_db=40.0), gates
    # a kernel that dropped the shared expert would be far off: it carries half of the output
    no_shared = orc.qwen2_moe_mxfp4_moe(hidden, a["router_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], a["shared_w1"],
                                        torch.zeros_like(a["shared_w2"]), a["shared_gate_weight"], cfg.topk, logits=logits)
    assert orc.sqnr_db(out.cpu().float(), no_shared) < 6.0
    # a shared expert whose width is not a multiple of 128 is outside the contract
    bad = {**d, "shared_w1": d["shared_w1"][:700].contiguous(), "shared_w2": d["shared_w2"][:, :350].contiguous()}
    assert ops.qwen2_moe_mxfp4_moe(**bad, topk=cfg.topk) is ops.FallbackReason.OUT_OF_CONTRACT


def test_minimax_m2_fp8_moe_op(ops, golden):
    """Float32 gate, biased sigmoid top-k without groups, this rank holding experts 4..11 of 16: against
    the reference's stored output, and at larger batches (tile router kernel, token-major experts)
    against the oracle fed the device's logits."""
    from aklr_b200.moe import router_logits_f32

    cfg, a = cases.minimax_layer()
    d = to_dev(a)
    out = ops.minimax_m2_fp8_moe(**d, topk=cfg.topk)
    assert isinstance(out, torch.Tensor) and out.dtype == torch.bfloat16
    logits = router_logits_f32(d["hidden_states"], d["router_weight"]).cpu()
    torch.testing.assert_close(logits, a["hidden_states"].float() @ a["router_weight"].T, atol=2e-5, rtol=1e-5)
    gates = orc.output_gates(out.cpu(), torch.from_numpy(np.asarray(golden["minimax.out"])))
    assert orc.gates_pass(gates), gates
    # every expert held here (no expert_offset), 700 tokens
    g = torch.Generator().manual_seed(3)
    hidden = torch.randn(700, cfg.hidden, generator=g).to(torch.bfloat16)
    router = a["router_weight"][:8].contiguous()
    bias = a["correction_bias"][:8].contiguous()
    out = ops.minimax_m2_fp8_moe(
        hidden_states=hidden.to(dev()), router_weight=router.to(dev()), correction_bias=bias.to(dev()), w1=d["w1"],
        w1_scale=d["w1_scale"], w2=d["w2"], w2_scale=d["w2_scale"], topk=2,
    )
    logits = router_logits_f32(hidden.to(dev()), router.to(dev())).cpu()
    ref = orc.minimax_m2_fp8_moe(hidden, None, bias, a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], 2, logits=logits)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates
    # out of contract: a bf16 gate, an offset past the router's rows
    assert ops.minimax_m2_fp8_moe(**{**d, "router_weight": d["router_weight"].bfloat16()}, topk=cfg.topk) is ops.FallbackReason.OUT_OF_CONTRACT
    assert ops.minimax_m2_fp8_moe(**{**d, "expert_offset": 9}, topk=cfg.topk) is ops.FallbackReason.OUT_OF_CONTRACT


def test_qwen2_moe_ops(ops, golden):
    """The three Qwen2-MoE ops against the reference's stored outputs: the router bit for bit where the
    device's bf16 logits equal the host's; the experts at the reference's routing; router + experts
    through the gates; then 640 tokens (token-major experts) against the oracle fed the device's logits."""
    from aklr_b200 import moe

    cfg, a = cases.qwen2_layer()
    d = to_dev(a)
    n_tokens = a["hidden_states"].shape[0]
    ids = torch.empty((n_tokens, cfg.topk), dtype=torch.int32, device=dev())
    wts = torch.empty((n_tokens, cfg.topk), dtype=torch.float32, device=dev())
    routed = ops.qwen2_moe_router(hidden_states=d["hidden_states"], router_weight=d["router_weight"], topk_weights=wts, topk_ids=ids)
    assert routed[0] is wts and routed[1] is ids
    logits = moe.router_logits(d["hidden_states"], d["router_weight"]).cpu()
    same = (logits == orc.router_logits(a["hidden_states"], a["router_weight"])).all(dim=1)
    assert same.float().mean() > 0.7  # a bf16 step apart where the accumulation order rounds differently
    ref_ids, ref_w = orc.softmax_topk(logits.float(), cfg.topk)
    assert torch.equal(ids.cpu().long(), ref_ids)
    torch.testing.assert_close(wts.cpu(), ref_w, atol=2e-6, rtol=1e-5)
    assert torch.equal(ids.cpu()[same], torch.from_numpy(np.asarray(golden["qwen2.ids"]))[same].int())
    # experts at the reference's routing
    g_ids = torch.from_numpy(np.asarray(golden["qwen2.ids"])).int().to(dev())
    g_w = torch.from_numpy(np.asarray(golden["qwen2.weights"])).to(dev())
    expert_args = {k: d[k] for k in ("hidden_states", "shared_gate_weight", "w1", "w1_scale", "w2", "w2_scale")}
    out = ops.qwen2_moe_fp8_experts(**expert_args, topk_weights=g_w, topk_ids=g_ids)
    gates = orc.output_gates(out.cpu(), torch.from_numpy(np.asarray(golden["qwen2.experts_out"])))
    assert orc.gates_pass(gates), gates
    # router + experts, against the oracle on the device's logits (a rerouted token is not an error of the experts)
    out = ops.qwen2_moe_fp8_router_experts(**d, topk=cfg.topk)
    ref = orc.qwen2_moe_fp8_router_experts(*(a[k] for k in ("hidden_states", "router_weight", "shared_gate_weight", "w1", "w1_scale", "w2", "w2_scale")), cfg.topk, logits=logits)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates
    assert orc.output_gates(out.cpu(), torch.from_numpy(np.asarray(golden["qwen2.out"])))["cosine"] > 0.999
    # 640 tokens: the token-major expert kernels
    hidden = torch.randn(640, cfg.hidden, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    big = {**d, "hidden_states": hidden.to(dev())}
    out = ops.qwen2_moe_fp8_router_experts(**big, topk=cfg.topk)
    logits = moe.router_logits(big["hidden_states"], d["router_weight"]).cpu()
    ref = orc.qwen2_moe_fp8_router_experts(hidden, a["router_weight"], a["shared_gate_weight"], a["w1"], a["w1_scale"], a["w2"], a["w2_scale"], cfg.topk, logits=logits)
    gates = orc.output_gates(out.cpu(), ref)
    # At these widths (one 128-wide scale block of 128 intermediate channels per expert) a single fp8
    # rounding flip of the requantised SiLU product moves a row by 1-3 % of its largest value, and a
    # 1e-6 relative change of the product is enough to flip some of the 400k elements here: the
    # per-row gate holds for all but a handful of rows, the aggregate gates hold outright.
    row_err = (out.cpu().double() - orc.bf16_round(ref).double()).abs().amax(-1) / orc.bf16_round(ref).double().abs().amax(-1)
    assert gates["sqnr_db"] > 45 and gates["cosine"] > 0.9999 and gates["max_rel_err"] < 5e-2, gates
    assert (row_err > 2e-2).sum() <= 3, row_err.topk(5)
    # out of contract: a gate of the wrong shape, ids of the wrong dtype, outputs that share memory
    assert ops.qwen2_moe_fp8_router_experts(**{**d, "shared_gate_weight": d["shared_gate_weight"][0]}, topk=cfg.topk) is ops.FallbackReason.OUT_OF_CONTRACT
    assert ops.qwen2_moe_fp8_experts(**expert_args, topk_weights=g_w, topk_ids=g_ids.long()) is ops.FallbackReason.OUT_OF_CONTRACT
    assert ops.qwen2_moe_router(hidden_states=d["hidden_states"], router_weight=d["router_weight"], topk_weights=wts, topk_ids=wts.view(torch.int32)) is ops.FallbackReason.OUT_OF_CONTRACT


def test_qwen3_moe_fp8_moe_op_and_fallbacks(ops, golden):
    cfg, a = cases.tiny_layer()
    d = to_dev(a)
    out = ops.qwen3_moe_fp8_moe(**d, topk=cfg.topk)
    assert isinstance(out, torch.Tensor)
    gates = orc.output_gates(out.cpu(), torch.from_numpy(np.asarray(golden["tiny.out"])))
    assert gates["cosine"] > 0.999  # a logit one bf16 step off may reroute a token; see the layer tests for the gates
    # out of contract: a non-contiguous input, a wrong dtype, an empty batch
    assert ops.qwen3_moe_fp8_moe(**{**d, "hidden_states": d["hidden_states"].t().contiguous().t()}, topk=2) is ops.FallbackReason.OUT_OF_CONTRACT
    assert ops.qwen3_moe_fp8_moe(**{**d, "hidden_states": d["hidden_states"].float()}, topk=2) is ops.FallbackReason.OUT_OF_CONTRACT
    assert ops.qwen3_moe_fp8_moe(**{**d, "hidden_states": d["hidden_states"][:0]}, topk=2) is ops.FallbackReason.OUT_OF_CONTRACT
    assert ops.qwen3_moe_fp8_moe.fallback_reason(**d, topk=2) is None
    assert ops.qwen3_moe_fp8_moe.serving(**d, topk=2).arch == "sm_100a"


def test_fused_moe_op_fp8_with_expert_mask(ops):
    cfg = wl.CONFIGS["tiny"]
    hidden, logits, _ = wl.router_inputs(cfg, 40, seed=31)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=32)
    ids, weights = orc.softmax_topk(logits.float(), cfg.topk)
    mask = torch.zeros(cfg.n_routed, dtype=torch.int32)
    mask[2:6] = 1
    d = dev()
    out_buffer = torch.empty((40, cfg.hidden), dtype=torch.bfloat16, device=d)
    out = ops.fused_moe(
        hidden.to(d), w1[2:6].to(d), w2[2:6].to(d), weights.to(d), ids.to(torch.int32).to(d), expert_mask=mask.to(d),
        activation="silu", quant_type="per_128x128", w1_scale=s1[2:6].to(d), w2_scale=s2[2:6].to(d), out=out_buffer,
    )
    assert out is out_buffer
    local = torch.where((ids >= 2) & (ids < 6), ids - 2, -1)
    ref = orc.fp8_experts(hidden, local, weights, w1[2:6], s1[2:6], w2[2:6], s2[2:6])
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates
    # an output buffer that overlaps an input is refused
    bad = ops.fused_moe(hidden.to(d), w1[2:6].to(d), w2[2:6].to(d), weights.to(d), ids.to(torch.int32).to(d),
                        quant_type="per_128x128", w1_scale=s1[2:6].to(d), w2_scale=s2[2:6].to(d), out=hidden.to(d)[:40])
    assert isinstance(bad, torch.Tensor)  # a fresh copy does not overlap: served
    x = hidden.to(d)
    assert ops.fused_moe(x, w1[2:6].to(d), w2[2:6].to(d), weights.to(d), ids.to(torch.int32).to(d), quant_type="per_128x128",
                         w1_scale=s1[2:6].to(d), w2_scale=s2[2:6].to(d), out=x) is ops.FallbackReason.OUT_OF_CONTRACT


def test_fused_moe_op_mxfp4(ops):
    cfg = wl.MoEConfig("mx", hidden=512, inter=256, n_routed=8, topk=2)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed=3)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(70, 512, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(8, generator=g)[:2] for _ in range(70)]).to(torch.int32)
    wts = torch.rand(70, 2, generator=g)
    d = dev()
    out = ops.fused_moe(x.to(d), w1.to(d), w2.to(d), wts.to(d), ids.to(d), activation="silu", quant_type="per_1x32",
                        w1_scale=s1.to(d), w2_scale=s2.to(d), act_quant=8)
    assert isinstance(out, torch.Tensor)
    ref = orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, act_bits=8)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates
    # the op's default arguments: MXFP4 activations (act_quant 4)
    out = ops.fused_moe(x.to(d), w1.to(d), w2.to(d), wts.to(d), ids.to(d), quant_type="per_1x32", w1_scale=s1.to(d), w2_scale=s2.to(d))
    assert isinstance(out, torch.Tensor)
    a4 = orc.output_gates(out.cpu(), orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, act_bits=4))
    assert a4["sqnr_db"] >= 25.0 and a4["cosine"] >= 0.998, a4
    assert ops.fused_moe(x.to(d), w1.to(d), w2.to(d), wts.to(d), ids.to(d), quant_type="per_1x32", w1_scale=s1.to(d),
                         w2_scale=s2.to(d), act_quant=6) is ops.FallbackReason.OUT_OF_CONTRACT


def test_fused_moe_op_mxfp4_attributes(ops):
    """The op's other attributes on the MXFP4 path against the oracle (itself pinned to the reference's
    outputs for each of them): gelu, gpt-oss's swiglu with its clamp, situv2, the route weight applied
    in stage 1, and an expert mask with a count of rows received.  300 tokens: three 128-row blocks per
    busy expert, and past the 256 rows from which the reference quantises swiglu's activations."""
    cfg = wl.MoEConfig("mx", hidden=512, inter=256, n_routed=8, topk=2)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed=5)
    g = torch.Generator().manual_seed(6)
    n = 300
    x = torch.randn(n, 512, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(8, generator=g)[:2] for _ in range(n)]).to(torch.int32)
    wts = torch.rand(n, 2, generator=g) + 0.25
    d = dev()

    def run(**kw):
        return ops.fused_moe(x.to(d), kw.pop("w1", w1).to(d), kw.pop("w2", w2).to(d), wts.to(d), ids.to(d), quant_type="per_1x32",
                             w1_scale=kw.pop("w1_scale", s1).to(d), w2_scale=kw.pop("w2_scale", s2).to(d), act_quant=8, **kw)

    def check(out, ref, what):
        assert isinstance(out, torch.Tensor), (what, out)
        gates = orc.output_gates(out.cpu(), ref)
        assert orc.gates_pass(gates), (what, gates)

    base = (x, ids.long(), wts, w1, s1, w2, s2)
    check(run(activation="gelu"), orc.mx_experts(*base, activation="gelu"), "gelu")
    check(run(activation="swiglu", swiglu_limit=7.0), orc.mx_experts(*base, activation="swiglu", swiglu_limit=7.0), "swiglu")
    check(run(activation="situv2", beta=3.0, linear_beta=5.0),
          orc.mx_experts(*base, activation="situv2", beta=3.0, linear_beta=5.0), "situv2")
    check(run(doweight_stage1=True), orc.mx_experts(*base, weight_in_stage1=True), "stage1")
    # experts 0, 2, 3, 5, 6 held here; rows from 211 on were not received
    mask = torch.tensor([1, 0, 1, 1, 0, 1, 1, 0], dtype=torch.int32)
    held = mask.bool()
    slot = torch.where(held[ids.long()], (mask.long().cumsum(0) - 1)[ids.long()], -1)
    received = torch.tensor([211], dtype=torch.int32)
    out = run(w1=w1[held], w1_scale=s1[held], w2=w2[held], w2_scale=s2[held], expert_mask=mask.to(d), num_local_tokens=received.to(d))
    ref = orc.mx_experts(x, slot, wts, w1[held], s1[held], w2[held], s2[held], num_local_tokens=211)
    check(out, ref, "mask + rows received")
    assert not out[211:].any() and out[:211].any()
    # activations kept in bf16, as the reference keeps them: gate_mode 'interleave' (silu with its clamp; the op's
    # default act_quant) with the mask and the rows-received bound, and gpt-oss swiglu below 256 tokens
    kept = dict(quant_type="per_1x32", w1_scale=s1[held].to(d), w2_scale=s2[held].to(d))
    out = ops.fused_moe(x.to(d), w1[held].to(d), w2[held].to(d), wts.to(d), ids.to(d), expert_mask=mask.to(d), gate_mode="interleave",
                        swiglu_limit=7.0, num_local_tokens=received.to(d), **kept)
    check(out, orc.mx_experts(x, slot, wts, w1[held], s1[held], w2[held], s2[held], num_local_tokens=211, swiglu_limit=7.0, act_bits=16),
          "interleave: bf16 activations")
    few = dict(quant_type="per_1x32", w1_scale=s1.to(d), w2_scale=s2.to(d), act_quant=8)
    out = ops.fused_moe(x[:100].to(d), w1.to(d), w2.to(d), wts[:100].to(d), ids[:100].to(d), activation="swiglu", swiglu_limit=7.0, **few)
    check(out, orc.mx_experts(x[:100], ids[:100].long(), wts[:100], w1, s1, w2, s2, activation="swiglu", swiglu_limit=7.0, act_bits=16),
          "swiglu below 256 rows: bf16 activations")
    # out of contract: swiglu or interleave without the clamp, interleave with another activation, situv2 without its
    # betas, a row count without a mask, activation bits other than 4 or 8
    assert run(activation="swiglu") is ops.FallbackReason.OUT_OF_CONTRACT
    assert run(gate_mode="interleave") is ops.FallbackReason.OUT_OF_CONTRACT
    assert run(gate_mode="interleave", activation="gelu", swiglu_limit=7.0) is ops.FallbackReason.OUT_OF_CONTRACT
    # the op's default arguments: MXFP4 activations (act_quant 4)
    out = ops.fused_moe(x.to(d), w1.to(d), w2.to(d), wts.to(d), ids.to(d), quant_type="per_1x32", w1_scale=s1.to(d), w2_scale=s2.to(d))
    assert isinstance(out, torch.Tensor)
    a4 = orc.output_gates(out.cpu(), orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, act_bits=4))
    assert a4["sqnr_db"] >= 25.0 and a4["cosine"] >= 0.998, a4
    assert ops.fused_moe(x.to(d), w1.to(d), w2.to(d), wts.to(d), ids.to(d), quant_type="per_1x32", w1_scale=s1.to(d),
                         w2_scale=s2.to(d), act_quant=6) is ops.FallbackReason.OUT_OF_CONTRACT
    assert run(activation="situv2", beta=3.0) is ops.FallbackReason.OUT_OF_CONTRACT
    assert run(num_local_tokens=received.to(d)) is ops.FallbackReason.OUT_OF_CONTRACT


def test_biased_grouped_topk_and_quant_ops(ops, golden):
    logits, bias = cases.bgt()
    d = dev()
    w = torch.empty((96, 8), dtype=torch.float32, device=d)
    ids = torch.empty((96, 8), dtype=torch.int32, device=d)
    got_w, got_ids = ops.biased_grouped_topk(logits.to(d), bias.to(d), w, ids, 1, 1, True, 2.5)
    assert got_w is w and got_ids is ids
    assert torch.equal(ids.cpu(), torch.from_numpy(np.asarray(golden["bgt.ids"])))
    torch.testing.assert_close(w.cpu(), torch.from_numpy(np.asarray(golden["bgt.weights"])), atol=1e-4, rtol=1e-4)
    x = cases.quant_x().to(d)
    q, s = ops.per_group_quant_fp8(x)
    assert torch.equal(q.cpu().float(), torch.from_numpy(np.asarray(golden["quant_fp8.q"])))
    assert s.shape == (4, 24)
    q, s = ops.per_group_quant_mxfp8(x)
    assert torch.equal(s.cpu(), torch.from_numpy(np.asarray(golden["quant_mxfp8.s"])))


def test_mega_moe_op_single_rank_and_emulated_group(ops):
    """ep_size 1 through the op; four emulated ranks through the phases, against the oracle over all
    experts with the reference's clamp at 10."""
    from aklr_b200.ep import CudaKernels, ExpertParallelMoE, run_in_process
    from aklr_b200.moe import Routing

    cfg = wl.MoEConfig("mx", hidden=256, inter=128, n_routed=8, topk=2)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed=11)
    d = dev()

    def inputs(seed, tokens):
        g = torch.Generator().manual_seed(seed)
        x = (torch.randn(tokens, 256, generator=g) * 3).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(8, generator=g)[:2] for _ in range(tokens)]).to(torch.int32)
        return x, ids, torch.rand(tokens, 2, generator=g)

    x, ids, wts = inputs(1, 50)
    out = ops.mega_moe(x.to(d), w1.to(d), w2.to(d), wts.to(d), ids.to(d), w1_scale=s1.to(d), w2_scale=s2.to(d), ep_size=1)
    assert isinstance(out, torch.Tensor)
    ref = orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, swiglu_limit=10.0)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates), gates

    world, layers, ins = 4, [], []
    for r in range(world):
        mine = slice(2 * r, 2 * r + 2)
        layers.append(ExpertParallelMoE(Routing(topk=2), w1[mine].to(d), s1[mine].to(d), w2[mine].to(d), s2[mine].to(d), r, world,
                                        kernels=CudaKernels("mxfp4", 10.0)))
        xr, idr, wtr = inputs(20 + r, 9 + 5 * r)
        ins.append((xr.to(d), None, None, (idr.to(d), wtr.to(d))))
    outs = run_in_process(layers, ins)
    for r in range(world):
        xr, idr, wtr = inputs(20 + r, 9 + 5 * r)
        ref = orc.mx_experts(xr, idr.long(), wtr, w1, s1, w2, s2, swiglu_limit=10.0)
        gates = orc.output_gates(outs[r].cpu(), ref)
        assert orc.gates_pass(gates), (r, gates)

    # from 512 tokens per rank the sender quantises each token once and copies its rows per route
    world, layers, ins = 2, [], []
    for r in range(world):
        mine = slice(4 * r, 4 * r + 4)
        layers.append(ExpertParallelMoE(Routing(topk=2), w1[mine].to(d), s1[mine].to(d), w2[mine].to(d), s2[mine].to(d), r, world,
                                        kernels=CudaKernels("mxfp4", 10.0)))
        xr, idr, wtr = inputs(40 + r, 520 + 80 * r)
        ins.append((xr.to(d), None, None, (idr.to(d), wtr.to(d))))
    outs = run_in_process(layers, ins)
    for r in range(world):
        xr, idr, wtr = inputs(40 + r, 520 + 80 * r)
        ref = orc.mx_experts(xr, idr.long(), wtr, w1, s1, w2, s2, swiglu_limit=10.0)
        gates = orc.output_gates(outs[r].cpu(), ref)
        assert orc.gates_pass(gates), (r, gates)
