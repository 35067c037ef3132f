"""The fused-MoE ops with the reference's api signatures, served by the sm_100a kernels.

    from aklr_b200 import ops
    ops.init()                                   # once per process, on the GPU rank's device
    out = ops.deepseek_v2_fp8_moe(hidden_states=..., router_weight=..., ...)
    if isinstance(out, ops.FallbackReason): ...  # run the engine's own code

Signatures follow aklr/plugins/sglang/models/deepseek_v2/api.py:35-50,
aklr/plugins/sglang/models/qwen3_moe/api.py:14-23, aklr/ops/fused_moe/api.py:17-44,
aklr/ops/topk/api.py:12-22 and aklr/ops/quant/api.py:8-13 parameter for parameter.
"""

from __future__ import annotations

import math
from collections.abc import Mapping
from typing import Any

import torch

from aklr_b200 import moe
from aklr_b200.core.dispatch import (
    DispatcherRegistry,
    FallbackReason,
    LoadError,
    OpContract,
    Param,
    api,
    overlaps,
    tensor_ok,
)

__all__ = [
    "FallbackReason",
    "LoadError",
    "biased_grouped_topk",
    "deepseek_v2_fp8_moe",
    "deepseek_v2_mxfp4_moe",
    "fused_moe",
    "init",
    "mega_moe",
    "minimax_m2_fp8_moe",
    "minimax_m2_mxfp4_moe",
    "per_group_quant_fp8",
    "per_group_quant_mxfp8",
    "qwen2_moe_fp8_experts",
    "qwen2_moe_fp8_router_experts",
    "qwen2_moe_mxfp4_moe",
    "qwen2_moe_router",
    "qwen3_moe_fp8_moe",
]

FP8 = torch.float8_e4m3fn
BF16 = torch.bfloat16
MAX_TOKENS = 65536


def init() -> None:
    """Start the runtime once per process (probe the device, load the library, open the ops)."""
    DispatcherRegistry.default().init_once()


def _attr_name(value: Any) -> Any:
    """An enum-like attr by its lower-case name, so engine enums match strings (the reference's
    attr_value, aklr/core/contract/spec/_points.py:45-59)."""
    name = getattr(value, "name", None)
    return name.lower() if isinstance(name, str) else (value.lower() if isinstance(value, str) else value)


def _layout(call: Mapping[str, Any]) -> str:
    """The weights' layout variant, first element of a dispatch key (the reference keys its variants the same way,
    aklr/plugins/sglang/models/deepseek_v2/contract.py:310-318)."""
    return "b200_tiled" if getattr(call["w1"], "is_b200_tiled", False) else "row_major"


def _fp8_weights_key(call: Mapping[str, Any], hidden: int, device) -> tuple | None:
    """(experts, inter) when w1/w2 and their 128 x 128 block scales are well formed, row-major."""
    w1, w2, s1, s2 = call["w1"], call["w2"], call["w1_scale"], call["w2_scale"]
    if not (tensor_ok(w1, FP8, 3, device) and tensor_ok(w2, FP8, 3, device)):
        return None
    if not (tensor_ok(s1, torch.float32, 3, device) and tensor_ok(s2, torch.float32, 3, device)):
        return None
    # the aiter-shuffled layout (16 x 16 tiles) is another layout variant, not served here
    if getattr(w1, "is_shuffled", False) or getattr(w2, "is_shuffled", False):
        return None
    # row-major as the checkpoint stores them, or both tile-contiguous (aklr_b200.layouts.to_b200_tiled)
    if bool(getattr(w1, "is_b200_tiled", False)) != bool(getattr(w2, "is_b200_tiled", False)):
        return None
    e, two_i, h = w1.shape
    inter = two_i // 2
    if h != hidden or two_i % 256 or hidden % 128 or not (128 <= inter <= 16384 and 128 <= hidden <= 16384):
        return None
    if tuple(w2.shape) != (e, hidden, inter):
        return None
    if tuple(s1.shape) != (e, two_i // 128, hidden // 128) or tuple(s2.shape) != (e, hidden // 128, inter // 128):
        return None
    return e, inter


# --------------------------------------------------------------------------------------------------
# deepseek_v2_fp8_moe@1.0  (aklr/plugins/sglang/models/deepseek_v2/contract.py:188-320)
# --------------------------------------------------------------------------------------------------
def _deepseek_key(call):
    x, rw, bias = call["hidden_states"], call["router_weight"], call["correction_bias"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS):
        return None
    if not tensor_ok(rw, BF16, 2, device) or rw.shape[1] != hidden:
        return None
    n_routed = rw.shape[0]
    if not tensor_ok(bias, BF16, 1, device) or bias.shape[0] != n_routed:
        return None
    weights = _fp8_weights_key(call, hidden, device)
    if weights is None or weights[0] != n_routed + 1 or not (1 <= n_routed <= 1024):
        return None
    topk, groups, topk_group = call["topk"], call["num_expert_group"], call["topk_group"]
    if not all(isinstance(v, int) and not isinstance(v, bool) for v in (topk, groups, topk_group)):
        return None
    if _attr_name(call["scoring_func"]) != "sigmoid" or not isinstance(call["renormalize"], bool):
        return None
    factor = call["routed_scaling_factor"]
    if not isinstance(factor, (int, float)) or not math.isfinite(factor) or factor <= 0:
        return None
    if (
        groups < 1
        or groups > 32
        or n_routed % groups
        or (groups > 1 and n_routed // groups < 2)
        or not (1 <= topk_group <= groups)
        or not (1 <= topk <= min(31, topk_group * (n_routed // groups)))
    ):
        return None
    return (_layout(call), hidden, n_routed, weights[1], topk, groups, topk_group, call["renormalize"], float(factor))


def _layer_alloc(call, key):
    return torch.empty_like(call["hidden_states"])


def _deepseek_run(call, out):
    x = call["hidden_states"]
    logits = moe.router_logits(x, call["router_weight"])
    routing = moe.Routing(
        topk=call["topk"],
        scoring="sigmoid",
        n_shared=1,
        num_expert_group=call["num_expert_group"],
        topk_group=call["topk_group"],
        renormalize=call["renormalize"],
        routed_scaling_factor=float(call["routed_scaling_factor"]),
    )
    moe.fused_moe_fp8(
        x, logits, call["correction_bias"], call["w1"], call["w1_scale"], call["w2"], call["w2_scale"], routing, out=out
    )


DEEPSEEK_V2_FP8_MOE = OpContract(
    contract_id="deepseek_v2_fp8_moe@1.0",
    description=(
        "sglang's DeepseekV2MoE on one rank with fp8 experts at a scale per 128 x 128 block and the "
        "shared expert in their last slot: router logits in bf16, sigmoid scores + correction bias, "
        "grouped top-k, renormalised unbiased scores x routed_scaling_factor, shared expert at "
        "weight 1; each expert down(silu(gate(x)) * up(x)) with both linears' inputs in bf16 then "
        "fp8 per 1 x 128 at amax/448."
    ),
    params=[
        Param("hidden_states"),
        Param("router_weight"),
        Param("correction_bias"),
        Param("w1"),
        Param("w1_scale"),
        Param("w2"),
        Param("w2_scale"),
        Param("topk"),
        Param("num_expert_group"),
        Param("topk_group"),
        Param("renormalize"),
        Param("scoring_func"),
        Param("routed_scaling_factor"),
    ],
    outputs=["out"],
    key=_deepseek_key,
    alloc=_layer_alloc,
    run=_deepseek_run,
)


# --------------------------------------------------------------------------------------------------
# deepseek_v2_mxfp4_moe@1.0 (aklr/plugins/sglang/models/deepseek_v2/contract.py:93-176): the same block with
# MXFP4 experts, ungrouped routing, a float32 correction bias, and activations that are never quantised
# --------------------------------------------------------------------------------------------------
def _deepseek_mx_key(call):
    x, rw, bias = call["hidden_states"], call["router_weight"], call["correction_bias"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS):
        return None
    if not tensor_ok(rw, BF16, 2, device) or rw.shape[1] != hidden:
        return None
    n_routed = rw.shape[0]
    if not tensor_ok(bias, torch.float32, 1, device) or bias.shape[0] != n_routed:
        return None
    weights = _mx_weights_key(call, hidden, device)
    if weights is None or weights[0] != n_routed + 1 or not (1 <= n_routed <= 1024) or weights[1] % 256:
        return None
    topk = call["topk"]
    if not isinstance(topk, int) or isinstance(topk, bool) or not (1 <= topk <= min(31, n_routed)):
        return None
    if call["num_expert_group"] != 1 or call["topk_group"] != 1:
        return None
    if _attr_name(call["scoring_func"]) != "sigmoid" or not isinstance(call["renormalize"], bool):
        return None
    factor = call["routed_scaling_factor"]
    if not isinstance(factor, (int, float)) or not math.isfinite(factor) or factor <= 0:
        return None
    return ("row_major", hidden, n_routed, weights[1], topk, call["renormalize"], float(factor))


def _deepseek_mx_run(call, out):
    x = call["hidden_states"]
    logits = moe.router_logits(x, call["router_weight"])
    routing = moe.Routing(topk=call["topk"], scoring="sigmoid", n_shared=1, renormalize=call["renormalize"],
                          routed_scaling_factor=float(call["routed_scaling_factor"]))
    moe.fused_moe_mxfp4(
        x, logits, call["correction_bias"], call["w1"].view(torch.uint8), call["w1_scale"].view(torch.uint8),
        call["w2"].view(torch.uint8), call["w2_scale"].view(torch.uint8), routing, out=out, act_bits=16,
    )


DEEPSEEK_V2_MXFP4_MOE = OpContract(
    contract_id="deepseek_v2_mxfp4_moe@1.0",
    description=(
        "sglang's DeepseekV2MoE on one rank with MXFP4 experts (fp4 values at an e8m0 scale per 32) and the shared "
        "expert in their last slot: router logits in bf16, sigmoid scores + float32 correction bias, plain top-k, "
        "renormalised unbiased scores x routed_scaling_factor, shared expert at weight 1; each expert "
        "down(silu(gate(x)) * up(x)) on activations that are not quantised."
    ),
    params=list(DEEPSEEK_V2_FP8_MOE.params),
    outputs=["out"],
    key=_deepseek_mx_key,
    alloc=_layer_alloc,
    run=_deepseek_mx_run,
)


@api(DEEPSEEK_V2_MXFP4_MOE)
def deepseek_v2_mxfp4_moe(
    hidden_states,
    router_weight,
    correction_bias,
    w1,
    w1_scale,
    w2,
    w2_scale,
    topk,
    num_expert_group,
    topk_group,
    renormalize,
    scoring_func,
    routed_scaling_factor,
): ...


@api(DEEPSEEK_V2_FP8_MOE)
def deepseek_v2_fp8_moe(
    hidden_states,
    router_weight,
    correction_bias,
    w1,
    w1_scale,
    w2,
    w2_scale,
    topk,
    num_expert_group,
    topk_group,
    renormalize,
    scoring_func,
    routed_scaling_factor,
): ...


# --------------------------------------------------------------------------------------------------
# qwen3_moe_fp8_moe@1.0  (aklr/plugins/sglang/models/qwen3_moe/contract.py:61-146; topk 2 added
# for the Mixtral-shaped configuration)
# --------------------------------------------------------------------------------------------------
def _qwen3_key(call):
    x, rw = call["hidden_states"], call["router_weight"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS) or not tensor_ok(rw, BF16, 2, device) or rw.shape[1] != hidden:
        return None
    n_routed = rw.shape[0]
    weights = _fp8_weights_key(call, hidden, device)
    if weights is None or weights[0] != n_routed or not (1 <= n_routed <= 1024):
        return None
    topk = call["topk"]
    if not isinstance(topk, int) or isinstance(topk, bool) or not (1 <= topk <= min(32, n_routed)):
        return None
    return (_layout(call), hidden, n_routed, weights[1], topk)


def _qwen3_run(call, out):
    x = call["hidden_states"]
    logits = moe.router_logits(x, call["router_weight"])
    moe.fused_moe_fp8(
        x, logits, None, call["w1"], call["w1_scale"], call["w2"], call["w2_scale"], moe.Routing(topk=call["topk"]), out=out
    )


QWEN3_MOE_FP8_MOE = OpContract(
    contract_id="qwen3_moe_fp8_moe@1.0",
    description=(
        "sglang's Qwen3MoeSparseMoeBlock on one rank with fp8 experts at a scale per 128 x 128 block: "
        "bf16 router logits, top-k by logit (ties to the lower id), softmax over the chosen, experts as "
        "in deepseek_v2_fp8_moe."
    ),
    params=[
        Param("hidden_states"),
        Param("router_weight"),
        Param("w1"),
        Param("w1_scale"),
        Param("w2"),
        Param("w2_scale"),
        Param("topk", 8),
    ],
    outputs=["out"],
    key=_qwen3_key,
    alloc=_layer_alloc,
    run=_qwen3_run,
)


@api(QWEN3_MOE_FP8_MOE)
def qwen3_moe_fp8_moe(
    hidden_states,
    router_weight,
    w1,
    w1_scale,
    w2,
    w2_scale,
    topk=8,
): ...


# --------------------------------------------------------------------------------------------------
# minimax_m2_fp8_moe@1.0  (aklr/plugins/sglang/models/minimax_m2/contract.py:48-110, api.py:17-28)
# --------------------------------------------------------------------------------------------------
def _minimax_key(call, mx: bool = False):
    x, rw, bias = call["hidden_states"], call["router_weight"], call["correction_bias"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS) or not tensor_ok(rw, torch.float32, 2, device) or rw.shape[1] != hidden:
        return None
    n_routed = rw.shape[0]
    if not (1 <= n_routed <= 1024) or not tensor_ok(bias, torch.float32, 1, device) or bias.shape[0] != n_routed:
        return None
    weights = (_mx_weights_key if mx else _fp8_weights_key)(call, hidden, device)
    if weights is None or not (1 <= weights[0] <= n_routed) or (mx and weights[1] % 256):
        return None
    topk, offset = call["topk"], call["expert_offset"]
    if not all(isinstance(v, int) and not isinstance(v, bool) for v in (topk, offset)):
        return None
    if not (1 <= topk <= min(32, n_routed)) or not (0 <= offset and offset + weights[0] <= n_routed):
        return None
    return (_layout(call), hidden, n_routed, weights[0], weights[1], topk, offset)


_EXPERT_MAPS: dict[tuple, torch.Tensor] = {}


def _held_expert_map(n_routed: int, offset: int, n_experts: int, device) -> torch.Tensor | None:
    """int32 [n_routed]: router row -> this rank's expert slot, -1 for experts held elsewhere."""
    if offset == 0 and n_experts == n_routed:
        return None
    key = (n_routed, offset, n_experts, str(device))
    if key not in _EXPERT_MAPS:
        table = torch.full((n_routed,), -1, dtype=torch.int32)
        table[offset : offset + n_experts] = torch.arange(n_experts, dtype=torch.int32)
        _EXPERT_MAPS[key] = table.to(device)
    return _EXPERT_MAPS[key]


def _minimax_run(call, out):
    x = call["hidden_states"]
    logits = moe.router_logits_f32(x, call["router_weight"])
    routing = moe.Routing(topk=call["topk"], scoring="sigmoid", renormalize=True, routed_scaling_factor=1.0)
    ids, weights = moe.route(logits, call["correction_bias"], routing)
    table = _held_expert_map(logits.shape[1], call["expert_offset"], call["w1"].shape[0], x.device)
    moe.fused_experts_fp8(
        x, ids, weights, call["w1"], call["w1_scale"], call["w2"], call["w2_scale"], expert_map=table, out=out
    )


MINIMAX_M2_FP8_MOE = OpContract(
    contract_id="minimax_m2_fp8_moe@1.0",
    description=(
        "sglang's MiniMaxM2MoE on one rank with fp8 experts at a scale per 128 x 128 block: float32 gate "
        "logits, each token's topk experts of the n_routed by sigmoid score + correction_bias, weighed by "
        "their unbiased scores renormalised to sum 1; out is the share of the experts this rank holds "
        "(expert_offset .. expert_offset + n_experts - 1), not yet summed over the ranks."
    ),
    params=[
        Param("hidden_states"),
        Param("router_weight"),
        Param("correction_bias"),
        Param("w1"),
        Param("w1_scale"),
        Param("w2"),
        Param("w2_scale"),
        Param("topk"),
        Param("expert_offset", 0),
    ],
    outputs=["out"],
    key=_minimax_key,
    alloc=_layer_alloc,
    run=_minimax_run,
)


def _minimax_mx_run(call, out):
    x = call["hidden_states"]
    logits = moe.router_logits_f32(x, call["router_weight"])
    routing = moe.Routing(topk=call["topk"], scoring="sigmoid", renormalize=True, routed_scaling_factor=1.0)
    ids, weights = moe.route(logits, call["correction_bias"], routing)
    table = _held_expert_map(logits.shape[1], call["expert_offset"], call["w1"].shape[0], x.device)
    moe.fused_experts_mxfp4(
        x, ids, weights, call["w1"].view(torch.uint8), call["w1_scale"].view(torch.uint8), call["w2"].view(torch.uint8),
        call["w2_scale"].view(torch.uint8), expert_map=table, out=out, act_bits=16,
    )


# minimax_m2_mxfp4_moe@1.0 (aklr/plugins/sglang/models/minimax_m2/contract.py, api.py:31-42; reference.py:114-132):
# the same routing over MXFP4 experts, activations never quantised
MINIMAX_M2_MXFP4_MOE = OpContract(
    contract_id="minimax_m2_mxfp4_moe@1.0",
    description=(
        "sglang's MiniMaxM2MoE on one rank with MXFP4 experts (fp4 values at an e8m0 scale per 32): float32 gate "
        "logits, biased sigmoid top-k, renormalised unbiased scores; each held expert down(silu(gate(x)) * up(x)) on "
        "activations that are not quantised; out is this rank's share."
    ),
    params=list(MINIMAX_M2_FP8_MOE.params),
    outputs=["out"],
    key=lambda call: _minimax_key(call, mx=True),
    alloc=_layer_alloc,
    run=_minimax_mx_run,
)


@api(MINIMAX_M2_MXFP4_MOE)
def minimax_m2_mxfp4_moe(
    hidden_states,
    router_weight,
    correction_bias,
    w1,
    w1_scale,
    w2,
    w2_scale,
    topk,
    expert_offset=0,
): ...


@api(MINIMAX_M2_FP8_MOE)
def minimax_m2_fp8_moe(
    hidden_states,
    router_weight,
    correction_bias,
    w1,
    w1_scale,
    w2,
    w2_scale,
    topk,
    expert_offset=0,
): ...


# --------------------------------------------------------------------------------------------------
# qwen2_moe_router@1.0, qwen2_moe_fp8_experts@1.0, qwen2_moe_fp8_router_experts@1.0
# (aklr/plugins/sglang/models/qwen2_moe/contract.py:161-265, api.py:24-52): softmax top-k over bf16
# logits, FP8 experts, and a shared expert in w1/w2's last slot weighed by sigmoid(x . shared_gate_weight)
# --------------------------------------------------------------------------------------------------
def _qwen2_common_key(call, with_router: bool):
    x, gate = call["hidden_states"], call["shared_gate_weight"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS) or not tensor_ok(gate, BF16, 2, device) or tuple(gate.shape) != (1, hidden):
        return None
    weights = _fp8_weights_key(call, hidden, device)
    if weights is None or not (2 <= weights[0] <= 1025):
        return None
    n_routed = weights[0] - 1
    if with_router:
        rw = call["router_weight"]
        if not tensor_ok(rw, BF16, 2, device) or tuple(rw.shape) != (n_routed, hidden):
            return None
    return n_tokens, hidden, n_routed, weights[1]


def _qwen2_router_experts_key(call):
    common = _qwen2_common_key(call, True)
    topk = call["topk"]
    if common is None or not isinstance(topk, int) or isinstance(topk, bool) or not (1 <= topk <= min(31, common[2])):
        return None
    return (_layout(call), *common[1:], topk)


def _qwen2_router_experts_run(call, out):
    x = call["hidden_states"]
    logits = moe.router_logits(x, call["router_weight"])
    topk, n_routed = call["topk"], logits.shape[1]
    ids, weights = moe.route(logits, None, moe.Routing(topk=topk, n_shared=1))  # slot topk = the shared expert
    moe.with_gated_shared_slot(x, call["shared_gate_weight"], ids, weights, n_routed)
    moe.fused_experts_fp8(x, ids, weights, call["w1"], call["w1_scale"], call["w2"], call["w2_scale"], out=out)


QWEN2_MOE_FP8_ROUTER_EXPERTS = OpContract(
    contract_id="qwen2_moe_fp8_router_experts@1.0",
    description=(
        "sglang's Qwen2MoeSparseMoeBlock router and experts on one rank with the shared expert fused in after "
        "the routed ones: bf16 router logits, top-k by logit (ties to the lower id), softmax over the chosen, "
        "and the shared expert by sigmoid(hidden_states shared_gate_weight^T); fp8 experts as in "
        "deepseek_v2_fp8_moe."
    ),
    params=[
        Param("hidden_states"),
        Param("router_weight"),
        Param("shared_gate_weight"),
        Param("w1"),
        Param("w1_scale"),
        Param("w2"),
        Param("w2_scale"),
        Param("topk", 10),
    ],
    outputs=["out"],
    key=_qwen2_router_experts_key,
    alloc=_layer_alloc,
    run=_qwen2_router_experts_run,
)


@api(QWEN2_MOE_FP8_ROUTER_EXPERTS)
def qwen2_moe_fp8_router_experts(
    hidden_states,
    router_weight,
    shared_gate_weight,
    w1,
    w1_scale,
    w2,
    w2_scale,
    topk=10,
): ...


def _qwen2_experts_key(call):
    common = _qwen2_common_key(call, False)
    if common is None:
        return None
    n_tokens, _, n_routed, _ = common
    wts, ids = call["topk_weights"], call["topk_ids"]
    device = call["hidden_states"].device
    if not tensor_ok(wts, torch.float32, 2, device) or not tensor_ok(ids, torch.int32, 2, device):
        return None
    if wts.shape != ids.shape or wts.shape[0] != n_tokens or not (1 <= wts.shape[1] <= min(31, n_routed)):
        return None
    return (_layout(call), *common[1:], wts.shape[1])


def _qwen2_experts_run(call, out):
    x, ids_in, w_in = call["hidden_states"], call["topk_ids"], call["topk_weights"]
    n_tokens, topk = ids_in.shape
    ids = torch.empty((n_tokens, topk + 1), dtype=torch.int32, device=x.device)
    weights = torch.empty((n_tokens, topk + 1), dtype=torch.float32, device=x.device)
    moe.with_gated_shared_slot(x, call["shared_gate_weight"], ids, weights, call["w1"].shape[0] - 1, copy_from=(ids_in, w_in))
    moe.fused_experts_fp8(x, ids, weights, call["w1"], call["w1_scale"], call["w2"], call["w2_scale"], out=out)


QWEN2_MOE_FP8_EXPERTS = OpContract(
    contract_id="qwen2_moe_fp8_experts@1.0",
    description=(
        "sglang's Qwen2MoeSparseMoeBlock experts on one rank at a given routing, the gated shared expert fused "
        "in after the routed ones (w1/w2's last slot)."
    ),
    params=[
        Param("hidden_states"),
        Param("topk_weights"),
        Param("topk_ids"),
        Param("shared_gate_weight"),
        Param("w1"),
        Param("w1_scale"),
        Param("w2"),
        Param("w2_scale"),
    ],
    outputs=["out"],
    key=_qwen2_experts_key,
    alloc=_layer_alloc,
    run=_qwen2_experts_run,
)


@api(QWEN2_MOE_FP8_EXPERTS)
def qwen2_moe_fp8_experts(
    hidden_states,
    topk_weights,
    topk_ids,
    shared_gate_weight,
    w1,
    w1_scale,
    w2,
    w2_scale,
): ...


# --------------------------------------------------------------------------------------------------
# qwen2_moe_mxfp4_moe@1.0 (aklr/plugins/sglang/models/qwen2_moe/contract.py:308-394, api.py:55-66): the whole
# block with MXFP4 routed experts on unquantised activations and the shared expert apart in bf16
# --------------------------------------------------------------------------------------------------
def _qwen2_mx_key(call):
    x, rw, gate = call["hidden_states"], call["router_weight"], call["shared_gate_weight"]
    sw1, sw2, topk = call["shared_w1"], call["shared_w2"], call["topk"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS) or not tensor_ok(gate, BF16, 2, device) or tuple(gate.shape) != (1, hidden):
        return None
    if not tensor_ok(rw, BF16, 2, device) or rw.shape[1] != hidden or not (1 <= rw.shape[0] <= 1024):
        return None
    n_routed = rw.shape[0]
    weights = _mx_weights_key(call, hidden, device)
    if weights is None or weights[0] != n_routed or weights[1] % 256:
        return None
    if not tensor_ok(sw1, BF16, 2, device) or not tensor_ok(sw2, BF16, 2, device):
        return None
    shared_inter = sw2.shape[1]
    if tuple(sw1.shape) != (2 * shared_inter, hidden) or sw2.shape[0] != hidden or shared_inter % 128 or not (128 <= shared_inter <= 16384):
        return None
    if not isinstance(topk, int) or isinstance(topk, bool) or not (1 <= topk <= min(32, n_routed)):
        return None
    return ("row_major", hidden, n_routed, weights[1], shared_inter, topk)


def _qwen2_mx_run(call, out):
    x = call["hidden_states"]
    logits = moe.router_logits(x, call["router_weight"])
    ids, weights = moe.route(logits, None, moe.Routing(topk=call["topk"]))
    moe.fused_experts_mxfp4(
        x, ids, weights, call["w1"].view(torch.uint8), call["w1_scale"].view(torch.uint8), call["w2"].view(torch.uint8),
        call["w2_scale"].view(torch.uint8), out=out, act_bits=16,
    )
    moe.add_bf16_shared_expert(x, call["shared_w1"], call["shared_w2"], call["shared_gate_weight"], out)


QWEN2_MOE_MXFP4_MOE = OpContract(
    contract_id="qwen2_moe_mxfp4_moe@1.0",
    description=(
        "sglang's Qwen2MoeSparseMoeBlock.forward on one rank with MXFP4 routed experts and the shared expert apart in "
        "bf16: bf16 router logits, top-k by logit, softmax over the chosen; each routed expert down(silu(gate(x)) * "
        "up(x)) of its MXFP4 weights on unquantised activations; the shared expert of its bf16 weights weighed by "
        "sigmoid(hidden_states shared_gate_weight^T) and added; out is this rank's share."
    ),
    params=[
        Param("hidden_states"),
        Param("router_weight"),
        Param("w1"),
        Param("w1_scale"),
        Param("w2"),
        Param("w2_scale"),
        Param("shared_w1"),
        Param("shared_w2"),
        Param("shared_gate_weight"),
        Param("topk", 10),
    ],
    outputs=["out"],
    key=_qwen2_mx_key,
    alloc=_layer_alloc,
    run=_qwen2_mx_run,
)


@api(QWEN2_MOE_MXFP4_MOE)
def qwen2_moe_mxfp4_moe(
    hidden_states,
    router_weight,
    w1,
    w1_scale,
    w2,
    w2_scale,
    shared_w1,
    shared_w2,
    shared_gate_weight,
    topk=10,
): ...


def _qwen2_router_key(call):
    x, rw, wts, ids = call["hidden_states"], call["router_weight"], call["topk_weights"], call["topk_ids"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS) or not tensor_ok(rw, BF16, 2, device) or rw.shape[1] != hidden or hidden % 8:
        return None
    n_routed = rw.shape[0]
    if not tensor_ok(wts, torch.float32, 2, device) or not tensor_ok(ids, torch.int32, 2, device):
        return None
    if wts.shape != ids.shape or wts.shape[0] != n_tokens or not (1 <= wts.shape[1] <= min(32, n_routed)) or n_routed > 1024:
        return None
    if overlaps(wts, ids) or overlaps(wts, x) or overlaps(ids, x):
        return None
    return (hidden, n_routed, wts.shape[1])


def _qwen2_router_alloc(call, key):
    return call["topk_weights"], call["topk_ids"]


def _qwen2_router_run(call, outputs):
    logits = moe.router_logits(call["hidden_states"], call["router_weight"])
    moe.route(logits, None, moe.Routing(topk=call["topk_ids"].shape[1]), call["topk_ids"], call["topk_weights"])


QWEN2_MOE_ROUTER = OpContract(
    contract_id="qwen2_moe_router@1.0",
    description=(
        "sglang's Qwen2MoeSparseMoeBlock router: bf16 logits, each token's topk experts by descending logit "
        "(ties to the lower id) weighed by the softmax of their logits."
    ),
    params=[Param("hidden_states"), Param("router_weight"), Param("topk_weights"), Param("topk_ids")],
    outputs=["topk_weights", "topk_ids"],
    key=_qwen2_router_key,
    alloc=_qwen2_router_alloc,
    run=_qwen2_router_run,
)


@api(QWEN2_MOE_ROUTER)
def qwen2_moe_router(hidden_states, router_weight, topk_weights, topk_ids): ...


# --------------------------------------------------------------------------------------------------
# fused_moe@1.0 -- experts only, routing given (aklr/ops/fused_moe/contract.py:75-300).  The
# reference's Points are MXFP4 (quant_type per_1x32); this build serves the FP8 block-scaled
# format, quant_type "per_128x128" (the aiter enum name sglang passes for it,
# aklr/plugins/sglang/models/deepseek_v2/baseline.py:159).
# --------------------------------------------------------------------------------------------------
def _mx_weights_key(call: Mapping[str, Any], hidden: int, device) -> tuple | None:
    """(experts, inter) when w1/w2 are packed e2m1 (uint8 or float4_e2m1fn_x2) with e8m0 scales per 32."""
    w1, w2, s1, s2 = call["w1"], call["w2"], call["w1_scale"], call["w2_scale"]
    fp4 = (torch.uint8,) + ((torch.float4_e2m1fn_x2,) if hasattr(torch, "float4_e2m1fn_x2") else ())
    e8 = (torch.uint8,) + ((torch.float8_e8m0fnu,) if hasattr(torch, "float8_e8m0fnu") else ())
    if not (tensor_ok(w1, fp4, 3, device) and tensor_ok(w2, fp4, 3, device) and tensor_ok(s1, e8, 3, device) and tensor_ok(s2, e8, 3, device)):
        return None
    if getattr(w1, "is_b200_tiled", False) or getattr(w2, "is_b200_tiled", False):
        return None  # the tile-contiguous layout is an FP8 layout
    e, two_i, half_h = w1.shape
    inter = two_i // 2
    if half_h * 2 != hidden or hidden % 256 or inter % 128 or two_i % 256:
        return None
    if tuple(w2.shape) != (e, hidden, inter // 2) or tuple(s1.shape) != (e, two_i, hidden // 32) or tuple(s2.shape) != (e, hidden, inter // 32):
        return None
    return e, inter


def _mx_act_bits(call, activation: str, n_tokens: int) -> int | None:
    """Bits the activations keep on the MXFP4 path, as the reference decides it
    (aklr/ops/fused_moe/reference.py:90-97): 16 (bf16, nothing rounded) under gate_mode 'interleave' and for
    gpt-oss swiglu below 256 rows, whatever act_quant says; else act_quant: 4 (MXFP4, the default) or 8 (MXFP8)."""
    if call["gate_mode"] == "interleave" or (activation == "swiglu" and n_tokens < 256):
        return 16
    return call["act_quant"] if call["act_quant"] in (4, 8) and not isinstance(call["act_quant"], bool) else None


def _fused_moe_mx_key(call, x, device, n_tokens, hidden):
    """MXFP4 experts (quant_type per_1x32), weights row-major with gate rows before up rows.  Activations
    quantised to MXFP8 (act_quant 8), or kept in bf16 where the reference keeps them: gate_mode 'interleave'
    (DeepSeek-V4's clamped SwiGLU: silu with its clamp) and gpt-oss swiglu below 256 tokens.  Activations
    silu, gelu, gpt-oss's swiglu (with its clamp) and situv2 (with both betas); an optional clamp; the route
    weight in either stage; an expert mask, with or without a count of rows received."""
    activation = _attr_name(call["activation"]) or "silu"
    if activation not in moe.ACTIVATIONS or call["gate_mode"] not in (None, "separated", "interleave"):
        return None
    act_bits = _mx_act_bits(call, activation, n_tokens)
    if act_bits is None:
        return None
    if call["gate_mode"] == "interleave" and (activation != "silu" or call["swiglu_limit"] is None):
        return None  # the reference's constraint: interleave is silu with the clamp
    if call["w1_scale"] is None or call["w2_scale"] is None:
        return None
    weights = _mx_weights_key(call, hidden, device)
    if weights is None:
        return None
    if any(call[name] is not None for name in ("a1_scale", "a2_scale", "bias1", "bias2")):
        return None
    if not isinstance(call["doweight_stage1"], bool):
        return None
    limit = call["swiglu_limit"]
    if limit is not None and not (isinstance(limit, (int, float)) and limit > 0):
        return None
    if activation == "swiglu" and limit is None:
        return None
    betas = (call["beta"], call["linear_beta"])
    if activation == "situv2":
        if not all(isinstance(b, (int, float)) and not isinstance(b, bool) and b > 0 for b in betas):
            return None
    elif any(b is not None for b in betas):
        return None
    received = call["num_local_tokens"]
    if received is not None and (call["expert_mask"] is None or not tensor_ok(received, torch.int32, 1, device) or received.numel() != 1):
        return None
    if call["out_dtype"] not in (None, BF16):
        return None
    ids, wts = call["topk_ids"], call["topk_weights"]
    if not tensor_ok(ids, torch.int32, 2, device) or not tensor_ok(wts, torch.float32, 2, device):
        return None
    if ids.shape != wts.shape or ids.shape[0] != n_tokens or not (1 <= ids.shape[1] <= 32):
        return None
    mask = call["expert_mask"]
    if mask is not None and not tensor_ok(mask, torch.int32, 1, device):
        return None
    out = call["out"]
    if out is not None and (not tensor_ok(out, BF16, 2, device) or out.shape != x.shape):
        return None
    return ("mxfp4", hidden, weights[0], weights[1], ids.shape[1], mask is not None, limit is not None, activation,
            call["doweight_stage1"], received is not None, act_bits)


def _fused_moe_key(call):
    x = call["hidden_states"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS):
        return None
    if _attr_name(call["quant_type"]) == "per_1x32":
        return _fused_moe_mx_key(call, x, device, n_tokens, hidden)
    if _attr_name(call["quant_type"]) != "per_128x128" or _attr_name(call["activation"]) not in ("silu", None):
        return None
    if call["w1_scale"] is None or call["w2_scale"] is None:
        return None
    weights = _fp8_weights_key(call, hidden, device)
    if weights is None:
        return None
    unsupported = ("a1_scale", "a2_scale", "bias1", "bias2", "swiglu_limit", "beta", "linear_beta", "num_local_tokens")
    if any(call[name] is not None for name in unsupported) or call["doweight_stage1"]:
        return None
    if call["gate_mode"] not in (None, "separated") or call["out_dtype"] not in (None, BF16):
        return None
    ids, wts = call["topk_ids"], call["topk_weights"]
    if not tensor_ok(ids, torch.int32, 2, device) or not tensor_ok(wts, torch.float32, 2, device):
        return None
    if ids.shape != wts.shape or ids.shape[0] != n_tokens or not (1 <= ids.shape[1] <= 32):
        return None
    mask = call["expert_mask"]
    global_experts = weights[0]
    if mask is not None:
        if not tensor_ok(mask, torch.int32, 1, device):
            return None
        global_experts = mask.shape[0]
    out = call["out"]
    if out is not None:
        if not tensor_ok(out, BF16, 2, device) or out.shape != x.shape:
            return None
        if any(isinstance(v, torch.Tensor) and overlaps(out, v) for k, v in call.items() if k != "out"):
            return None
    return (_layout(call), hidden, weights[0], weights[1], ids.shape[1], global_experts, mask is not None)


def _fused_moe_alloc(call, key):
    return call["out"] if call["out"] is not None else torch.empty_like(call["hidden_states"])


def _fused_moe_run(call, out):
    mask = call["expert_mask"]
    expert_map = None
    if mask is not None:  # a global id to its slot in w1, -1 off this rank (fused_moe/reference.py:78-84)
        expert_map = torch.where(mask == 1, torch.cumsum(mask, 0, dtype=torch.int32) - 1, -1).to(torch.int32)
    if _attr_name(call["quant_type"]) == "per_1x32":
        moe.fused_experts_mxfp4(
            call["hidden_states"],
            call["topk_ids"],
            call["topk_weights"],
            call["w1"].view(torch.uint8),
            call["w1_scale"].view(torch.uint8),
            call["w2"].view(torch.uint8),
            call["w2_scale"].view(torch.uint8),
            expert_map=expert_map,
            swiglu_limit=call["swiglu_limit"],
            out=out,
            activation=_attr_name(call["activation"]) or "silu",
            weight_in_stage1=call["doweight_stage1"],
            beta=call["beta"],
            linear_beta=call["linear_beta"],
            num_local_tokens=call["num_local_tokens"],
            act_bits=_mx_act_bits(call, _attr_name(call["activation"]) or "silu", call["hidden_states"].shape[0]),
        )
        return
    moe.fused_experts_fp8(
        call["hidden_states"],
        call["topk_ids"],
        call["topk_weights"],
        call["w1"],
        call["w1_scale"],
        call["w2"],
        call["w2_scale"],
        expert_map=expert_map,
        out=out,
    )


FUSED_MOE = OpContract(
    contract_id="fused_moe@1.0",
    description="Each token through its top-k experts given the routing, weighted, summed (FP8 128 x 128 experts).",
    params=[
        Param("hidden_states"),
        Param("w1"),
        Param("w2"),
        Param("topk_weights"),
        Param("topk_ids"),
        Param("expert_mask", None),
        Param("activation", None),
        Param("quant_type", None),
        Param("doweight_stage1", False),
        Param("w1_scale", None),
        Param("w2_scale", None),
        Param("a1_scale", None),
        Param("a2_scale", None),
        Param("bias1", None),
        Param("bias2", None),
        Param("swiglu_limit", None),
        Param("beta", None),
        Param("linear_beta", None),
        Param("gate_mode", None),
        Param("out_dtype", None),
        Param("num_local_tokens", None),
        Param("act_quant", 4),
        Param("out", None),
    ],
    outputs=["out"],
    key=_fused_moe_key,
    alloc=_fused_moe_alloc,
    run=_fused_moe_run,
)


@api(FUSED_MOE)
def fused_moe(
    hidden_states,
    w1,
    w2,
    topk_weights,
    topk_ids,
    expert_mask=None,
    activation=None,
    quant_type=None,
    doweight_stage1=False,
    w1_scale=None,
    w2_scale=None,
    a1_scale=None,
    a2_scale=None,
    bias1=None,
    bias2=None,
    swiglu_limit=None,
    beta=None,
    linear_beta=None,
    gate_mode=None,
    out_dtype=None,
    num_local_tokens=None,
    act_quant=4,
    out=None,
): ...


# --------------------------------------------------------------------------------------------------
# mega_moe@1.0 -- expert parallel MXFP4 MoE given routing (aklr/ops/mega_moe/contract.py:42-151):
# every rank of the group calls once per step; global expert e is local e % n_local of rank
# e // n_local; MXFP8 activations, clamped SwiGLU, weighted sum back on the token's rank.
# --------------------------------------------------------------------------------------------------
def _mega_moe_key(call):
    x = call["hidden_states"]
    if not tensor_ok(x, BF16, 2):
        return None
    device = x.device
    n_tokens, hidden = x.shape
    if not (1 <= n_tokens <= MAX_TOKENS) or call["w1_scale"] is None or call["w2_scale"] is None:
        return None
    weights = _mx_weights_key(call, hidden, device)
    if weights is None:
        return None
    ids, wts = call["topk_ids"], call["topk_weights"]
    if not tensor_ok(ids, torch.int32, 2, device) or not tensor_ok(wts, torch.float32, 2, device) or ids.shape != wts.shape:
        return None
    if ids.shape[0] != n_tokens or not (1 <= ids.shape[1] <= 32):
        return None
    ep_size, limit = call["ep_size"], call["swiglu_limit"]
    if not isinstance(ep_size, int) or ep_size < 1 or not isinstance(limit, (int, float)) or limit <= 0:
        return None
    if call["out_dtype"] not in (None, BF16):
        return None
    import torch.distributed as dist

    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if world != ep_size:
        return None
    return (hidden, weights[0], weights[1], ids.shape[1], ep_size)


# one layer object per (weight tensors, group size, top-k, clamp): building it is host work only, but
# it holds the side stream and the views of the weights, which a serving loop reuses every step
_MEGA_MOE_LAYERS: dict = {}


def _mega_moe_layer(call):
    import torch.distributed as dist

    from aklr_b200.ep import CudaKernels, ExpertParallelMoE

    ep_size, topk, limit = call["ep_size"], call["topk_ids"].shape[1], float(call["swiglu_limit"])
    tensors = (call["w1"], call["w1_scale"], call["w2"], call["w2_scale"])
    key = tuple((t.data_ptr(), tuple(t.shape)) for t in tensors) + (ep_size, topk, limit)
    layer = _MEGA_MOE_LAYERS.get(key)
    if layer is None:
        if len(_MEGA_MOE_LAYERS) >= 64:  # weights are long-lived; a churn of keys means the caller rebuilt them
            _MEGA_MOE_LAYERS.clear()
        rank = dist.get_rank() if ep_size > 1 else 0
        layer = _MEGA_MOE_LAYERS[key] = ExpertParallelMoE(
            moe.Routing(topk=topk), *(t.view(torch.uint8) for t in tensors), rank, ep_size, kernels=CudaKernels("mxfp4", limit)
        )
    return layer


def _mega_moe_run(call, out):
    ep_size = call["ep_size"]
    layer = _mega_moe_layer(call)
    routed = (call["topk_ids"], call["topk_weights"])
    if ep_size == 1:
        from aklr_b200.ep import run_in_process

        result = run_in_process([layer], [(call["hidden_states"], None, None, routed)])[0]
    else:
        result = layer.forward(call["hidden_states"], None, None, routed=routed)
    out.copy_(result)


MEGA_MOE = OpContract(
    contract_id="mega_moe@1.0",
    description="Expert-parallel MXFP4 MoE given the routing: each rank's tokens through experts held anywhere in the group.",
    params=[
        Param("hidden_states"),
        Param("w1"),
        Param("w2"),
        Param("topk_weights"),
        Param("topk_ids"),
        Param("w1_scale", None),
        Param("w2_scale", None),
        Param("ep_size", 1),
        Param("swiglu_limit", 10.0),
        Param("out_dtype", None),
    ],
    outputs=["out"],
    key=_mega_moe_key,
    alloc=_layer_alloc,
    run=_mega_moe_run,
    ranks="ep_size",
    capturable=False,  # the uneven all-to-all takes its split sizes on the host
)


@api(MEGA_MOE)
def mega_moe(
    hidden_states,
    w1,
    w2,
    topk_weights,
    topk_ids,
    w1_scale=None,
    w2_scale=None,
    ep_size=1,
    swiglu_limit=10.0,
    out_dtype=None,
): ...


# --------------------------------------------------------------------------------------------------
# biased_grouped_topk@1.0 (aklr/ops/topk/contract.py:36-109); group dropping is also served
# --------------------------------------------------------------------------------------------------
def _topk_key(call):
    logits, bias = call["router_logits"], call["correction_bias"]
    if not tensor_ok(logits, (BF16, torch.float32), 2):
        return None
    device = logits.device
    n_tokens, n_experts = logits.shape
    if not (1 <= n_tokens <= MAX_TOKENS and 1 <= n_experts <= 1024):
        return None
    if not tensor_ok(bias, (BF16, torch.float32), 1, device) or bias.shape[0] != n_experts:
        return None
    wts, ids = call["topk_weights"], call["topk_ids"]
    if not tensor_ok(wts, torch.float32, 2, device) or not tensor_ok(ids, torch.int32, 2, device):
        return None
    if wts.shape != ids.shape or wts.shape[0] != n_tokens or not (1 <= wts.shape[1] <= 32):
        return None
    if overlaps(wts, logits) or overlaps(ids, logits) or overlaps(wts, ids):
        return None
    groups, topk_group, topk = call["num_expert_group"], call["topk_group"], wts.shape[1]
    if not (isinstance(groups, int) and isinstance(topk_group, int) and isinstance(call["renormalize"], bool)):
        return None
    if groups < 1 or groups > 32 or n_experts % groups or not (1 <= topk_group <= groups):
        return None
    if groups > 1 and topk_group < groups and n_experts // groups < 2:
        return None
    if topk > topk_group * (n_experts // groups):
        return None
    factor = call["routed_scaling_factor"]
    if not isinstance(factor, (int, float)) or not math.isfinite(factor):
        return None
    return (str(logits.dtype), str(bias.dtype), n_experts, topk, groups, topk_group, call["renormalize"])


def _topk_alloc(call, key):
    return call["topk_weights"], call["topk_ids"]


def _topk_run(call, outputs):
    routing = moe.Routing(
        topk=call["topk_weights"].shape[1],
        scoring="sigmoid",
        num_expert_group=call["num_expert_group"],
        topk_group=call["topk_group"],
        renormalize=call["renormalize"],
        routed_scaling_factor=float(call["routed_scaling_factor"]),
    )
    moe.route(call["router_logits"], call["correction_bias"], routing, call["topk_ids"], call["topk_weights"])


BIASED_GROUPED_TOPK = OpContract(
    contract_id="biased_grouped_topk@1.0",
    description="Each token's top-k experts by sigmoid score + bias (ties to the lower expert), weighted by the unbiased scores.",
    params=[
        Param("router_logits"),
        Param("correction_bias"),
        Param("topk_weights"),
        Param("topk_ids"),
        Param("num_expert_group"),
        Param("topk_group"),
        Param("renormalize"),
        Param("routed_scaling_factor", 1.0),
    ],
    outputs=["topk_weights", "topk_ids"],
    key=_topk_key,
    alloc=_topk_alloc,
    run=_topk_run,
)


@api(BIASED_GROUPED_TOPK)
def biased_grouped_topk(
    router_logits,
    correction_bias,
    topk_weights,
    topk_ids,
    num_expert_group,
    topk_group,
    renormalize,
    routed_scaling_factor=1.0,
): ...


# --------------------------------------------------------------------------------------------------
# per_group_quant_fp8@1.0 / per_group_quant_mxfp8@1.0 (aklr/ops/quant/contract.py:17-76)
# --------------------------------------------------------------------------------------------------
def _quant_key(group: int, max_hidden: int):
    def key(call):
        x = call["x"]
        if not tensor_ok(x, BF16, 2):
            return None
        rows, hidden = x.shape
        if not (1 <= rows <= 131072) or hidden % group or not (group <= hidden <= max_hidden):
            return None
        return (hidden,)

    return key


def _quant_fp8_alloc(call, key):
    x = call["x"]
    rows, hidden = x.shape
    return (
        torch.empty((rows, hidden), dtype=FP8, device=x.device),
        torch.empty((hidden // 128, rows), dtype=torch.float32, device=x.device),
    )


def _quant_mxfp8_alloc(call, key):
    x = call["x"]
    rows, hidden = x.shape
    return (
        torch.empty((rows, hidden), dtype=FP8, device=x.device),
        torch.empty((rows, hidden // 32), dtype=torch.uint8, device=x.device),
    )


PER_GROUP_QUANT_FP8 = OpContract(
    contract_id="per_group_quant_fp8@1.0",
    description="Groups of 128 bf16 values to e4m3 with group-major float32 scales amax*(1/448).",
    params=[Param("x")],
    outputs=["quantized", "scales"],
    key=_quant_key(128, 21504),
    alloc=_quant_fp8_alloc,
    run=lambda call, outs: moe.per_group_quant_fp8(call["x"], outs[0], outs[1]),
)

PER_GROUP_QUANT_MXFP8 = OpContract(
    contract_id="per_group_quant_mxfp8@1.0",
    description="Groups of 32 bf16 values to e4m3 with row-major e8m0 scales rounded up to a power of two.",
    params=[Param("x")],
    outputs=["quantized", "scales"],
    key=_quant_key(32, 21504),
    alloc=_quant_mxfp8_alloc,
    run=lambda call, outs: moe.per_group_quant_mxfp8(call["x"], outs[0], outs[1]),
)


@api(PER_GROUP_QUANT_FP8)
def per_group_quant_fp8(x): ...


@api(PER_GROUP_QUANT_MXFP8)
def per_group_quant_mxfp8(x): ...


CONTRACTS = (
    DEEPSEEK_V2_FP8_MOE,
    DEEPSEEK_V2_MXFP4_MOE,
    QWEN3_MOE_FP8_MOE,
    MINIMAX_M2_FP8_MOE,
    MINIMAX_M2_MXFP4_MOE,
    QWEN2_MOE_ROUTER,
    QWEN2_MOE_FP8_EXPERTS,
    QWEN2_MOE_FP8_ROUTER_EXPERTS,
    QWEN2_MOE_MXFP4_MOE,
    FUSED_MOE,
    MEGA_MOE,
    BIASED_GROUPED_TOPK,
    PER_GROUP_QUANT_FP8,
    PER_GROUP_QUANT_MXFP8,
)
