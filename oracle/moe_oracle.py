"""CPU oracle for the fused-MoE path: TEST INFRASTRUCTURE, never a product path.

A plain-torch (CPU, float32) restatement of the reference library's arithmetic for the
fused Mixture-of-Experts layer.  Only tests, the smoke check and the benchmark's CPU
baseline leg may import this module; the product (``aklr_b200``) never does.

Each function names the reference function it restates (paths relative to the reference
project root).  Parity status: PINNED -- ``tests/golden/`` holds outputs of the
reference's own functions on seeded inputs (written by ``tests/golden/make_golden.py``
in a container that has the reference), and ``tests/test_oracle.py`` checks this file
against them bit for bit, plus the reference's known-answer tests.

Conventions
-----------
* every tensor is float32 unless said otherwise; FP8 codes are ``torch.float8_e4m3fn``
* w1 is ``[experts, 2*inter, hidden]`` with gate rows first, then up rows
* block scales are one float32 per 128 x 128 block of a weight; activations are
  quantised per 1 x 128 group at scale ``amax / 448``
"""

from __future__ import annotations

import math

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
BLOCK = 128
MX_BLOCK = 32
E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


# --------------------------------------------------------------------------------------
# dtype decoding -- aklr/core/contract/semantics/_dtypes.py:88-115
# --------------------------------------------------------------------------------------
def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """float32 values at their nearest bfloat16 (ties to even), kept in float32.
    Follows ``rounded_to_bfloat16`` (_dtypes.py:113)."""
    return x.to(torch.bfloat16).to(torch.float32)


def decode_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """Two 4-bit e2m1 codes per byte, low nibble first; doubles the last dim.
    Follows ``to_float32`` nibble_table branch (_dtypes.py:97-101)."""
    codes = packed.view(torch.uint8).long()
    table = torch.tensor(E2M1_GRID + tuple(-v for v in E2M1_GRID), dtype=torch.float32)
    return table[torch.stack((codes & 0xF, codes >> 4), dim=-1).flatten(-2)]


def decode_e8m0(codes: torch.Tensor) -> torch.Tensor:
    """2^(byte-127); byte 255 is NaN.  Follows ``to_float32`` power_of_two branch
    (_dtypes.py:102-109)."""
    raw = codes.view(torch.uint8)
    return torch.exp2(raw.to(torch.float32) - 127.0).masked_fill(raw == 255, math.nan)


# --------------------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------------------
def router_logits(hidden: torch.Tensor, router_weight: torch.Tensor) -> torch.Tensor:
    """bf16-rounded ``hidden @ router_weight^T`` in float32.
    Follows ``_router_logits`` (aklr/plugins/sglang/models/qwen3_moe/reference.py:24-31)."""
    return bf16_round(hidden.float() @ router_weight.float().T)


def first_largest(values: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest per row, lower index first among equals.
    Follows ``_first_largest`` (aklr/plugins/sglang/models/deepseek_v2/reference.py:114-118)."""
    return torch.sort(values, dim=-1, descending=True, stable=True).indices[..., :k]


def softmax_topk(logits: torch.Tensor, topk: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(ids int64 [T,K], weights f32 [T,K]): top-k by logit, softmax over the chosen logits.
    Follows ``_routed`` (aklr/plugins/sglang/models/qwen3_moe/reference.py:34-41)."""
    ids = first_largest(logits, topk)
    return ids, logits.gather(-1, ids).softmax(dim=-1)


def grouped_sigmoid_topk(
    logits: torch.Tensor,
    bias: torch.Tensor,
    topk: int,
    num_expert_group: int,
    topk_group: int,
    renormalize: bool,
    routed_scaling_factor: float,
) -> tuple[torch.Tensor, torch.Tensor]:
    """(ids, weights): sigmoid scores + bias rank the experts inside the ``topk_group`` best
    groups (a group scores the sum of its two best biased scores); the weights are the
    unbiased scores, renormalised and scaled.
    Follows ``_grouped_routed`` (aklr/plugins/sglang/models/deepseek_v2/reference.py:121-143)."""
    scores = logits.sigmoid()
    biased = scores + bias
    groups = biased.unflatten(-1, (num_expert_group, -1))
    group_scores = groups.topk(2, dim=-1).values.sum(dim=-1)
    kept = torch.zeros_like(group_scores, dtype=torch.bool)
    kept.scatter_(-1, first_largest(group_scores, topk_group), True)
    allowed = kept.repeat_interleave(groups.shape[-1], dim=-1)
    ids = first_largest(biased.masked_fill(~allowed, float("-inf")), topk)
    weights = scores.gather(-1, ids)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return ids, weights * routed_scaling_factor


def with_shared_slot(ids: torch.Tensor, weights: torch.Tensor, n_routed: int):
    """Append the shared expert (id ``n_routed``) at weight 1 as the last slot.
    Follows ``_with_shared_slot`` (aklr/plugins/sglang/models/deepseek_v2/reference.py:80-88)."""
    shared = torch.full_like(ids[:, :1], n_routed)
    return (
        torch.cat([ids, shared], dim=-1),
        torch.cat([weights, torch.ones_like(weights[:, :1])], dim=-1),
    )


def biased_grouped_topk(
    logits: torch.Tensor,
    bias: torch.Tensor,
    topk: int,
    renormalize: bool,
    routed_scaling_factor: float = 1.0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """(weights f32, ids int32) of the standalone routing op: every group kept.
    Follows ``biased_grouped_topk_reference`` (aklr/ops/topk/reference.py:17-35)."""
    scores = logits.float().sigmoid()
    chosen = first_largest(scores + bias.float(), topk)
    weights = scores.gather(-1, chosen)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights * routed_scaling_factor, chosen.to(torch.int32)


def moe_align(ids: torch.Tensor, n_experts: int, block_m: int):
    """Canonical token sort.  The reference defines no order (its kernels sort with atomics),
    so this build fixes one: routes ``token*K + slot`` sorted stably by expert id, each
    expert's run padded with -1 to a multiple of ``block_m``.

    Returns (sorted_route_ids int32 [capacity_used], expert_of_block int32 [blocks],
    counts int64 [n_experts]).  Negative ids (routes to experts this rank does not hold) are
    dropped.  Shapes the reference kernels produce the same way:
    deepseek_v2 ``_scatter_and_describe`` (kernel JSON e5adae63cb11d836, kernel.py:305-361)."""
    flat = ids.reshape(-1).long()
    keep = flat >= 0
    routes = torch.arange(flat.numel())[keep]
    experts = flat[keep]
    order = torch.sort(experts, stable=True).indices
    routes, experts = routes[order], experts[order]
    counts = torch.bincount(experts, minlength=n_experts)
    sorted_ids: list[int] = []
    block_expert: list[int] = []
    start = 0
    for e in range(n_experts):
        c = int(counts[e])
        if c == 0:
            continue
        run = routes[start : start + c].tolist()
        start += c
        pad = (-c) % block_m
        sorted_ids.extend(run + [-1] * pad)
        block_expert.extend([e] * ((c + pad) // block_m))
    return (
        torch.tensor(sorted_ids, dtype=torch.int32),
        torch.tensor(block_expert, dtype=torch.int32),
        counts,
    )


# --------------------------------------------------------------------------------------
# FP8 quantisation
# --------------------------------------------------------------------------------------
def fp8_group_quant(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(codes e4m3 [.., H], scales f32 [.., H/128]) of the MoE layer's activation scheme:
    round to bf16, per 1 x 128 group scale = max(amax/448, FLT_MIN), code = e4m3(x / scale).
    Follows ``_fp8_input`` (aklr/plugins/sglang/models/qwen3_moe/reference.py:44-54) and the
    first half of ``_fp8_linear`` (aklr/plugins/sglang/models/deepseek_v2/reference.py:156-159)."""
    groups = bf16_round(x.float()).unflatten(-1, (-1, BLOCK))
    scale = groups.abs().amax(-1, keepdim=True) / FP8_MAX
    scale = scale.clamp(min=torch.finfo(torch.float32).tiny)
    codes = (groups / scale).to(FP8)
    return codes.flatten(-2), scale.squeeze(-1)


def fp8_input(x: torch.Tensor) -> torch.Tensor:
    """``x`` as an FP8 expert linear takes it: quantised per 1 x 128, dequantised (float32)."""
    codes, scale = fp8_group_quant(x)
    return (codes.float().unflatten(-1, (-1, BLOCK)) * scale.unsqueeze(-1)).flatten(-2)


def per_group_quant_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Standalone quant op: (decoded codes f32 [T,H], scales f32 [H/128, T] group-major).
    scale = max(amax,1e-10) * (1/448), code = e4m3(clamp(x * (1/scale), +-448)).
    Follows ``per_group_quant_fp8_reference`` (aklr/ops/quant/reference.py:9-28)."""
    x = x.float()
    rows, cols = x.shape
    grouped = x.reshape(rows, cols // BLOCK, BLOCK)
    amax = grouped.abs().amax(-1).clamp_min(1e-10)
    scales = amax * (1.0 / FP8_MAX)
    recip = 1.0 / scales
    values = (grouped * recip.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX)
    return values.to(FP8).float().reshape(rows, cols), scales.t().contiguous()


def per_group_quant_mxfp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Standalone MXFP8 quant op: (decoded codes f32 [T,H], e8m0 exponent bytes [T,H/32]).
    The scale is the smallest power of two >= max(amax,1e-10)/448.
    Follows ``per_group_quant_mxfp8_reference`` (aklr/ops/quant/reference.py:31-48)."""
    x = x.float()
    rows, cols = x.shape
    grouped = x.reshape(rows, cols // MX_BLOCK, MX_BLOCK)
    amax = grouped.abs().amax(-1).clamp_min(1e-10)
    raw = (amax * (1.0 / FP8_MAX)).contiguous().view(torch.int32)
    exponent = (raw >> 23) + ((raw & 0x7FFFFF) != 0).to(torch.int32)
    scale = (exponent << 23).contiguous().view(torch.float32)
    values = (grouped / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX)
    return values.to(FP8).float().reshape(rows, cols), exponent.to(torch.uint8)


def dequant_block_weight(weight: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """An e4m3 weight [rows, cols] decoded, times its scale per 128 x 128 block.
    Follows ``_dequantized`` (aklr/plugins/sglang/models/qwen3_moe/reference.py:57-61)."""
    rows, cols = weight.shape
    blocks = scale.float().repeat_interleave(BLOCK, 0)[:rows].repeat_interleave(BLOCK, 1)
    return weight.float() * blocks[:, :cols]


# --------------------------------------------------------------------------------------
# FP8 fused MoE layers
# --------------------------------------------------------------------------------------
def fp8_experts(
    x: torch.Tensor,
    ids: torch.Tensor,
    weights: torch.Tensor,
    w1: torch.Tensor,
    w1_scale: torch.Tensor,
    w2: torch.Tensor,
    w2_scale: torch.Tensor,
) -> torch.Tensor:
    """sum_k weight * down(fp8(silu(gate(fp8(x))) * up(fp8(x)))) per token, experts visited in
    ascending id order, float32 accumulation with index_add.  Negative ids add nothing.
    Follows the expert loop of ``qwen3_moe_fp8_moe_reference``
    (aklr/plugins/sglang/models/qwen3_moe/reference.py:77-88) and ``_experts`` + ``mlp``
    (aklr/plugins/sglang/models/deepseek_v2/reference.py:64-77,177-183)."""
    x = x.float()
    xq = fp8_input(x)
    out = torch.zeros_like(x)
    for e in ids.unique().tolist():
        if e < 0:
            continue
        tokens, slots = (ids == e).nonzero(as_tuple=True)
        wa = dequant_block_weight(w1[e], w1_scale[e])
        wb = dequant_block_weight(w2[e], w2_scale[e])
        gate, up = (xq[tokens] @ wa.T).chunk(2, dim=-1)
        y = fp8_input(torch.nn.functional.silu(gate) * up) @ wb.T
        out.index_add_(0, tokens, weights[tokens, slots, None] * y)
    return out


def qwen3_moe_fp8_moe(hidden, router_weight, w1, w1_scale, w2, w2_scale, topk, logits=None):
    """Softmax-routed FP8 MoE layer.  ``logits`` (bf16 values) override the router GEMM.
    Follows ``qwen3_moe_fp8_moe_reference`` (aklr/plugins/sglang/models/qwen3_moe/reference.py:64-88)."""
    if logits is None:
        logits = router_logits(hidden, router_weight)
    ids, weights = softmax_topk(logits.float(), topk)
    return fp8_experts(hidden, ids, weights, w1, w1_scale, w2, w2_scale)


def deepseek_v2_fp8_moe(
    hidden,
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
    routed_scaling_factor,
    logits=None,
):
    """Sigmoid/grouped-routed FP8 MoE layer with the shared expert in w1/w2's last slot.
    Follows ``deepseek_v2_fp8_moe_reference``
    (aklr/plugins/sglang/models/deepseek_v2/reference.py:163-183)."""
    if logits is None:
        logits = router_logits(hidden, router_weight)
    n_routed = logits.shape[-1]
    ids, weights = grouped_sigmoid_topk(
        logits.float(),
        correction_bias.float(),
        topk,
        num_expert_group,
        topk_group,
        renormalize,
        routed_scaling_factor,
    )
    ids, weights = with_shared_slot(ids, weights, n_routed)
    return fp8_experts(hidden, ids, weights, w1, w1_scale, w2, w2_scale)


def with_gated_shared_slot(hidden, shared_gate_weight, ids, weights, shared_slot: int):
    """Append the shared expert ``shared_slot`` weighed by sigmoid(hidden . shared_gate_weight[0]).
    Follows the head of ``_experts`` (aklr/plugins/sglang/models/qwen2_moe/reference.py:84-90)."""
    shared_weight = (hidden.float() @ shared_gate_weight.float()[0]).sigmoid()
    ids = torch.cat([ids, torch.full_like(ids[:, :1], shared_slot)], dim=-1)
    return ids, torch.cat([weights, shared_weight[:, None]], dim=-1)


def qwen2_moe_fp8_experts(hidden, topk_weights, topk_ids, shared_gate_weight, w1, w1_scale, w2, w2_scale):
    """Routed experts at the given routing plus the gated shared expert in w1/w2's last slot.
    Follows ``qwen2_moe_fp8_experts_reference`` (aklr/plugins/sglang/models/qwen2_moe/reference.py:135-143)."""
    ids, weights = with_gated_shared_slot(hidden, shared_gate_weight, topk_ids.long(), topk_weights.float(), w1.shape[0] - 1)
    return fp8_experts(hidden, ids, weights, w1, w1_scale, w2, w2_scale)


def qwen2_moe_fp8_router_experts(hidden, router_weight, shared_gate_weight, w1, w1_scale, w2, w2_scale, topk, logits=None):
    """bf16 router logits, softmax top-k, routed experts and the gated shared one.
    Follows ``qwen2_moe_fp8_router_experts_reference`` (aklr/plugins/sglang/models/qwen2_moe/reference.py:146-155)."""
    if logits is None:
        logits = router_logits(hidden, router_weight)
    ids, weights = softmax_topk(logits.float(), topk)
    return qwen2_moe_fp8_experts(hidden, weights, ids, shared_gate_weight, w1, w1_scale, w2, w2_scale)


def sigmoid_bias_topk(logits: torch.Tensor, bias: torch.Tensor, topk: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(ids, weights): the ``topk`` experts by sigmoid score + bias (ties to the lower id), weighed by
    their unbiased scores renormalised to sum 1.
    Follows ``_routed`` (aklr/plugins/sglang/models/minimax_m2/reference.py:43-50)."""
    scores = logits.sigmoid()
    ids = first_largest(scores + bias, topk)
    weights = scores.gather(-1, ids)
    return ids, weights / weights.sum(dim=-1, keepdim=True)


def minimax_m2_fp8_moe(hidden, router_weight, correction_bias, w1, w1_scale, w2, w2_scale, topk, expert_offset=0, logits=None):
    """This rank's share of a MiniMax-M2 FP8 MoE: float32 gate (nothing rounded), biased sigmoid
    top-k, the experts ``expert_offset .. expert_offset + len(w1) - 1`` held here; routes to the others
    add nothing.  Follows ``minimax_m2_fp8_moe_reference`` and ``_held_experts``
    (aklr/plugins/sglang/models/minimax_m2/reference.py:53-70,103-117)."""
    if logits is None:
        logits = hidden.float() @ router_weight.float().T
    ids, weights = sigmoid_bias_topk(logits.float(), correction_bias.float(), topk)
    local = ids - expert_offset
    local = torch.where((local >= 0) & (local < w1.shape[0]), local, torch.full_like(local, -1))
    return fp8_experts(hidden, local, weights, w1, w1_scale, w2, w2_scale)


# --------------------------------------------------------------------------------------
# MX formats (weights e2m1 + e8m0 per 32, activations MXFP8 e4m3 + power-of-two scale per 32)
# --------------------------------------------------------------------------------------
def mxfp8_input(x: torch.Tensor) -> torch.Tensor:
    """``x`` quantised to e4m3 per 1 x 32 at the smallest power-of-two scale >= amax/448,
    dequantised.  Follows ``_mxfp8`` (aklr/ops/fused_moe/reference.py:40-51)."""
    blocks = x.unflatten(-1, (-1, MX_BLOCK))
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    finite = amax.isfinite()
    mantissa, exponent = torch.frexp(torch.where(finite, amax, 0.0) / FP8_MAX)
    exponent = (exponent - 1 + (mantissa != 0.5).int()).clamp(-126, 127)
    scale = torch.where(finite, torch.exp2(exponent.to(x.dtype)), float("nan"))
    scaled = torch.where(finite, blocks, 0.0) / scale
    return (scaled.to(FP8).to(x.dtype) * scale).flatten(-2)


def mxfp4_input(x: torch.Tensor) -> torch.Tensor:
    """``x`` quantised to e2m1 per 1 x 32 (amax/scale in (3,6]), ties to the even code,
    dequantised.  Follows ``_mxfp4`` (aklr/ops/fused_moe/reference.py:21-37)."""
    grid = torch.tensor(E2M1_GRID, dtype=x.dtype)
    blocks = x.unflatten(-1, (-1, MX_BLOCK))
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    finite = amax.isfinite()
    mantissa, exponent = torch.frexp(torch.where(finite, amax, 0.0).clamp_min(1e-10))
    exponent = (exponent - 3 + (mantissa > 0.75).int()).clamp(-127, 127)
    scale = torch.where(finite, torch.exp2(exponent.to(x.dtype)), float("nan"))
    scaled = torch.where(finite, blocks, 0.0) / scale
    m = scaled.abs()
    lo = torch.bucketize(m, grid, right=True) - 1
    hi = (lo + 1).clamp_max(len(grid) - 1)
    below, above = m - grid[lo], grid[hi] - m
    up = (above < below) | ((above == below) & (hi % 2 == 0))
    codes = torch.where(up, grid[hi], grid[lo]) * scaled.sign()
    return (codes * scale).flatten(-2)


def mx_weight(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e2m1 weight [rows, cols/2 bytes] times its e8m0 scale per 32 along the row.
    Follows ``_weight`` (aklr/ops/fused_moe/reference.py:54-61)."""
    return decode_e2m1(w) * decode_e8m0(scale).repeat_interleave(MX_BLOCK, dim=-1)


def mx_experts(
    hidden: torch.Tensor,
    ids: torch.Tensor,
    weights: torch.Tensor,
    w1: torch.Tensor,
    w1_scale: torch.Tensor,
    w2: torch.Tensor,
    w2_scale: torch.Tensor,
    swiglu_limit: float | None = None,
    act_bits: int = 8,
    activation: str = "silu",
    weight_in_stage1: bool = False,
    beta: float | None = None,
    linear_beta: float | None = None,
    num_local_tokens: int | None = None,
) -> torch.Tensor:
    """MXFP4-weight experts given the routing: activations MXFP8 (act_bits 8) or MXFP4 (4) per
    1 x 32, or left as they are (16: what the reference does under gate_mode 'interleave' and for
    gpt-oss swiglu below 256 rows, aklr/ops/fused_moe/reference.py:90-93), the gated product rounded
    to bf16 before it is quantised, each route weighted,
    the routes of a token summed.  Negative ids add nothing.  ``swiglu_limit`` clamps gate
    (above) and up (both sides) before the activation when given.
    ``activation`` silu, gelu (erf), swiglu (gpt-oss: gate sigmoid(1.702 gate) (up + 1)) or situv2
    (beta tanh(gate/beta) sigmoid(gate) times linear_beta tanh(up/linear_beta)); ``weight_in_stage1``
    multiplies the gate_up projection by the route weight instead of the output; rows at or past
    ``num_local_tokens`` add nothing.
    Follows ``fused_moe_reference`` (aklr/ops/fused_moe/reference.py:64-127) and
    ``mega_moe_reference`` (aklr/ops/mega_moe/reference.py:18-48)."""
    if act_bits not in (4, 8, 16):
        raise ValueError("act_bits: 4 (MXFP4), 8 (MXFP8) or 16 (activations kept in bf16)")
    quantize = mxfp8_input if act_bits == 8 else mxfp4_input if act_bits == 4 else (lambda t: t)
    weights = weights.float()
    if num_local_tokens is not None:
        ids = ids.clone()
        ids[num_local_tokens:] = -1
    x = quantize(hidden.float())
    out = x.new_zeros((*ids.shape, x.shape[-1]))
    for e in ids.unique().tolist():
        if e < 0:
            continue
        routed = ids == e
        tokens = routed.nonzero(as_tuple=True)[0]
        projected = x[tokens] @ mx_weight(w1[e], w1_scale[e]).mT
        if weight_in_stage1:
            projected = projected * weights[routed].unsqueeze(-1)
        gate, up = projected.chunk(2, dim=-1)
        if swiglu_limit is not None:
            gate, up = gate.clamp(max=swiglu_limit), up.clamp(-swiglu_limit, swiglu_limit)
        if activation == "silu":
            gated = torch.nn.functional.silu(gate) * up
        elif activation == "gelu":
            gated = torch.nn.functional.gelu(gate) * up
        elif activation == "swiglu":
            gated = gate * torch.sigmoid(1.702 * gate) * (up + 1)
        elif activation == "situv2":
            gated = beta * torch.tanh(gate / beta) * torch.sigmoid(gate) * (linear_beta * torch.tanh(up / linear_beta))
        else:
            raise ValueError(f"activation {activation!r}")
        out[routed] = quantize(bf16_round(gated)) @ mx_weight(w2[e], w2_scale[e]).mT
    if not weight_in_stage1:
        out = out * weights.unsqueeze(-1)
    return out.sum(dim=1)


def deepseek_v2_mxfp4_moe(hidden, router_weight, correction_bias, w1, w1_scale, w2, w2_scale, topk, renormalize,
                          routed_scaling_factor, logits=None):
    """Ungrouped sigmoid routing (scores + bias pick, unbiased scores weigh), the shared expert appended at
    weight 1, MXFP4 experts on activations that are never quantised or rounded in between.
    Follows ``deepseek_v2_mxfp4_moe_reference`` with ``_routed`` and ``_mlp``
    (aklr/plugins/sglang/models/deepseek_v2/reference.py:41-62, 91-111)."""
    x = hidden.float()
    if logits is None:
        logits = router_logits(hidden, router_weight)
    scores = logits.sigmoid()
    ids = first_largest(scores + correction_bias.float(), topk)
    weights = scores.gather(-1, ids)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    ids, weights = with_shared_slot(ids, weights * routed_scaling_factor, logits.shape[-1])
    return mx_experts_unquantised(x, ids, weights, w1, w1_scale, w2, w2_scale)


def mx_experts_unquantised(x, ids, weights, w1, w1_scale, w2, w2_scale):
    """MXFP4 experts on float32 activations, nothing rounded: the experts hit in ascending order, each one's rows
    weighed and added in float32 (``index_add_``), ids below 0 adding nothing -- the loop the three layer
    references share (``_experts``, aklr/plugins/sglang/models/deepseek_v2/reference.py:91-111; ``_held_experts``,
    aklr/plugins/sglang/models/minimax_m2/reference.py:53-70; aklr/plugins/sglang/models/qwen2_moe/reference.py:179-183)."""
    out = torch.zeros_like(x)
    for e in ids.unique().tolist():
        if e < 0:
            continue
        tokens, slots = (ids == e).nonzero(as_tuple=True)
        gate, up = (x[tokens] @ mx_weight(w1[e], w1_scale[e]).T).chunk(2, dim=-1)
        y = (torch.nn.functional.silu(gate) * up) @ mx_weight(w2[e], w2_scale[e]).T
        out.index_add_(0, tokens, weights[tokens, slots, None] * y)
    return out


def minimax_m2_mxfp4_moe(hidden, router_weight, correction_bias, w1, w1_scale, w2, w2_scale, topk, expert_offset=0, logits=None):
    """This rank's share of a MiniMax-M2 MoE over MXFP4 experts: float32 gate, biased sigmoid top-k, unquantised
    activations.  Follows ``minimax_m2_mxfp4_moe_reference`` (aklr/plugins/sglang/models/minimax_m2/reference.py:114-132)."""
    x = hidden.float()
    if logits is None:
        logits = x @ router_weight.float().T
    ids, weights = sigmoid_bias_topk(logits.float(), correction_bias.float(), topk)
    local = ids - expert_offset
    local = torch.where((local >= 0) & (local < w1.shape[0]), local, torch.full_like(local, -1))
    return mx_experts_unquantised(x, local, weights, w1, w1_scale, w2, w2_scale)


def qwen2_moe_mxfp4_moe(hidden, router_weight, w1, w1_scale, w2, w2_scale, shared_w1, shared_w2, shared_gate_weight, topk,
                        logits=None):
    """bf16 router logits, softmax top-k, MXFP4 routed experts on unquantised activations, plus the bf16 shared
    expert weighed by sigmoid(hidden . shared_gate_weight[0]).  Follows ``qwen2_moe_mxfp4_moe_reference`` and
    ``_silu_mlp`` (aklr/plugins/sglang/models/qwen2_moe/reference.py:152-185)."""
    x = hidden.float()
    if logits is None:
        logits = router_logits(hidden, router_weight)
    ids, weights = softmax_topk(logits.float(), topk)
    out = mx_experts_unquantised(x, ids, weights, w1, w1_scale, w2, w2_scale)
    shared_weight = (x @ shared_gate_weight.float()[0]).sigmoid()
    gate, up = (x @ shared_w1.float().T).chunk(2, dim=-1)
    return out + shared_weight[:, None] * ((torch.nn.functional.silu(gate) * up) @ shared_w2.float().T)


# --------------------------------------------------------------------------------------
# comparison measures
# --------------------------------------------------------------------------------------
def sqnr_db(actual: torch.Tensor, reference: torch.Tensor) -> float:
    """20 log10(||ref|| / ||actual - ref||) over the whole output, the reference rounded to
    the output dtype by the caller.  Follows ``SqnrBound.compare``
    (aklr/core/contract/semantics/_compare.py:424-466)."""
    a, r = actual.double().flatten(), reference.double().flatten()
    noise = torch.linalg.vector_norm(a - r).item()
    if noise == 0.0:
        return math.inf
    signal = torch.linalg.vector_norm(r).item()
    return 20.0 * math.log10(signal / noise) if signal else -math.inf


def cosine(actual: torch.Tensor, reference: torch.Tensor) -> float:
    a, r = actual.double().flatten(), reference.double().flatten()
    return float((a @ r) / (torch.linalg.vector_norm(a) * torch.linalg.vector_norm(r)).clamp_min(1e-300))


def max_rel_err(actual: torch.Tensor, reference: torch.Tensor) -> float:
    """max |actual-ref| / max|ref| taken per row (a token's output), the largest row's value."""
    a, r = actual.double(), reference.double()
    scale = r.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((a - r).abs() / scale).max())


def output_gates(actual: torch.Tensor, reference_f32: torch.Tensor) -> dict:
    """The three float gates of the layer output against the float32 oracle, which is first
    rounded to bf16 (the output dtype) as the reference's compare does."""
    ref = bf16_round(reference_f32)
    act = actual.float()
    return {
        "max_rel_err": max_rel_err(act, ref),
        "cosine": cosine(act, ref),
        "sqnr_db": sqnr_db(act, ref),
    }


def gates_pass(g: dict, min_sqnr_db: float = 30.0) -> bool:
    return g["max_rel_err"] <= 2e-2 and g["cosine"] >= 0.9995 and g["sqnr_db"] >= min_sqnr_db


def sha256_of(t: torch.Tensor) -> str:
    import hashlib

    raw = t.contiguous().view(torch.uint8) if t.dtype != torch.bool else t.to(torch.uint8)
    return hashlib.sha256(np.ascontiguousarray(raw.numpy()).tobytes()).hexdigest()
