"""Qwen2-MoE on sglang: ``Qwen2MoeSparseMoeBlock._forward_router_experts`` served by the three Qwen2
ops (the reference routes the same function: aklr/plugins/sglang/models/qwen2_moe/api.py:104-154).

A checkpoint with Quark's MXFP4 experts keeps its shared expert in bf16, apart from the experts; sglang
cannot fuse it as a slot, so for those blocks the whole ``forward`` is routed to ``qwen2_moe_mxfp4_moe``
(as the reference does: api.py:67-101) and every other block runs sglang's ``forward``, which reaches the
``_forward_router_experts`` route below.

The ops form a ladder, widest first; a rung that declines (a shape or dtype outside its contract)
hands over to the next:

1. ``qwen2_moe_fp8_router_experts``: gate GEMM, softmax top-k, sigmoid-gated shared slot, experts;
2. ``qwen2_moe_router`` for the routing, then ``qwen2_moe_fp8_experts``;
3. ``qwen2_moe_router`` for the routing, then sglang's own experts on it.
"""

from __future__ import annotations

import torch

from aklr_b200.core.dispatch import FallbackReason
from aklr_b200.ops import qwen2_moe_fp8_experts, qwen2_moe_fp8_router_experts, qwen2_moe_mxfp4_moe, qwen2_moe_router
from aklr_b200.plugins.sglang.conditions import leave_to_sglang, when
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks

TARGET = "sglang.srt.models.qwen2_moe.Qwen2MoeSparseMoeBlock._forward_router_experts"
BLOCK_TARGET = "sglang.srt.models.qwen2_moe.Qwen2MoeSparseMoeBlock.forward"


def _unmet(block, hidden_states, defer_finalize) -> str | None:
    from sglang.srt.runtime_context import get_parallel

    return (
        when(defer_finalize, "finalize not deferred")
        or when(not torch.is_tensor(hidden_states), "a tensor in, not a quantised pair")
        or moe_blocks.runtime_unmet()
        # w1 is indexed by the router's ids, so this rank must hold every expert
        or when(get_parallel().moe_ep_size != 1, "expert parallelism of one")
        or when(block.num_fused_shared_experts != 1, "one shared expert fused as the last slot")
        or moe_blocks.topk_unmet(block.topk, scoring_func="softmax", biased=False)
        or moe_blocks.experts_unmet(block.experts, ("Fp8MoEMethod",))
    )


def _sglang_experts_on(block, hidden_states, topk_weights, topk_ids):
    """Rung 3: sglang's experts, fed the op's routing the way sglang's small-batch router leaves its
    own (weights and ids, no logits), the shared slot appended by the block's own method."""
    from sglang.srt.layers.moe.topk import StandardTopKOutput

    routed = StandardTopKOutput(topk_weights=topk_weights, topk_ids=topk_ids, router_logits=None)
    return block.experts(hidden_states, block._append_shared_to_topk_output(routed, hidden_states))


@sglang_route(TARGET, versions=("0.5.22", "0.5.23"))
def _forward_router_experts(self, hidden_states, *, defer_finalize=False):
    """This rank's share of router + experts (shared expert last), as sglang's function returns it."""
    if (why := _unmet(self, hidden_states, defer_finalize)) is not None:
        return leave_to_sglang(TARGET, why)
    top_k = self.topk.topk_config.top_k
    common = dict(
        hidden_states=hidden_states,
        shared_gate_weight=self.shared_expert_gate.weight,
        **moe_blocks.fp8_expert_weights(self.experts),
    )
    out = qwen2_moe_fp8_router_experts(router_weight=self.gate.weight, topk=top_k, **common)
    if not isinstance(out, FallbackReason):
        return out

    picks = (hidden_states.shape[0], top_k)
    routing = qwen2_moe_router(
        hidden_states=hidden_states,
        router_weight=self.gate.weight,
        topk_weights=hidden_states.new_empty(picks, dtype=torch.float32),
        topk_ids=hidden_states.new_empty(picks, dtype=torch.int32),
    )
    if isinstance(routing, FallbackReason):
        return routing
    topk_weights, topk_ids = routing
    out = qwen2_moe_fp8_experts(topk_weights=topk_weights, topk_ids=topk_ids, **common)
    if isinstance(out, FallbackReason):
        out = _sglang_experts_on(self, hidden_states, topk_weights, topk_ids)
    return out


def _plain_bf16_linear_unmet(layer, kind: str, what: str) -> str | None:
    """``layer`` multiplies by its weight as stored: a plain ``kind`` on the unquantised method, no bias (a LoRA
    layer wraps it in another class)."""
    return when(
        type(layer).__name__ != kind or type(layer.quant_method).__name__ != "UnquantizedLinearMethod" or layer.bias is not None,
        f"{what} a plain bf16 {kind} without a bias",
    )


def _shared_expert_unmet(shared) -> str | None:
    """The shared expert computes down(silu(gate(x)) * up(x)) of its bf16 weights and returns this rank's share."""
    up, down = shared.gate_up_proj, shared.down_proj
    return (
        when(type(shared).__name__ != "Qwen2MoeMLP", "the shared expert a Qwen2MoeMLP")
        or when(type(shared.act_fn).__name__ != "SiluAndMul", "SiLU in the shared expert")
        or when(shared._enable_silu_fp4_quant_fusion, "no FP4 quantisation fused into the shared expert's SiLU")
        or _plain_bf16_linear_unmet(up, "MergedColumnParallelLinear", "the shared gate_up projection")
        or _plain_bf16_linear_unmet(down, "RowParallelLinear", "the shared down projection")
        or when(up.gather_output or not down.input_is_parallel, "the shared expert split over the TP group by rows of its intermediate")
        # the down projection would sum the shared expert over the TP group by itself
        or when(down.reduce_results or down.use_decode_attn_tp, "the shared expert's sum over the ranks left to the block")
    )


def _block_unmet(block, hidden_states, defer_finalize) -> str | None:
    """What keeps the whole block from running as qwen2_moe_mxfp4_moe computes it (the reference's
    _unfused_block_falls_back, aklr/plugins/sglang/models/qwen2_moe/api.py:167-192)."""
    from sglang.srt.models import qwen2_moe
    from sglang.srt.runtime_context import get_forward, get_parallel

    gate = block.shared_expert_gate
    return (
        when(defer_finalize, "finalize not deferred")
        or when(not torch.is_tensor(hidden_states) or hidden_states.dim() != 2, "a [tokens, hidden] tensor in")
        or moe_blocks.runtime_unmet()
        or when(get_parallel().moe_ep_size != 1, "expert parallelism of one")
        # sequence parallelism gathers the shared expert's input and scatters its output
        or when(get_forward().sp_active, "sequence parallelism off")
        or when(block.num_fused_shared_experts != 0 or block.shared_expert is None, "a shared expert apart from the routed ones")
        or when(type(gate) is not torch.nn.Linear or gate.bias is not None, "a plain linear shared-expert gate")
        or when(qwen2_moe._SGLANG_EXPERIMENTAL_LORA_OPTI, "the LoRA MoE dispatch off")
        or _plain_bf16_linear_unmet(block.gate, "ReplicatedLinear", "the router")
        or _shared_expert_unmet(block.shared_expert)
        or moe_blocks.topk_unmet(block.topk, scoring_func="softmax", biased=False)
        or moe_blocks.experts_unmet(block.experts, ("QuarkW4A4MXFp4MoE",))
    )


def _block_arguments(block, hidden_states) -> dict:
    shared = block.shared_expert
    return dict(
        hidden_states=hidden_states,
        router_weight=block.gate.weight,
        **moe_blocks.mxfp4_expert_weights(block.experts),
        shared_w1=shared.gate_up_proj.weight,
        shared_w2=shared.down_proj.weight,
        shared_gate_weight=block.shared_expert_gate.weight,
        topk=block.topk.topk_config.top_k,
    )


@sglang_route(BLOCK_TARGET, versions=("0.5.22", "0.5.23"))
def _forward(self, hidden_states, forward_batch=None, defer_finalize=False):
    """The whole block with MXFP4 experts and its bf16 shared expert as one op, then the sum over the TP group
    where sglang's forward does it."""
    if (why := _block_unmet(self, hidden_states, defer_finalize)) is not None:
        return leave_to_sglang(BLOCK_TARGET, why)
    out = qwen2_moe_mxfp4_moe(**_block_arguments(self, hidden_states))
    if isinstance(out, FallbackReason) or not self.reduce_results:
        return out
    from sglang.srt.layers.moe import reduce_moe_output

    return reduce_moe_output(out)
