"""Qwen2-MoE on sglang: ``Qwen2MoeSparseMoeBlock._forward_router_experts`` served by the three Qwen2
ops (the reference routes the same function: aklr/plugins/sglang/models/qwen2_moe/api.py:104-154).

The reference also routes the block's whole ``forward`` for MXFP4 experts with a separate bf16 shared
expert (api.py:67-101); this build has no kernel for that format and leaves those blocks to sglang.

The ops form a ladder, widest first; a rung that declines (a shape or dtype outside its contract)
hands over to the next:

1. ``qwen2_moe_fp8_router_experts``: gate GEMM, softmax top-k, sigmoid-gated shared slot, experts;
2. ``qwen2_moe_router`` for the routing, then ``qwen2_moe_fp8_experts``;
3. ``qwen2_moe_router`` for the routing, then sglang's own experts on it.
"""

from __future__ import annotations

import torch

from aklr_b200.core.dispatch import FallbackReason
from aklr_b200.ops import qwen2_moe_fp8_experts, qwen2_moe_fp8_router_experts, qwen2_moe_router
from aklr_b200.plugins.sglang.conditions import leave_to_sglang, when
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks

TARGET = "sglang.srt.models.qwen2_moe.Qwen2MoeSparseMoeBlock._forward_router_experts"


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
