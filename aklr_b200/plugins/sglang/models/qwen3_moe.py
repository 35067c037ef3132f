"""Qwen3-MoE on sglang: ``Qwen3MoeSparseMoeBlock.forward_normal`` served by ``qwen3_moe_fp8_moe``
(the reference routes the same function: aklr/plugins/sglang/models/qwen3_moe/api.py:26-77)."""

from __future__ import annotations

from aklr_b200.ops import qwen3_moe_fp8_moe
from aklr_b200.plugins.sglang.conditions import leave_to_sglang, when
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks

TARGET = "sglang.srt.models.qwen3_moe.Qwen3MoeSparseMoeBlock.forward_normal"


def _unmet(block) -> str | None:
    """Why ``block`` is not a softmax top-k over a replicated bf16 gate feeding FP8 experts that this
    rank holds in full."""
    from sglang.srt.runtime_context import get_parallel

    gate = block.gate
    return (
        when(moe_blocks.masks_padded_rows(), "no padded rows masked by the top-k")
        or moe_blocks.runtime_unmet()
        # the op indexes w1 by the router's ids, so every expert has to be on this rank
        or when(get_parallel().moe_ep_size != 1, "expert parallelism of one")
        or when(type(gate).__name__ != "ReplicatedLinear", "a replicated gate")
        or when(type(gate.quant_method).__name__ != "UnquantizedLinearMethod", "an unquantised gate")
        or moe_blocks.topk_unmet(block.topk, scoring_func="softmax", biased=False)
        or moe_blocks.experts_unmet(block.experts, ("Fp8MoEMethod",))
    )


@sglang_route(TARGET, versions=("0.5.22", "0.5.23"))
def _moe_forward_normal(self, hidden_states):
    """This rank's share of the block's output; sglang sums the ranks at the layer boundary."""
    if (why := _unmet(self)) is not None:
        return leave_to_sglang(TARGET, why)
    return qwen3_moe_fp8_moe(
        hidden_states=hidden_states,
        router_weight=self.gate.weight,
        topk=self.topk.topk_config.top_k,
        **moe_blocks.fp8_expert_weights(self.experts),
    )
