"""MiniMax-M2 on sglang: ``MiniMaxM2MoE.forward_normal`` served by ``minimax_m2_fp8_moe`` (the
reference routes the same function: aklr/plugins/sglang/models/minimax_m2/api.py:47-88).

Only FP8 experts are served.  The model's MXFP4 checkpoints keep their activations unquantised
against e8m0-per-32 weights (minimax_m2/reference.py:120-132), a mix this build has no kernel for, so
those stay on sglang."""

from __future__ import annotations

from aklr_b200.ops import minimax_m2_fp8_moe
from aklr_b200.plugins.sglang.conditions import leave_to_sglang, when
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks

TARGET = "sglang.srt.models.minimax_m2.MiniMaxM2MoE.forward_normal"


def _unmet(moe) -> str | None:
    from sglang.srt.layers.dp_attention import is_dp_attention_enabled

    return (
        moe_blocks.runtime_unmet()
        # under DP attention the experts see rows gathered from every attention rank
        or when(is_dp_attention_enabled(), "DP attention off")
        or moe_blocks.topk_unmet(moe.topk, scoring_func="sigmoid", biased=True)
        or moe_blocks.experts_unmet(moe.experts, ("Fp8MoEMethod",))
    )


@sglang_route(TARGET, versions=("0.5.22", "0.5.23"))
def _moe_forward_normal(self, hidden_states):
    """Gate, biased sigmoid top-k and the experts this rank holds; the ranks' shares are summed by
    sglang after the block, as they are for its own path."""
    if (why := _unmet(self)) is not None:
        return leave_to_sglang(TARGET, why)
    experts, routing = self.experts, self.topk.topk_config
    first_local_expert = experts.moe_ep_rank * experts._num_local_routed
    return minimax_m2_fp8_moe(
        hidden_states=hidden_states,
        router_weight=self.gate.weight,
        correction_bias=routing.correction_bias,
        topk=routing.top_k,
        expert_offset=first_local_expert,  # the gate row of w1[0]
        **moe_blocks.fp8_expert_weights(experts),
    )
