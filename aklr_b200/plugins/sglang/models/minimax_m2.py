"""sglang's MiniMaxM2MoE.forward_normal as one op call (the reference's route:
aklr/plugins/sglang/models/minimax_m2/api.py:47-88).  Only the FP8 experts are served here; the
MXFP4 checkpoints of this model (weights at an e8m0 scale per 32 with UNQUANTISED activations,
minimax_m2/reference.py:120-132) fall back to the engine."""

from __future__ import annotations

from aklr_b200.core.dispatch import FallbackReason
from aklr_b200.ops import minimax_m2_fp8_moe
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks


@sglang_route("sglang.srt.models.minimax_m2.MiniMaxM2MoE.forward_normal", versions=("0.5.22", "0.5.23"))
def _moe_forward_normal(self, hidden_states):
    """The MoE's gate, routing and this rank's experts as one op call; sglang's layer boundary sums
    the ranks' shares after it, as it does sglang's own."""
    if moe_blocks.runtime_falls_back() or _moe_falls_back(self):
        return FallbackReason.OUT_OF_CONTRACT
    experts, routing = self.experts, self.topk.topk_config
    return minimax_m2_fp8_moe(
        hidden_states=hidden_states,
        router_weight=self.gate.weight,
        correction_bias=routing.correction_bias,
        w1=experts.w13_weight,
        w1_scale=experts.w13_weight_scale_inv,
        w2=experts.w2_weight,
        w2_scale=experts.w2_weight_scale_inv,
        topk=routing.top_k,
        # the router row of this rank's first expert
        expert_offset=experts.moe_ep_rank * experts._num_local_routed,
    )


def _moe_falls_back(moe) -> bool:
    from sglang.srt.layers.dp_attention import is_dp_attention_enabled

    return bool(
        # the experts would take the rows gathered over the attention ranks, not this rank's
        is_dp_attention_enabled()
        or moe_blocks.topk_falls_back(moe.topk, scoring_func="sigmoid", biased=True)
        or moe_blocks.experts_fall_back(moe.experts, ("Fp8MoEMethod",))
    )
