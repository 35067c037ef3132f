"""MiniMax-M2 on sglang: ``MiniMaxM2MoE.forward_normal`` served by ``minimax_m2_fp8_moe`` (experts in FP8 at a
scale per 128 x 128 block) or ``minimax_m2_mxfp4_moe`` (Quark's MXFP4 experts, activations left unquantised) -- the
reference routes the same function to the same two ops: aklr/plugins/sglang/models/minimax_m2/api.py:45-88."""

from __future__ import annotations

from aklr_b200.ops import minimax_m2_fp8_moe, minimax_m2_mxfp4_moe
from aklr_b200.plugins.sglang.conditions import leave_to_sglang, when
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks

TARGET = "sglang.srt.models.minimax_m2.MiniMaxM2MoE.forward_normal"
EXPERT_FORMATS = ("Fp8MoEMethod", "QuarkW4A4MXFp4MoE")


def _unmet(moe) -> str | None:
    from sglang.srt.layers.dp_attention import is_dp_attention_enabled

    return (
        moe_blocks.runtime_unmet()
        # under DP attention the experts see rows gathered from every attention rank
        or when(is_dp_attention_enabled(), "DP attention off")
        or moe_blocks.topk_unmet(moe.topk, scoring_func="sigmoid", biased=True)
        or moe_blocks.experts_unmet(moe.experts, EXPERT_FORMATS)
    )


def _moe_call(moe):
    """(op, its keyword arguments but the input) for the experts' format; ``expert_offset`` is the gate row of
    this rank's first expert."""
    experts, routing = moe.experts, moe.topk.topk_config
    arguments = dict(
        router_weight=moe.gate.weight,
        correction_bias=routing.correction_bias,
        topk=routing.top_k,
        expert_offset=experts.moe_ep_rank * experts._num_local_routed,
    )
    if moe_blocks.experts_format(experts) == "QuarkW4A4MXFp4MoE":
        return minimax_m2_mxfp4_moe, {**arguments, **moe_blocks.mxfp4_expert_weights(experts)}
    return minimax_m2_fp8_moe, {**arguments, **moe_blocks.fp8_expert_weights(experts)}


@sglang_route(TARGET, versions=("0.5.22", "0.5.23"))
def _moe_forward_normal(self, hidden_states):
    """Gate, biased sigmoid top-k and the experts this rank holds; the ranks' shares are summed by
    sglang after the block, as they are for its own path."""
    if (why := _unmet(self)) is not None:
        return leave_to_sglang(TARGET, why)
    op, arguments = _moe_call(self)
    return op(hidden_states=hidden_states, **arguments)
