"""DeepSeek-V2/V3 on sglang: ``DeepseekV2MoE.forward_normal`` served by ``deepseek_v2_fp8_moe`` (experts in FP8
at a scale per 128 x 128 block) or ``deepseek_v2_mxfp4_moe`` (Quark's MXFP4 experts, ungrouped routing) -- the
reference routes the same function to the same two ops: aklr/plugins/sglang/models/deepseek_v2/api.py:53-139."""

from __future__ import annotations

from aklr_b200.core.dispatch import FallbackReason
from aklr_b200.ops import deepseek_v2_fp8_moe, deepseek_v2_mxfp4_moe
from aklr_b200.plugins.sglang.conditions import leave_to_sglang, when
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks

TARGET = "sglang.srt.models.deepseek_v2.DeepseekV2MoE.forward_normal"
EXPERT_FORMATS = ("QuarkW4A4MXFp4MoE", "Fp8MoEMethod")  # the experts' formats the two ops take


def _unmet(mlp, call_flags: dict) -> str | None:
    """Why this call is not the plain one: a flag of forward_normal asks for something else, or the
    module is set up in a way the op does not compute."""
    for flag, value in call_flags.items():
        if value:
            return f"{flag} not set"
    return (
        when(moe_blocks.masks_padded_rows(), "no padded rows masked by the top-k")
        or moe_blocks.runtime_unmet()
        or moe_blocks.experts_unmet(mlp.experts, EXPERT_FORMATS)
        or when(mlp._fuse_shared_experts_inside_sbo, "shared experts not fused into single-batch overlap")
        or when(mlp.is_hash, "no hash routing")
        or when(mlp.gate.e_score_correction_bias_vl is not None, "no vision-language correction bias")
    )


def _moe_call(mlp, hidden_states):
    """(op, keyword arguments) for the experts' format."""
    if moe_blocks.experts_format(mlp.experts) == "QuarkW4A4MXFp4MoE":
        arguments = _moe_arguments(mlp, hidden_states, keep_bias_dtype=True, weights=False)
        arguments.update(moe_blocks.mxfp4_expert_weights(mlp.experts))
        return deepseek_v2_mxfp4_moe, arguments
    return deepseek_v2_fp8_moe, _moe_arguments(mlp, hidden_states)


def _moe_arguments(mlp, hidden_states, keep_bias_dtype: bool = False, weights: bool = True) -> dict:
    """The layer ops' keyword arguments read off the module (``deepseek_v2_fp8_moe`` takes the bias in the logits'
    dtype, ``deepseek_v2_mxfp4_moe`` as the module holds it, in float32)."""
    routing = mlp.topk.topk_config
    groups, kept_groups = (routing.num_expert_group, routing.topk_group) if routing.use_grouped_topk else (1, 1)
    bias = routing.correction_bias
    if not keep_bias_dtype and bias is not None and bias.dtype != hidden_states.dtype:
        bias = routing.correction_bias_for_dtype(hidden_states.dtype)  # the op adds it to logits of that dtype
    return dict(
        hidden_states=hidden_states,
        router_weight=mlp.gate.weight,
        correction_bias=bias,
        # sglang counts the fused shared expert as one more routed pick; the op appends it itself
        topk=routing.top_k - routing.num_fused_shared_experts,
        num_expert_group=groups,
        topk_group=kept_groups,
        renormalize=routing.renormalize,
        scoring_func=routing.scoring_func,
        routed_scaling_factor=mlp.routed_scaling_factor,
        **(moe_blocks.fp8_expert_weights(mlp.experts) if weights else {}),
    )


@sglang_route(TARGET, versions=("0.5.23",))
def _moe_forward_normal(
    self,
    hidden_states,
    gemm_output_zero_allocator=None,
    input_ids=None,
    input_ids_global=None,
    skip_shared_experts=False,
    use_vision_topk=False,
    return_moe_output=False,
    leave_output_sum=False,
):
    """The whole block (shared expert as the last slot) in one op call, followed by the all-reduce
    forward_normal itself would do when the module reduces its own results."""
    flags = dict(
        skip_shared_experts=skip_shared_experts,
        use_vision_topk=use_vision_topk,
        return_moe_output=return_moe_output,
        leave_output_sum=leave_output_sum,
    )
    if (why := _unmet(self, flags)) is not None:
        return leave_to_sglang(TARGET, why)
    op, arguments = _moe_call(self, hidden_states)
    out = op(**arguments)
    if self.reduce_results and not isinstance(out, FallbackReason):
        from sglang.srt.layers.moe import post_experts_all_reduce

        out = post_experts_all_reduce(out)
    return out
