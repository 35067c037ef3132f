"""sglang's DeepseekV2MoE.forward_normal as one op call (the reference's route:
aklr/plugins/sglang/models/deepseek_v2/api.py:53-139)."""

from __future__ import annotations

from aklr_b200.core.dispatch import FallbackReason
from aklr_b200.ops import deepseek_v2_fp8_moe
from aklr_b200.plugins.sglang.hook import sglang_route
from aklr_b200.plugins.sglang.models import moe_blocks

_EXPERT_FORMATS = ("Fp8MoEMethod",)


@sglang_route("sglang.srt.models.deepseek_v2.DeepseekV2MoE.forward_normal", versions=("0.5.23",))
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
    """Router, top-k and experts (the shared one last) as one op call, then forward_normal's
    all-reduce unless a later step sums the ranks."""
    if _forward_normal_falls_back(self, skip_shared_experts, use_vision_topk, return_moe_output or leave_output_sum):
        return FallbackReason.OUT_OF_CONTRACT
    out = deepseek_v2_fp8_moe(**_moe_arguments(self, hidden_states))
    if isinstance(out, FallbackReason) or not self.reduce_results:
        return out
    from sglang.srt.layers.moe import post_experts_all_reduce

    return post_experts_all_reduce(out)


def _forward_normal_falls_back(mlp, skip_shared_experts, use_vision_topk, return_moe_output) -> bool:
    return bool(
        skip_shared_experts
        or use_vision_topk
        or return_moe_output
        or _masks_padded_rows()
        or moe_blocks.runtime_falls_back()
        or moe_blocks.experts_fall_back(mlp.experts, _EXPERT_FORMATS)
        or mlp._fuse_shared_experts_inside_sbo
        or mlp.is_hash
        or mlp.gate.e_score_correction_bias_vl is not None
    )


def _masks_padded_rows() -> bool:
    """Whether sglang's top-k masks padded rows here (the op routes every row)."""
    from sglang.srt.model_executor.forward_context import get_forward_context, has_forward_context

    if not has_forward_context():
        return False
    get_bound = get_forward_context().moe_num_token_non_padded
    return get_bound is not None and get_bound() is not None


def _moe_arguments(mlp, hidden_states) -> dict:
    """The op's arguments: the module's weights and its input."""
    experts, routing = mlp.experts, mlp.topk.topk_config
    grouped = routing.use_grouped_topk
    bias = routing.correction_bias
    if bias is not None and bias.dtype != hidden_states.dtype:  # the op reads the bias in the logits' dtype
        bias = routing.correction_bias_for_dtype(hidden_states.dtype)
    return {
        "hidden_states": hidden_states,
        "router_weight": mlp.gate.weight,
        "correction_bias": bias,
        "w1": experts.w13_weight,
        "w1_scale": experts.w13_weight_scale_inv,
        "w2": experts.w2_weight,
        "w2_scale": experts.w2_weight_scale_inv,
        "topk": routing.top_k - routing.num_fused_shared_experts,
        "num_expert_group": routing.num_expert_group if grouped else 1,
        "topk_group": routing.topk_group if grouped else 1,
        "renormalize": routing.renormalize,
        "scoring_func": routing.scoring_func,
        "routed_scaling_factor": mlp.routed_scaling_factor,
    }
