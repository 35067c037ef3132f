"""Fallback checks the MoE routes share (the reference's aklr/plugins/sglang/models/moe_blocks.py);
shapes, dtypes and empty calls are the ops' to decline.

Every semantic predicate of the reference is kept.  What pinned ROCm there -- "the experts run on
aiter's fused_moe" -- becomes "the experts sit on a CUDA device of compute capability 10.0".
"""

from __future__ import annotations

import torch

__all__ = ["experts_fall_back", "experts_format", "runtime_falls_back", "topk_falls_back"]


def runtime_falls_back() -> bool:
    """Whether sglang's graph mode or configuration keeps MoE calls on sglang."""
    from sglang.srt.environ import envs
    from sglang.srt.layers.moe import get_moe_a2a_backend
    from sglang.srt.model_executor.runner_backend_utils.breakable_cuda_graph.context import (
        is_in_breakable_cuda_graph,
    )
    from sglang.srt.model_executor.runner_backend_utils.tc_piecewise_cuda_graph.context_manager import (
        is_in_tc_piecewise_cuda_graph,
    )
    from sglang.srt.runtime_context import get_exec, get_parallel

    exec_, parallel = get_exec(), get_parallel()
    moe = exec_.moe
    return bool(
        is_in_tc_piecewise_cuda_graph()
        or is_in_breakable_cuda_graph()
        or not get_moe_a2a_backend().is_none()
        or moe.ep_join_mode is not None
        or parallel.dwdp_size > 1
        or exec_.deterministic.enable_deterministic_inference
        or moe.enable_waterfill
        or moe.enable_eplb
        or moe.init_expert_location != "trivial"
        or moe.ep_num_redundant_experts > 0
        or moe.expert_distribution_recorder_mode is not None
        or exec_.features.enable_return_routed_experts
        or envs.SGLANG_SIMULATE_UNIFORM_EXPERTS.get()
        or envs.SGLANG_SIMULATE_ROUND_ROBIN_EXPERTS.get()
    )


def topk_falls_back(topk, *, scoring_func: str, biased: bool) -> bool:
    """Whether ``topk`` routes other than a plain ungrouped top-k of ``scoring_func`` scores with a
    correction bias exactly when ``biased``."""
    config = topk.topk_config
    return bool(
        config.use_grouped_topk
        or config.custom_routing_function is not None
        or config.scoring_func != scoring_func
        or (config.correction_bias is not None) != biased
        or not config.renormalize
        or config.num_fused_shared_experts != 0
        or config.routed_scaling_factor not in (None, 1.0)
        or config.apply_routed_scaling_factor_on_output
    )


def experts_format(experts) -> str:
    """The class naming the experts' format: their scheme's, else their quant method's."""
    return type(getattr(experts, "scheme", None) or experts.quant_method).__name__


def _on_sm100(experts) -> bool:
    weight = getattr(experts, "w13_weight", None)
    if not isinstance(weight, torch.Tensor) or not weight.is_cuda:
        return False
    return torch.cuda.get_device_capability(weight.device)[0] == 10


def experts_fall_back(experts, formats) -> bool:
    """Whether ``experts`` run other than as the ops take them: in none of ``formats``, not gated
    SiLU at sglang's standard dispatch, or not on a B200."""
    if (
        experts_format(experts) not in formats
        or type(experts).__name__ != "FusedMoE"
        or type(experts.dispatcher).__name__ != "StandardDispatcher"
        or experts.reduce_results
    ):
        return True
    runner = _supported_runner(experts)
    if runner is None or not _on_sm100(experts):
        return True
    config = runner.config
    return bool(
        config.activation != "silu"
        or not config.is_gated
        or config.apply_router_weight_on_input
        or config.no_combine
        or config.gemm1_alpha is not None
        or config.gemm1_clamp_limit is not None
        or config.swiglu_limit not in (None, 0.0)
        or getattr(experts, "w13_weight_bias", None) is not None
        or getattr(experts, "w2_weight_bias", None) is not None
        or getattr(experts, "fp8_activations", False)
    )


def _supported_runner(experts):
    """The runner of experts held as the ops take them (fp8 at a scale per 128 x 128 block, weights
    row-major), else None."""
    if experts_format(experts) != "Fp8MoEMethod":
        return None
    method = experts.quant_method
    if (
        not method.block_quant
        or getattr(method, "use_mxfp8", False)
        or getattr(method, "is_fp4_expert", False)
        or list(method.weight_block_size) != [128, 128]
    ):
        return None
    return getattr(method, "runner", None)
