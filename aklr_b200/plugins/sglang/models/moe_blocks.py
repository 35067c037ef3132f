"""What every MoE route asks of sglang before it serves a call, as tables of named conditions.

The requirements are the reference's (aklr/plugins/sglang/models/moe_blocks.py) with one substitution:
where it asks that the experts run on aiter's ROCm fused_moe, this build asks that they sit on a CUDA
device of compute capability 10.x.  Shapes, dtypes and empty inputs are not checked here: the ops'
contracts decline those themselves.

Three subjects are checked: the process (``runtime_unmet``), a block's TopK module (``topk_unmet``) and
its FusedMoE experts (``experts_unmet``).  Each returns the label of the first unmet condition or None;
the ``*_falls_back`` forms are their truth values.
"""

from __future__ import annotations

from types import SimpleNamespace

import torch

from aklr_b200.plugins.sglang.conditions import Condition, attr, first_unmet

__all__ = [
    "experts_fall_back",
    "experts_format",
    "experts_unmet",
    "fp8_expert_weights",
    "masks_padded_rows",
    "runtime_falls_back",
    "runtime_unmet",
    "topk_falls_back",
    "topk_unmet",
]

FP8_BLOCK = [128, 128]


# ------------------------------------------------------------------------------------------------
# the process: graph capture modes and MoE features that change what a MoE call must compute
# ------------------------------------------------------------------------------------------------
def _runtime_snapshot() -> SimpleNamespace:
    """sglang's process-wide state, read once per call into plain fields."""
    from sglang.srt.environ import envs
    from sglang.srt.layers.moe import get_moe_a2a_backend
    from sglang.srt.model_executor.runner_backend_utils.breakable_cuda_graph.context import (
        is_in_breakable_cuda_graph,
    )
    from sglang.srt.model_executor.runner_backend_utils.tc_piecewise_cuda_graph.context_manager import (
        is_in_tc_piecewise_cuda_graph,
    )
    from sglang.srt.runtime_context import get_exec, get_parallel

    executor = get_exec()
    return SimpleNamespace(
        executor=executor,
        moe=executor.moe,
        parallel=get_parallel(),
        piecewise_graph=is_in_tc_piecewise_cuda_graph(),
        breakable_graph=is_in_breakable_cuda_graph(),
        all_to_all=not get_moe_a2a_backend().is_none(),
        simulated_routing=bool(
            envs.SGLANG_SIMULATE_UNIFORM_EXPERTS.get() or envs.SGLANG_SIMULATE_ROUND_ROBIN_EXPERTS.get()
        ),
    )


_RUNTIME = (
    Condition("not inside a piecewise CUDA graph", lambda s: not s.piecewise_graph),
    Condition("not inside a breakable CUDA graph", lambda s: not s.breakable_graph),
    Condition("no all-to-all MoE backend", lambda s: not s.all_to_all),
    Condition("no expert-parallel join mode", lambda s: s.moe.ep_join_mode is None),
    Condition("no DWDP", lambda s: s.parallel.dwdp_size <= 1),
    Condition("deterministic inference off", lambda s: not s.executor.deterministic.enable_deterministic_inference),
    Condition("waterfill off", lambda s: not s.moe.enable_waterfill),
    Condition("expert load balancing off", lambda s: not s.moe.enable_eplb),
    Condition("experts at their trivial locations", lambda s: s.moe.init_expert_location == "trivial"),
    Condition("no redundant experts", lambda s: s.moe.ep_num_redundant_experts <= 0),
    Condition("expert distribution not recorded", lambda s: s.moe.expert_distribution_recorder_mode is None),
    Condition("routed experts not returned", lambda s: not s.executor.features.enable_return_routed_experts),
    Condition("routing not simulated", lambda s: not s.simulated_routing),
)


def runtime_unmet() -> str | None:
    return first_unmet(_runtime_snapshot(), _RUNTIME)


def runtime_falls_back() -> bool:
    """Whether sglang's graph mode or configuration keeps MoE calls on sglang."""
    return runtime_unmet() is not None


def masks_padded_rows() -> bool:
    """Whether sglang's top-k masks the rows past a bound in this forward (the ops route every row)."""
    from sglang.srt.model_executor.forward_context import get_forward_context, has_forward_context

    if not has_forward_context():
        return False
    bound = get_forward_context().moe_num_token_non_padded
    return bound is not None and bound() is not None


# ------------------------------------------------------------------------------------------------
# the TopK module: a plain, renormalised, ungrouped top-k with nothing applied afterwards
# ------------------------------------------------------------------------------------------------
_PLAIN_TOPK = (
    Condition("ungrouped top-k", lambda c: not c.use_grouped_topk),
    Condition("no custom routing function", lambda c: c.custom_routing_function is None),
    Condition("renormalised weights", lambda c: bool(c.renormalize)),
    Condition("no shared expert fused into the top-k", lambda c: c.num_fused_shared_experts == 0),
    Condition("routed scaling factor of one", lambda c: c.routed_scaling_factor in (None, 1.0)),
    Condition("no scaling applied on the output", lambda c: not c.apply_routed_scaling_factor_on_output),
)


def topk_unmet(topk, *, scoring_func: str, biased: bool) -> str | None:
    """What keeps ``topk`` from being a plain top-k over ``scoring_func`` scores, carrying a correction
    bias exactly when ``biased``."""
    config = topk.topk_config
    if config.scoring_func != scoring_func:
        return f"{scoring_func} scores"
    if (config.correction_bias is not None) != biased:
        return "a correction bias" if biased else "no correction bias"
    return first_unmet(config, _PLAIN_TOPK)


def topk_falls_back(topk, *, scoring_func: str, biased: bool) -> bool:
    return topk_unmet(topk, scoring_func=scoring_func, biased=biased) is not None


# ------------------------------------------------------------------------------------------------
# the experts: FusedMoE at sglang's standard dispatch, block-scaled FP8, gated SiLU, on a B200
# ------------------------------------------------------------------------------------------------
def experts_format(experts) -> str:
    """The class that names the experts' format: their scheme's when they have one, else their
    quantisation method's."""
    scheme = getattr(experts, "scheme", None)
    return type(scheme if scheme else experts.quant_method).__name__


def _on_sm100(experts) -> bool:
    weight = getattr(experts, "w13_weight", None)
    return bool(
        isinstance(weight, torch.Tensor)
        and weight.is_cuda
        and torch.cuda.get_device_capability(weight.device)[0] == 10
    )


_MODULE = (
    Condition("a FusedMoE module", lambda e: type(e).__name__ == "FusedMoE"),
    Condition("sglang's standard dispatcher", lambda e: type(e.dispatcher).__name__ == "StandardDispatcher"),
    Condition("the ranks' sum left to the caller", lambda e: not e.reduce_results),
    Condition("no bias on the expert weights", lambda e: attr(e, "w13_weight_bias", None) is None and attr(e, "w2_weight_bias", None) is None),
    Condition("bf16 activations in", lambda e: not attr(e, "fp8_activations", False)),
)

_FP8_METHOD = (
    Condition("block-quantised weights", lambda m: bool(m.block_quant)),
    Condition("not MXFP8", lambda m: not attr(m, "use_mxfp8", False)),
    Condition("not FP4 experts", lambda m: not attr(m, "is_fp4_expert", False)),
    Condition("a scale per 128 x 128 block", lambda m: list(m.weight_block_size) == FP8_BLOCK),
    Condition("a runner", lambda m: attr(m, "runner", None) is not None),
)

_GATED_SILU = (
    Condition("SiLU activation", lambda c: c.activation == "silu"),
    Condition("gated", lambda c: bool(c.is_gated)),
    Condition("router weights applied on the output", lambda c: not c.apply_router_weight_on_input),
    Condition("combined output", lambda c: not c.no_combine),
    Condition("no gemm1 alpha", lambda c: c.gemm1_alpha is None),
    Condition("no gemm1 clamp", lambda c: c.gemm1_clamp_limit is None),
    Condition("no SwiGLU limit", lambda c: c.swiglu_limit in (None, 0.0)),
)


# Quark's MXFP4 experts at dynamic input scales (the reference's _supported_runner,
# aklr/plugins/sglang/models/moe_blocks.py:104-126)
_QUARK_MXFP4 = (
    Condition("Quark's fused-MoE method itself", lambda e: type(e.quant_method).__name__ == "QuarkFusedMoEMethod"),
    Condition("dynamic input scales", lambda e: not e.scheme.static_input_scales),
    Condition("no zeroed intermediate padding on presharded weights",
              lambda e: not (attr(e, "intermediate_pad", 0) != 0 and e.use_presharded_weights)),
    Condition("a runner", lambda e: attr(e.scheme, "runner", None) is not None),
)


def experts_unmet(experts, formats) -> str | None:
    """What keeps ``experts`` from running as the ops compute them; ``formats`` are the format class
    names the calling route serves."""
    found = experts_format(experts)
    if found not in formats:
        return f"experts in {found}, not one of {', '.join(formats)}"
    if found == "QuarkW4A4MXFp4MoE":
        unmet = first_unmet(experts, _MODULE) or first_unmet(experts, _QUARK_MXFP4)
        if unmet is None and not _on_sm100(experts):
            unmet = "weights on a compute capability 10.x device"
        return unmet or first_unmet(experts.scheme.runner.config, _GATED_SILU)
    if found != "Fp8MoEMethod":
        return f"{found} experts have no kernel here"
    method = experts.quant_method
    unmet = first_unmet(experts, _MODULE) or first_unmet(method, _FP8_METHOD)
    if unmet is None and not _on_sm100(experts):
        unmet = "weights on a compute capability 10.x device"
    return unmet or first_unmet(method.runner.config, _GATED_SILU)


def experts_fall_back(experts, formats) -> bool:
    return experts_unmet(experts, formats) is not None


def fp8_expert_weights(experts) -> dict:
    """The four weight arguments every FP8 op takes, from a FusedMoE's parameters."""
    return {
        "w1": experts.w13_weight,
        "w1_scale": experts.w13_weight_scale_inv,
        "w2": experts.w2_weight,
        "w2_scale": experts.w2_weight_scale_inv,
    }


def mxfp4_expert_weights(experts) -> dict:
    """The four weight arguments every MXFP4 op takes, from a FusedMoE under Quark's W4A4 MXFP4 scheme."""
    return {
        "w1": experts.w13_weight,
        "w1_scale": experts.w13_weight_scale,
        "w2": experts.w2_weight,
        "w2_scale": experts.w2_weight_scale,
    }
