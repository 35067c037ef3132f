"""vLLM's fused experts on CUDA -> ``fused_moe`` (FP8, 128 x 128 block scales).

On ROCm the reference reaches vLLM's MoE through aiter's ``fused_moe`` (aklr/plugins/vllm/hook.py:
8-13, aklr/plugins/aiter/provider/moe.py:19-131); on CUDA there is no aiter, so the route stands in
for the function vLLM's opaque custom op ``vllm::outplace_fused_experts`` looks up when it runs.
"""

from __future__ import annotations

import torch

from aklr_b200.core.dispatch import FallbackReason
from aklr_b200.ops import fused_moe
from aklr_b200.plugins.vllm.hook import vllm_route

_MODULE = "vllm.model_executor.layers.fused_moe.fused_moe"

# expert maps already looked at: (address, length, tensor version) -> whether the kept experts' local
# slots are 0, 1, 2, ... in order of their global id.  The map is a long-lived tensor of the layer, so
# the one host read it costs happens on the first eager call, never inside a graph capture.
_ASCENDING_MAPS: dict[tuple, bool] = {}


def _slots_ascend(expert_map: torch.Tensor) -> bool:
    key = (expert_map.data_ptr(), expert_map.numel(), expert_map._version, str(expert_map.device))
    known = _ASCENDING_MAPS.get(key)
    if known is None:
        if expert_map.is_cuda and torch.cuda.is_current_stream_capturing():
            return False  # not seen eagerly yet: decline rather than read from the host inside a capture
        kept = expert_map[expert_map >= 0].cpu()
        known = bool(torch.equal(kept, torch.arange(kept.numel(), dtype=kept.dtype)))
        if len(_ASCENDING_MAPS) >= 256:
            _ASCENDING_MAPS.clear()
        _ASCENDING_MAPS[key] = known
    return known


@vllm_route(f"{_MODULE}.outplace_fused_experts", f"{_MODULE}.fused_experts_impl", versions=("0.22.0",))
def _fused_experts_impl(
    hidden_states,
    w1,
    w2,
    topk_weights,
    topk_ids,
    inplace,
    activation="silu",
    apply_router_weight_on_input=False,
    use_fp8_w8a8=False,
    use_int8_w8a8=False,
    use_int8_w8a16=False,
    use_int4_w4a16=False,
    ocp_mx_scheme=None,
    per_channel_quant=False,
    global_num_experts=-1,
    expert_map=None,
    w1_scale=None,
    w2_scale=None,
    w1_zp=None,
    w2_zp=None,
    a1_scale=None,
    a2_scale=None,
    block_shape=None,
    w1_bias=None,
    w2_bias=None,
):
    """FP8 experts with 128 x 128 block scales, gated SiLU, dynamic activation scales: one op call.
    Anything else is vLLM's."""
    if (
        inplace
        or not use_fp8_w8a8
        or use_int8_w8a8
        or use_int8_w8a16
        or use_int4_w4a16
        or ocp_mx_scheme is not None
        or per_channel_quant
        or apply_router_weight_on_input
        or block_shape is None
        or list(block_shape) != [128, 128]
        or any(t is not None for t in (w1_zp, w2_zp, a1_scale, a2_scale, w1_bias, w2_bias))
        or getattr(activation, "value", activation) != "silu"
    ):
        return FallbackReason.OUT_OF_CONTRACT
    expert_mask = None
    if expert_map is not None:
        # vLLM maps a global id to its local slot or -1; the op takes the 0/1 mask and numbers the
        # kept experts in order, which is the same map only when local slots ascend with the global id
        if not _slots_ascend(expert_map):
            return FallbackReason.OUT_OF_CONTRACT
        expert_mask = (expert_map >= 0).to(torch.int32)
    return fused_moe(
        hidden_states=hidden_states,
        w1=w1,
        w2=w2,
        topk_weights=topk_weights,
        topk_ids=topk_ids,
        expert_mask=expert_mask,
        activation="silu",
        quant_type="per_128x128",
        w1_scale=w1_scale,
        w2_scale=w2_scale,
    )
