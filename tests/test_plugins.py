"""Engine hooks with stand-in engines (the reference tests its hooks the same way:
tests/plugins/sglang/test_hook.py:113-260, tests/plugins/vllm/test_hook.py)."""

from __future__ import annotations

import enum
import inspect
import sys
import types
from types import SimpleNamespace

import pytest
import torch

from aklr_b200.core import dispatch as d
from aklr_b200.core.dispatch import FallbackReason
from aklr_b200.core.env import all_names


@pytest.fixture(autouse=True)
def clean_env(monkeypatch):
    for name in all_names():
        monkeypatch.delenv(name, raising=False)
    yield
    d._trace = None


# ------------------------------------------------------------------------------------------------
# sglang
# ------------------------------------------------------------------------------------------------
@pytest.fixture
def fake_sglang(monkeypatch):
    """A stand-in ``sglang.srt.plugins.hook_registry`` that records registrations."""
    registered = []

    class HookType(enum.Enum):
        AROUND = "around"
        AFTER = "after"

    class HookRegistry:
        @staticmethod
        def register(target, fn, hook_type):
            registered.append((target, fn, hook_type))

    modules = {name: types.ModuleType(name) for name in ("sglang", "sglang.srt", "sglang.srt.plugins", "sglang.srt.plugins.hook_registry", "sglang.srt.models", "sglang.srt.models.deepseek_v2", "sglang.srt.models.qwen3_moe", "sglang.srt.models.minimax_m2", "sglang.srt.models.qwen2_moe")}
    modules["sglang.srt.plugins.hook_registry"].HookRegistry = HookRegistry
    modules["sglang.srt.plugins.hook_registry"].HookType = HookType
    modules["sglang.srt.models.deepseek_v2"].DeepseekV2MoE = type("DeepseekV2MoE", (), {"forward_normal": lambda self, hidden_states: "sglang"})
    modules["sglang.srt.models.qwen3_moe"].Qwen3MoeSparseMoeBlock = type("Qwen3MoeSparseMoeBlock", (), {"forward_normal": lambda self, hidden_states: "sglang"})
    modules["sglang.srt.models.qwen2_moe"].Qwen2MoeSparseMoeBlock = type("Qwen2MoeSparseMoeBlock", (), {"_forward_router_experts": lambda self, hidden_states, *, defer_finalize=False: "sglang", "forward": lambda self, hidden_states, forward_batch=None, defer_finalize=False: "sglang"})
    modules["sglang.srt.models.minimax_m2"].MiniMaxM2MoE = type("MiniMaxM2MoE", (), {"forward_normal": lambda self, hidden_states: "sglang"})
    for name, module in modules.items():
        monkeypatch.setitem(sys.modules, name, module)
        parent, _, child = name.rpartition(".")
        if parent:
            setattr(modules[parent], child, module)
    return SimpleNamespace(registered=registered, HookType=HookType)


def test_sglang_install_hooks_only_routes_tested_on_the_installed_release(fake_sglang, monkeypatch):
    from aklr_b200.plugins.sglang import hook
    from aklr_b200.plugins.sglang.models import deepseek_v2, minimax_m2, qwen2_moe, qwen3_moe  # noqa: F401  (declare the routes)

    monkeypatch.setattr(hook, "sglang_version", lambda: "0.5.22")
    assert hook.install() == 4
    assert sorted(t for t, _, _ in fake_sglang.registered) == [
        "sglang.srt.models.minimax_m2.MiniMaxM2MoE.forward_normal",
        "sglang.srt.models.qwen2_moe.Qwen2MoeSparseMoeBlock._forward_router_experts",
        "sglang.srt.models.qwen2_moe.Qwen2MoeSparseMoeBlock.forward",
        "sglang.srt.models.qwen3_moe.Qwen3MoeSparseMoeBlock.forward_normal",
    ]
    fake_sglang.registered.clear()
    monkeypatch.setattr(hook, "sglang_version", lambda: "0.5.23")
    assert hook.install() == 5
    assert all(kind is fake_sglang.HookType.AROUND for _, _, kind in fake_sglang.registered)
    fake_sglang.registered.clear()
    monkeypatch.setattr(hook, "sglang_version", lambda: "0.9.0")
    assert hook.install() == 0


def test_sglang_around_serves_falls_back_and_skips_compiled_regions(monkeypatch, caplog):
    import logging

    from aklr_b200.plugins.sglang import hook

    served = hook.around(lambda x: x + 1, "pkg.target")
    assert served(lambda x: "orig", 1) == 2
    declined = hook.around(lambda x: FallbackReason.OUT_OF_CONTRACT, "pkg.target")
    assert declined(lambda x: "orig", 1) == "orig"
    d._trace = d.Trace("plugin")
    with caplog.at_level(logging.INFO, logger="aklr.trace.plugin"):
        declined(lambda x: "orig", 1)
        declined(lambda x: "orig", 1)
    assert len([r for r in caplog.records if r.name == "aklr.trace.plugin"]) == 1
    monkeypatch.setattr(torch.compiler, "is_compiling", lambda: True)
    assert served(lambda x: "orig", 1) == "orig"


def test_sglang_routes_take_their_targets_parameters():
    from aklr_b200.plugins.sglang.models import deepseek_v2, minimax_m2, qwen2_moe, qwen3_moe

    assert list(inspect.signature(minimax_m2._moe_forward_normal).parameters) == ["self", "hidden_states"]
    assert list(inspect.signature(qwen2_moe._forward_router_experts).parameters) == ["self", "hidden_states", "defer_finalize"]
    assert list(inspect.signature(qwen2_moe._forward).parameters) == ["self", "hidden_states", "forward_batch", "defer_finalize"]
    assert list(inspect.signature(deepseek_v2._moe_forward_normal).parameters) == [
        "self", "hidden_states", "gemm_output_zero_allocator", "input_ids", "input_ids_global",
        "skip_shared_experts", "use_vision_topk", "return_moe_output", "leave_output_sum",
    ]
    assert list(inspect.signature(qwen3_moe._moe_forward_normal).parameters) == ["self", "hidden_states"]


def test_sglang_register_starts_only_when_switched_on(fake_sglang, monkeypatch):
    from aklr_b200.plugins import sglang as plugin
    from aklr_b200.plugins.sglang import hook

    monkeypatch.setattr(hook, "sglang_version", lambda: "0.5.23")
    plugin.register()  # AKLR_SGLANG_PLUGIN unset: only the start hook
    assert [t for t, _, _ in fake_sglang.registered] == [plugin.SGLANG_HOOKED_METHOD]
    fake_sglang.registered.clear()
    monkeypatch.setenv("AKLR_SGLANG_PLUGIN", "1")
    plugin.register()
    assert len(fake_sglang.registered) == 6  # the start hook + five model routes
    monkeypatch.setenv("AKLR_SGLANG_PLUGIN", "maybe")
    with pytest.raises(SystemExit, match="cannot start"):
        plugin.register()


def _experts(**overrides):
    method_cls = type("Fp8MoEMethod", (), {})
    method = method_cls()
    method.block_quant, method.use_mxfp8, method.is_fp4_expert, method.weight_block_size = True, False, False, [128, 128]
    config = SimpleNamespace(activation="silu", is_gated=True, apply_router_weight_on_input=False, no_combine=False,
                             gemm1_alpha=None, gemm1_clamp_limit=None, swiglu_limit=None)
    method.runner = SimpleNamespace(config=config)
    experts = type("FusedMoE", (), {})()
    experts.quant_method = method
    experts.dispatcher = type("StandardDispatcher", (), {})()
    experts.reduce_results = False
    experts.w13_weight = torch.zeros(1)
    for key, value in overrides.items():
        setattr(experts, key, value)
    return experts


def test_moe_blocks_predicates(monkeypatch):
    from aklr_b200.plugins.sglang.models import moe_blocks

    monkeypatch.setattr(moe_blocks, "_on_sm100", lambda experts: True)
    good = _experts()
    assert moe_blocks.experts_format(good) == "Fp8MoEMethod"
    assert not moe_blocks.experts_fall_back(good, ("Fp8MoEMethod",))
    assert moe_blocks.experts_fall_back(good, ("QuarkW4A4MXFp4MoE",))
    assert moe_blocks.experts_fall_back(_experts(reduce_results=True), ("Fp8MoEMethod",))
    assert moe_blocks.experts_fall_back(_experts(w13_weight_bias=torch.zeros(1)), ("Fp8MoEMethod",))
    wrong_block = _experts()
    wrong_block.quant_method.weight_block_size = [64, 64]
    assert moe_blocks.experts_fall_back(wrong_block, ("Fp8MoEMethod",))
    clamped = _experts()
    clamped.quant_method.runner.config.swiglu_limit = 7.0
    assert moe_blocks.experts_fall_back(clamped, ("Fp8MoEMethod",))
    monkeypatch.setattr(moe_blocks, "_on_sm100", lambda experts: False)
    assert moe_blocks.experts_fall_back(good, ("Fp8MoEMethod",))  # not on a B200: sglang's own code

    def topk(**kw):
        base = dict(use_grouped_topk=False, custom_routing_function=None, scoring_func="softmax", correction_bias=None,
                    renormalize=True, num_fused_shared_experts=0, routed_scaling_factor=None, apply_routed_scaling_factor_on_output=False)
        return SimpleNamespace(topk_config=SimpleNamespace(**{**base, **kw}))

    assert not moe_blocks.topk_falls_back(topk(), scoring_func="softmax", biased=False)
    assert moe_blocks.topk_falls_back(topk(use_grouped_topk=True), scoring_func="softmax", biased=False)
    assert moe_blocks.topk_falls_back(topk(renormalize=False), scoring_func="softmax", biased=False)
    assert moe_blocks.topk_falls_back(topk(scoring_func="sigmoid"), scoring_func="softmax", biased=False)


def test_conditions_name_what_is_unmet(monkeypatch, caplog):
    import logging

    from aklr_b200.plugins.sglang import conditions
    from aklr_b200.plugins.sglang.models import moe_blocks

    monkeypatch.setattr(moe_blocks, "_on_sm100", lambda experts: True)
    assert moe_blocks.experts_unmet(_experts(), ("Fp8MoEMethod",)) is None
    assert moe_blocks.experts_unmet(_experts(reduce_results=True), ("Fp8MoEMethod",)) == "the ranks' sum left to the caller"
    gelu = _experts()
    gelu.quant_method.runner.config.activation = "gelu"
    assert moe_blocks.experts_unmet(gelu, ("Fp8MoEMethod",)) == "SiLU activation"
    assert "QuarkW4A4MXFp4MoE" in moe_blocks.experts_unmet(_experts(), ("QuarkW4A4MXFp4MoE",))
    assert conditions.attr(gelu, "quant_method.runner.config.activation") == "gelu"
    assert conditions.attr(gelu, "quant_method.nothing.here", 7) == 7
    with pytest.raises(AttributeError, match="nothing"):
        conditions.attr(gelu, "quant_method.nothing")
    with caplog.at_level(logging.INFO, logger=conditions.__name__):
        assert conditions.leave_to_sglang("pkg.f", "SiLU activation") is FallbackReason.OUT_OF_CONTRACT
        conditions.leave_to_sglang("pkg.f", "SiLU activation")
    assert len([r for r in caplog.records if "pkg.f stays on sglang: SiLU activation" in r.getMessage()]) == 1


def test_deepseek_route_maps_the_module_to_the_op_arguments():
    from aklr_b200.plugins.sglang.models import deepseek_v2

    bias = torch.zeros(4, dtype=torch.bfloat16)
    routing = SimpleNamespace(use_grouped_topk=True, correction_bias=bias, top_k=9, num_fused_shared_experts=1,
                              num_expert_group=8, topk_group=4, renormalize=True, scoring_func="sigmoid")
    experts = SimpleNamespace(w13_weight="w13", w13_weight_scale_inv="s13", w2_weight="w2", w2_weight_scale_inv="s2")
    mlp = SimpleNamespace(experts=experts, topk=SimpleNamespace(topk_config=routing), gate=SimpleNamespace(weight="gate"), routed_scaling_factor=2.5)
    args = deepseek_v2._moe_arguments(mlp, torch.zeros(2, 4, dtype=torch.bfloat16))
    assert args["topk"] == 8 and args["num_expert_group"] == 8 and args["topk_group"] == 4
    assert args["router_weight"] == "gate" and args["w1"] == "w13" and args["w2_scale"] == "s2"
    assert args["correction_bias"] is bias and args["routed_scaling_factor"] == 2.5
    routing.use_grouped_topk = False
    assert deepseek_v2._moe_arguments(mlp, torch.zeros(2, 4, dtype=torch.bfloat16))["num_expert_group"] == 1
    # Quark's MXFP4 experts go to the other op, with the bias as the module holds it (float32) and the e8m0 scales
    from aklr_b200 import ops

    QuarkW4A4MXFp4MoE = type("QuarkW4A4MXFp4MoE", (), {})
    bias32 = torch.zeros(4, dtype=torch.float32)
    routing.correction_bias = bias32
    mlp.experts = SimpleNamespace(scheme=QuarkW4A4MXFp4MoE(), w13_weight="w13", w13_weight_scale="e13", w2_weight="w2", w2_weight_scale="e2")
    op, args = deepseek_v2._moe_call(mlp, torch.zeros(2, 4, dtype=torch.bfloat16))
    assert op is ops.deepseek_v2_mxfp4_moe and args["correction_bias"] is bias32
    assert args["w1_scale"] == "e13" and args["w2_scale"] == "e2" and args["topk"] == 8


def test_minimax_and_qwen2_routes_pick_the_op_for_the_experts_format():
    from aklr_b200 import ops
    from aklr_b200.plugins.sglang.models import minimax_m2, qwen2_moe

    QuarkW4A4MXFp4MoE = type("QuarkW4A4MXFp4MoE", (), {})
    quark = SimpleNamespace(scheme=QuarkW4A4MXFp4MoE(), w13_weight="w13", w13_weight_scale="e13", w2_weight="w2", w2_weight_scale="e2",
                            moe_ep_rank=2, _num_local_routed=32)
    fp8 = _experts(w13_weight="w13", w13_weight_scale_inv="s13", w2_weight="w2", w2_weight_scale_inv="s2", moe_ep_rank=1, _num_local_routed=64)
    topk = SimpleNamespace(topk_config=SimpleNamespace(correction_bias="bias", top_k=8))
    gate = SimpleNamespace(weight="gate")
    op, args = minimax_m2._moe_call(SimpleNamespace(experts=quark, topk=topk, gate=gate))
    assert op is ops.minimax_m2_mxfp4_moe and args["expert_offset"] == 64 and args["w1_scale"] == "e13" and args["topk"] == 8
    op, args = minimax_m2._moe_call(SimpleNamespace(experts=fp8, topk=topk, gate=gate))
    assert op is ops.minimax_m2_fp8_moe and args["expert_offset"] == 64 and args["w2_scale"] == "s2"
    # Qwen2: the whole block's arguments, the bf16 shared expert's two weights among them
    shared = SimpleNamespace(gate_up_proj=SimpleNamespace(weight="sw1"), down_proj=SimpleNamespace(weight="sw2"))
    block = SimpleNamespace(experts=quark, shared_expert=shared, gate=gate, shared_expert_gate=SimpleNamespace(weight="sg"),
                            topk=SimpleNamespace(topk_config=SimpleNamespace(top_k=10)))
    args = qwen2_moe._block_arguments(block, "x")
    assert set(args) == {"hidden_states", "router_weight", "w1", "w1_scale", "w2", "w2_scale", "shared_w1", "shared_w2",
                         "shared_gate_weight", "topk"}
    assert args["shared_w1"] == "sw1" and args["shared_w2"] == "sw2" and args["shared_gate_weight"] == "sg" and args["topk"] == 10
    # what the shared expert has to look like, by name
    def linear(kind, **kw):
        layer = type(kind, (), {})()
        layer.quant_method, layer.bias = type("UnquantizedLinearMethod", (), {})(), None
        for k, v in kw.items():
            setattr(layer, k, v)
        return layer
    mlp = type("Qwen2MoeMLP", (), {})()
    mlp.act_fn, mlp._enable_silu_fp4_quant_fusion = type("SiluAndMul", (), {})(), False
    mlp.gate_up_proj = linear("MergedColumnParallelLinear", gather_output=False)
    mlp.down_proj = linear("RowParallelLinear", input_is_parallel=True, reduce_results=False, use_decode_attn_tp=False)
    assert qwen2_moe._shared_expert_unmet(mlp) is None
    mlp.down_proj.reduce_results = True
    assert "sum over the ranks" in qwen2_moe._shared_expert_unmet(mlp)
    mlp.down_proj.reduce_results, mlp.gate_up_proj.bias = False, torch.zeros(1)
    assert "gate_up projection a plain bf16" in qwen2_moe._shared_expert_unmet(mlp)


# ------------------------------------------------------------------------------------------------
# vLLM: against the vLLM installed in this image (0.22.0), no GPU needed
# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def vllm_fused_moe():
    try:
        from vllm.model_executor.layers.fused_moe import fused_moe
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM is not importable here: {e!r}")
    return fused_moe


def test_vllm_route_binds_validates_and_restores(vllm_fused_moe, monkeypatch):
    from aklr_b200.plugins.vllm import fused_experts, hook  # noqa: F401

    if hook.vllm_version() != "0.22.0":
        pytest.skip("the route is declared for vLLM 0.22.0")
    native = vllm_fused_moe.fused_experts_impl
    callee = "vllm.model_executor.layers.fused_moe.fused_moe.fused_experts_impl"
    try:
        assert hook.install() == [callee]
        assert vllm_fused_moe.fused_experts_impl is not native
        assert hook.original(callee) is native
        # a call the op does not take (no fp8) goes to vLLM's own function
        calls = []
        monkeypatch.setitem(hook._INSTALLED, callee, (vllm_fused_moe, "fused_experts_impl", native))
        hooked = hook._around(fused_experts._fused_experts_impl, lambda *a, **k: calls.append(a) or "vllm", callee)
        x = torch.zeros(2, 128, dtype=torch.bfloat16)
        assert hooked(x, None, None, None, None, False) == "vllm" and len(calls) == 1
    finally:
        hook.restore()
    assert vllm_fused_moe.fused_experts_impl is native


def test_vllm_route_declines_what_the_op_does_not_take():
    from aklr_b200.plugins.vllm.fused_experts import _fused_experts_impl as route

    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    assert route(x, None, None, None, None, False) is FallbackReason.OUT_OF_CONTRACT  # not fp8
    assert route(x, None, None, None, None, True, use_fp8_w8a8=True, block_shape=[128, 128]) is FallbackReason.OUT_OF_CONTRACT  # inplace
    assert route(x, None, None, None, None, False, use_fp8_w8a8=True, block_shape=[64, 64]) is FallbackReason.OUT_OF_CONTRACT
    assert route(x, None, None, None, None, False, "gelu", use_fp8_w8a8=True, block_shape=[128, 128]) is FallbackReason.OUT_OF_CONTRACT
    # in contract as far as the route can tell: the op itself answers (closed registry: no_schema)
    assert route(x, None, None, None, None, False, use_fp8_w8a8=True, block_shape=[128, 128]) in (
        FallbackReason.NO_SCHEMA, FallbackReason.OUT_OF_CONTRACT)


def test_vllm_route_takes_an_expert_map_only_when_local_slots_ascend(monkeypatch):
    """vLLM's expert_map names a local slot per global expert; the op numbers the kept experts in order of
    their global id.  The two agree only for ascending slots: any other map stays with vLLM."""
    from aklr_b200.plugins.vllm import fused_experts

    seen = {}
    monkeypatch.setattr(fused_experts, "fused_moe", lambda **kw: seen.update(kw) or "served")
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    ascending = torch.tensor([-1, 0, -1, 1, 2, -1], dtype=torch.int32)
    shuffled = torch.tensor([-1, 2, -1, 0, 1, -1], dtype=torch.int32)
    kw = dict(use_fp8_w8a8=True, block_shape=[128, 128])
    assert fused_experts._fused_experts_impl(x, None, None, None, None, False, expert_map=ascending, **kw) == "served"
    assert seen["expert_mask"].tolist() == [0, 1, 0, 1, 1, 0]
    assert fused_experts._fused_experts_impl(x, None, None, None, None, False, expert_map=shuffled, **kw) is FallbackReason.OUT_OF_CONTRACT
    shuffled.copy_(ascending)  # rewritten in place: looked at again
    assert fused_experts._fused_experts_impl(x, None, None, None, None, False, expert_map=shuffled, **kw) == "served"


def test_vllm_groups_install_together_or_not_at_all(monkeypatch):
    from aklr_b200.plugins.vllm import hook

    module = types.ModuleType("fake_vllm_mod")
    exec("def helper_a(x):\n    return 'a'\ndef helper_b(x):\n    return 'b'\ndef caller(x):\n    return helper_a(x) + helper_b(x)\n", module.__dict__)
    monkeypatch.setitem(sys.modules, "fake_vllm_mod", module)
    monkeypatch.setattr(inspect, "getsource", lambda fn: "helper_a( helper_b(")
    saved = dict(hook._ROUTES)
    hook._ROUTES.clear()
    try:
        @hook.vllm_route("fake_vllm_mod.caller", "fake_vllm_mod.helper_a", versions=("1.0",), group="g")
        def route_a(x):
            return "A"

        @hook.vllm_route("fake_vllm_mod.caller", "fake_vllm_mod.helper_b", versions=("2.0",), group="g")
        def route_b(x):
            return "B"

        monkeypatch.setattr(hook, "vllm_version", lambda: "1.0")
        assert hook.install() == []  # route_b is untested on 1.0, so its group stays out
        assert module.caller(0) == "ab"
        hook._ROUTES[route_b]["fake_vllm_mod.helper_b"] = hook._Route("fake_vllm_mod.caller", ("1.0",), "g")
        assert sorted(hook.install()) == ["fake_vllm_mod.helper_a", "fake_vllm_mod.helper_b"]
        assert module.caller(0) == "AB"
        hook.restore()
        assert module.caller(0) == "ab"

        @hook.vllm_route("fake_vllm_mod.caller", "fake_vllm_mod.helper_a", versions=("1.0",))
        def wrong_parameters(x, y):
            return "A"

        with pytest.raises(RuntimeError, match="incompatible parameters"):
            hook.install()
    finally:
        hook.restore()
        hook._ROUTES.clear()
        hook._ROUTES.update(saved)
