"""The contract/dispatch layer on CPU with a pure-Python stand-in kernel (the reference tests its
registry the same way: tests/core/runtime/test_dispatch.py with a fake `run`)."""

from __future__ import annotations

import inspect
import json
import logging

import pytest
import torch

from aklr_b200.core import dispatch as d
from aklr_b200.core.env import RuntimeEnv, all_names


@pytest.fixture(autouse=True)
def clean_env(monkeypatch):
    for name in all_names():
        monkeypatch.delenv(name, raising=False)
    yield
    d._trace = None


def make_contract(contract_id="toy_gemm@1.0"):
    def key(call):
        a, b = call["a"], call["b"]
        if not (isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor)) or a.dim() != 2 or a.shape[1] != b.shape[1]:
            return None
        return (a.shape[1], str(a.dtype))

    return d.OpContract(
        contract_id=contract_id,
        params=[d.Param("a"), d.Param("b"), d.Param("scale", 1.0)],
        outputs=["out"],
        key=key,
        alloc=lambda call, k: torch.empty(call["a"].shape[0], call["b"].shape[0]),
        run=lambda call, out: out.copy_(call["a"] @ call["b"].mT * call["scale"]),
    )


def make_api(contract):
    dispatcher = d.KernelDispatcher(contract)

    def toy_gemm(a, b, scale=1.0): ...

    return dispatcher, dispatcher.make_api_fn(toy_gemm)


def test_closed_dispatcher_returns_no_schema():
    _, fn = make_api(make_contract())
    assert fn(torch.ones(2, 3), torch.ones(4, 3)) is d.FallbackReason.NO_SCHEMA


def test_open_dispatcher_serves_and_keeps_the_signature():
    dispatcher, fn = make_api(make_contract())
    dispatcher.open()
    out = fn(torch.ones(2, 3), torch.ones(4, 3), scale=2.0)
    assert torch.equal(out, torch.full((2, 4), 6.0))
    assert list(inspect.signature(fn).parameters) == ["a", "b", "scale"]
    assert fn.fallback_reason(torch.ones(2, 3), torch.ones(4, 3)) is None
    assert fn.serving(torch.ones(2, 3), torch.ones(4, 3)).arch == "sm_100a"
    assert (3, "torch.float32") in dispatcher.warmed_keys


def test_out_of_contract_call_falls_back_without_raising():
    dispatcher, fn = make_api(make_contract())
    dispatcher.open()
    assert fn(torch.ones(2, 3), torch.ones(4, 5)) is d.FallbackReason.OUT_OF_CONTRACT
    assert fn.fallback_reason(torch.ones(2, 3), torch.ones(4, 5)) is d.FallbackReason.OUT_OF_CONTRACT


def test_kernel_errors_are_raised_not_swallowed(caplog):
    contract = make_contract()
    contract.run = lambda call, out: (_ for _ in ()).throw(RuntimeError("boom"))
    dispatcher, fn = make_api(contract)
    dispatcher.open()
    with caplog.at_level(logging.ERROR), pytest.raises(RuntimeError, match="boom"):
        fn(torch.ones(2, 3), torch.ones(4, 3))
    assert "AKLR_DISABLE=toy_gemm@1.0" in caplog.text


def test_api_signature_must_match_the_contract():
    dispatcher = d.KernelDispatcher(make_contract())

    def wrong(a, b, factor=1.0): ...

    with pytest.raises(TypeError, match="takes"):
        dispatcher.make_api_fn(wrong)

    def wrong_default(a, b, scale=2.0): ...

    with pytest.raises(TypeError, match="default"):
        dispatcher.make_api_fn(wrong_default)


def test_registry_disable_all_closes_every_op(monkeypatch):
    registry = d.DispatcherRegistry()
    dispatcher = registry.dispatcher(make_contract())
    monkeypatch.setenv("AKLR_DISABLE", "1")
    registry.init()
    assert registry.is_initialized
    assert dispatcher.dispatch({"a": torch.ones(1, 1), "b": torch.ones(1, 1), "scale": 1.0}) is d.FallbackReason.DISABLED


def test_registry_needs_a_gpu_unless_disabled():
    if torch.cuda.is_available():
        pytest.skip("checks the no-GPU start")
    registry = d.DispatcherRegistry()
    registry.dispatcher(make_contract())
    with pytest.raises(d.LoadError, match="no GPU visible"):
        registry.init()


def test_registry_refuses_two_contracts_with_one_id():
    registry = d.DispatcherRegistry()
    registry.dispatcher(make_contract())
    with pytest.raises(ValueError, match="already has this id"):
        registry.dispatcher(make_contract())


def test_bad_environment_values_name_their_variable(monkeypatch):
    monkeypatch.setenv("AKLR_SGLANG_PLUGIN", "yes")
    with pytest.raises(ValueError, match="AKLR_SGLANG_PLUGIN"):
        RuntimeEnv()
    monkeypatch.delenv("AKLR_SGLANG_PLUGIN")
    monkeypatch.setenv("AKLR_TRACE", "verbose")
    with pytest.raises(ValueError, match="AKLR_TRACE"):
        RuntimeEnv()
    monkeypatch.setenv("AKLR_TRACE", "op")
    monkeypatch.setenv("AKLR_DISABLE", "fused_moe@1.0, topk@1.0")
    env = RuntimeEnv()
    assert env.disabled_contracts == {"fused_moe@1.0", "topk@1.0"} and not env.is_all_disabled


def test_trace_logs_each_distinct_dispatch_once(caplog):
    dispatcher, fn = make_api(make_contract())
    dispatcher.open()
    d._trace = d.Trace("op")
    with caplog.at_level(logging.INFO, logger="aklr.trace.op"):
        for _ in range(3):
            fn(torch.ones(2, 3), torch.ones(4, 3))
        fn(torch.ones(2, 3), torch.ones(4, 5))
    lines = [r.getMessage() for r in caplog.records if r.name == "aklr.trace.op"]
    assert len(lines) == 2 and "served" in lines[0] and "out_of_contract" in lines[1]


def test_recorder_counts_calls_and_fallbacks(tmp_path):
    dispatcher, fn = make_api(make_contract())
    recorder = d.CallRecorder(str(tmp_path))
    dispatcher.open(recorder)
    fn(torch.ones(2, 3), torch.ones(4, 3))
    fn(torch.ones(5, 3), torch.ones(4, 3))
    fn(torch.ones(2, 3), torch.ones(4, 5))
    rows = [json.loads(line) for line in open(recorder.save())]
    assert {(r["fallback"], r["calls"]) for r in rows} == {(None, 2), ("out_of_contract", 1)}


def test_concurrent_init_once_initialises_once(monkeypatch):
    import threading

    registry = d.DispatcherRegistry()
    registry.dispatcher(make_contract())
    monkeypatch.setenv("AKLR_DISABLE", "1")
    calls = []
    original = registry.init
    monkeypatch.setattr(registry, "init", lambda: (calls.append(1), original()))
    threads = [threading.Thread(target=registry.init_once) for _ in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert len(calls) == 1


def test_real_ops_keep_the_reference_signatures():
    from aklr_b200 import ops

    assert list(inspect.signature(ops.deepseek_v2_fp8_moe).parameters) == [
        "hidden_states", "router_weight", "correction_bias", "w1", "w1_scale", "w2", "w2_scale", "topk",
        "num_expert_group", "topk_group", "renormalize", "scoring_func", "routed_scaling_factor",
    ]
    assert list(inspect.signature(ops.qwen3_moe_fp8_moe).parameters)[-1] == "topk"
    assert inspect.signature(ops.qwen3_moe_fp8_moe).parameters["topk"].default == 8
    params = inspect.signature(ops.fused_moe).parameters
    assert list(params)[:5] == ["hidden_states", "w1", "w2", "topk_weights", "topk_ids"]
    assert params["act_quant"].default == 4 and params["out"].default is None
    assert list(inspect.signature(ops.biased_grouped_topk).parameters)[-1] == "routed_scaling_factor"


def test_real_ops_decline_cpu_tensors_instead_of_computing():
    """No CPU path: with the dispatcher open, host tensors are out of contract."""
    from aklr_b200 import ops

    dispatcher = d.DispatcherRegistry.default().dispatcher(ops.PER_GROUP_QUANT_FP8)
    was_open = dispatcher.is_open
    dispatcher.open()
    try:
        assert ops.per_group_quant_fp8(torch.zeros(4, 128, dtype=torch.bfloat16)) is d.FallbackReason.OUT_OF_CONTRACT
    finally:
        if not was_open:
            dispatcher.close(d.FallbackReason.NO_SCHEMA)


def test_an_op_whose_run_reads_the_host_is_not_served_inside_a_capture(monkeypatch):
    """``capturable=False`` (mega_moe: split sizes of the uneven all-to-all are read on the host): inside a
    CUDA-graph capture the api returns a FallbackReason instead of breaking the capture, warm key or not."""
    contract = make_contract()
    contract.capturable = False
    dispatcher, fn = make_api(contract)
    dispatcher.open()
    a, b = torch.ones(2, 3), torch.ones(4, 3)
    assert torch.equal(fn(a, b), torch.full((2, 4), 3.0))  # eager: served, and the key is warm now
    monkeypatch.setattr(d, "_is_capturing", lambda: True)
    assert fn(a, b) is d.FallbackReason.OUT_OF_CONTRACT
    assert fn.fallback_reason(a, b) is d.FallbackReason.OUT_OF_CONTRACT
    capturable, fn2 = make_api(make_contract("toy_gemm2@1.0"))
    capturable.open()
    assert fn2(a, b) is d.FallbackReason.NOT_WARMED  # an ordinary op: only its first sight inside a capture falls back
    monkeypatch.setattr(d, "_is_capturing", lambda: False)
    fn2(a, b)
    monkeypatch.setattr(d, "_is_capturing", lambda: True)
    assert torch.equal(fn2(a, b), torch.full((2, 4), 3.0))


def test_mega_moe_declares_that_it_cannot_be_captured():
    from aklr_b200 import ops

    assert ops.MEGA_MOE.capturable is False
    assert all(c.capturable for c in (ops.FUSED_MOE, ops.BIASED_GROUPED_TOPK))



def test_tile_contiguous_layout_round_trips_on_the_host():
    """from_b200_tiled undoes the layout [.., rows/128, cols/128, 128, 128] (the converter itself is a device kernel)."""
    import torch

    from aklr_b200 import layouts

    w = torch.arange(2 * 256 * 384, dtype=torch.int64).remainder(251).to(torch.uint8).reshape(2, 256, 384)
    tiled = w.reshape(2, 2, 128, 3, 128).permute(0, 1, 3, 2, 4).contiguous().reshape(2, 256, 384)
    assert torch.equal(layouts.from_b200_tiled(tiled), w)
    assert not layouts.is_b200_tiled(w)
    import pytest

    with pytest.raises(ValueError, match="CUDA"):
        layouts.to_b200_tiled(w)
