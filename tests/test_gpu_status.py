"""A device-side wait that gives up: the kernel returns, the failure is recorded where the host sees
it without asking, the next call reports it, and the call after that works.

No GPU is faulted or hung here: ``aklr_selftest_wait_expiry`` waits on a barrier that nothing arrives
on with a limit of well under a millisecond and then reports exactly as a stuck pipeline would.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from aklr_b200 import workloads as wl
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

WAIT_TIMEOUT = -6  # AKLR_ERR_KERNEL_WAIT_TIMEOUT


def test_an_expired_wait_returns_and_reaches_the_next_call():
    from aklr_b200 import _lib
    from aklr_b200.moe import Routing, fused_moe_fp8, route

    lib = _lib.load()
    d = torch.device("cuda:0")
    cfg = wl.CONFIGS["deepseek_small"]
    hidden, logits, bias = (x.to(d) for x in wl.router_inputs(cfg, 37, seed=7))
    routing = Routing(cfg.topk, cfg.scoring, cfg.n_shared, cfg.num_expert_group, cfg.topk_group, True, cfg.routed_scaling_factor)
    route(logits, bias, routing)  # an eager call first: it sets up the host-visible status words
    pair = (ctypes.c_int32 * 2)()
    assert lib.aklr_device_status(pair, 1) == 0 and list(pair) == [0, 0]

    status = torch.full((2,), 123, dtype=torch.int32, device=d)
    _lib.check(lib.aklr_selftest_wait_expiry(200_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()  # the kernel came back by itself
    assert status.cpu().tolist() == [WAIT_TIMEOUT, 99]
    assert lib.aklr_device_status(pair, 0) == 0 and list(pair) == [WAIT_TIMEOUT, 99]

    # the next call of any kind launches nothing and reports the failure ...
    with pytest.raises(_lib.AklrError) as err:
        route(logits, bias, routing)
    assert err.value.code == WAIT_TIMEOUT and "location 99" in str(err.value)
    assert lib.aklr_device_status(pair, 0) == 0 and list(pair) == [0, 0]

    # ... and the one after it works, with the right answer
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed=8)
    out, ws = fused_moe_fp8(hidden, logits, bias, w1.to(d), s1.to(d), w2.to(d), s2.to(d), routing, return_workspace=True)
    ws.check_status()
    ref_ids, ref_w = orc.grouped_sigmoid_topk(logits.cpu().float(), bias.cpu().float(), cfg.topk, cfg.num_expert_group, cfg.topk_group, True, 2.5)
    ref_ids, ref_w = orc.with_shared_slot(ref_ids, ref_w, cfg.n_routed)
    assert torch.equal(ws.topk_ids().cpu().long(), ref_ids)
    gates = orc.output_gates(out.cpu(), orc.fp8_experts(hidden.cpu(), ref_ids, ref_w, w1, s1, w2, s2))
    assert orc.gates_pass(gates), gates


def test_selftest_rejects_limits_that_could_stall_a_device():
    from aklr_b200 import _lib

    lib = _lib.load()
    status = torch.zeros(2, dtype=torch.int32, device="cuda:0")
    assert lib.aklr_selftest_wait_expiry(0, status.data_ptr(), None) == -1
    assert lib.aklr_selftest_wait_expiry(5_000_000_000, status.data_ptr(), None) == -1
    assert lib.aklr_selftest_wait_expiry(1000, None, None) == -1
