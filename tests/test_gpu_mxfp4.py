"""MXFP4-weight / MXFP8-activation experts on the device against the CPU oracle (itself pinned to
the reference's fused_moe / mega_moe outputs).  Gates: the float gates of the FP8 layer with the
SQNR floor the reference sets for this op family (20 dB for mega_moe, aklr/ops/mega_moe/contract.py:
140) -- measured values are far above it because the same codes are used."""

from __future__ import annotations

import pytest
import torch

from aklr_b200 import workloads as wl
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def case(hidden, inter, experts, topk, tokens, seed):
    cfg = wl.MoEConfig("mx", hidden=hidden, inter=inter, n_routed=experts, topk=topk)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)]).to(torch.int32)
    wts = torch.rand(tokens, topk, generator=g)
    return x, ids, wts, w1, s1, w2, s2


@pytest.mark.parametrize("shape", [(256, 128, 6, 2, 40), (512, 256, 8, 4, 150), (1024, 384, 4, 2, 300)])
@pytest.mark.parametrize("limit", [None, 10.0, 0.5])
def test_mxfp4_experts_match_the_oracle(shape, limit):
    from aklr_b200.moe import fused_experts_mxfp4

    hidden, inter, experts, topk, tokens = shape
    x, ids, wts, w1, s1, w2, s2 = case(hidden, inter, experts, topk, tokens, seed=tokens)
    d = dev()
    out, ws = fused_experts_mxfp4(x.to(d), ids.to(d), wts.to(d), w1.to(d), s1.to(d), w2.to(d), s2.to(d),
                                  swiglu_limit=limit, return_workspace=True)
    ws.check_status()
    ref = orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, swiglu_limit=limit, act_bits=8)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates, min_sqnr_db=30.0), gates


@pytest.mark.parametrize("shape", [(256, 128, 6, 2, 40), (512, 256, 8, 4, 150), (1024, 384, 4, 2, 300)])
def test_blocks_with_few_rows_load_only_those_rows(shape):
    """A 128-row block with at most 32 or 64 routed rows loads only those activation rows (13, 75 and
    128 + 22 rows per expert here): bit for bit the output of loading all 128."""
    from aklr_b200 import _lib
    from aklr_b200.moe import fused_experts_mxfp4

    hidden, inter, experts, topk, tokens = shape
    args = [t.to(dev()) for t in case(hidden, inter, experts, topk, tokens, seed=7 + tokens)]
    outs = []
    for variant in (0, _lib.VARIANT_FULL_ACTIVATION_BOXES):
        out, ws = fused_experts_mxfp4(*args, return_workspace=True, variant=variant)
        ws.check_status()
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("act_bits", [8, 4])
def test_first_activation_quantisation_is_bit_exact(act_bits):
    """MXFP8 (act_quant 8) and MXFP4 (act_quant 4, whose grid values are stored as e4m3 bytes): codes and scale
    bytes of the input rows reproduce the oracle's dequantised values exactly, zero rows and tiny rows included."""
    from aklr_b200.moe import fused_experts_mxfp4

    x, ids, wts, w1, s1, w2, s2 = case(256, 128, 6, 2, 40, seed=3)
    x[3] = 0
    x[5] = (x[5].float() * 2.0**-60).to(torch.bfloat16)
    x[7, :32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 4).to(torch.bfloat16)  # exact ties of the e2m1 grid
    d = dev()
    out, ws = fused_experts_mxfp4(x.to(d), ids.to(d), wts.to(d), w1.to(d), s1.to(d), w2.to(d), s2.to(d), return_workspace=True, act_bits=act_bits)
    sorted_ids = ws.sorted_ids().cpu()
    xq = ws._view(ws.layout.xq, ws.layout.capacity * 256, torch.float8_e4m3fn).view(-1, 256).cpu().float()
    sf = ws._view(ws.layout.xs, ws.layout.capacity * 8, torch.uint8).cpu()
    rows = (sorted_ids >= 0).nonzero().flatten()
    tokens = sorted_ids[rows].long() // 2
    ref = (orc.mxfp8_input if act_bits == 8 else orc.mxfp4_input)(x.float())  # dequantised
    # rebuild the dequantised rows from codes and the scale bytes in their tcgen05.cp order
    kb_count = 256 // 128
    for r, tok in zip(rows.tolist(), tokens.tolist()):
        b, rr = divmod(r, 128)
        for grp in range(256 // 32):
            kb, ks = divmod(grp, 4)
            byte = int(sf[(b * kb_count + kb) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + ks])
            got = xq[r, grp * 32 : (grp + 1) * 32] * 2.0 ** (byte - 127)
            assert torch.equal(got, ref[tok, grp * 32 : (grp + 1) * 32])


def test_mxfp4_layer_from_logits_with_deepseek_routing():
    from aklr_b200.moe import Routing, fused_moe_mxfp4

    cfg = wl.MoEConfig("mx_ds", hidden=512, inter=256, n_routed=32, topk=4, scoring="sigmoid", n_shared=1,
                       num_expert_group=4, topk_group=2, renormalize=True, routed_scaling_factor=2.5)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed=5)
    hidden, logits, bias = wl.router_inputs(cfg, 200, seed=6)
    d = dev()
    routing = Routing(cfg.topk, cfg.scoring, cfg.n_shared, cfg.num_expert_group, cfg.topk_group, True, 2.5)
    out, ws = fused_moe_mxfp4(hidden.to(d), logits.to(d), bias.to(d), w1.to(d), s1.to(d), w2.to(d), s2.to(d), routing, return_workspace=True)
    ws.check_status()
    ids, w = orc.grouped_sigmoid_topk(logits.float(), bias.float(), 4, 4, 2, True, 2.5)
    ids, w = orc.with_shared_slot(ids, w, cfg.n_routed)
    assert torch.equal(ws.topk_ids().cpu().long(), ids)
    ref = orc.mx_experts(hidden, ids, w, w1, s1, w2, s2, act_bits=8)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates, min_sqnr_db=30.0), gates


@pytest.mark.parametrize("shape", [(256, 128, 6, 2, 40), (512, 256, 8, 4, 150), (1024, 384, 4, 2, 300), (7168, 2048, 3, 2, 200)])
@pytest.mark.parametrize("limit", [None, 7.0])
def test_mxfp4_experts_with_bf16_activations_match_the_oracle(shape, limit):
    """Activations kept in bf16 (the reference's gate_mode 'interleave' and small-batch swiglu): every value enters
    the block-scaled MMAs as two e4m3 terms whose sum is the bf16 value, so the result is the oracle's over
    unquantised activations up to float32 summation order -- far inside the gates (the last shape has DeepSeek-V3's
    widths: 56 and 16 K-blocks per tile)."""
    from aklr_b200.moe import fused_experts_mxfp4

    hidden, inter, experts, topk, tokens = shape
    x, ids, wts, w1, s1, w2, s2 = case(hidden, inter, experts, topk, tokens, seed=100 + tokens)
    x = (x.float() * torch.exp2(torch.randint(-6, 7, (tokens, 1)).float())).to(torch.bfloat16)  # rows of very different size
    d = dev()
    out, ws = fused_experts_mxfp4(x.to(d), ids.to(d), wts.to(d), w1.to(d), s1.to(d), w2.to(d), s2.to(d), swiglu_limit=limit,
                                  return_workspace=True, act_bits=16)
    ws.check_status()
    ref = orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, swiglu_limit=limit, act_bits=16)
    gates = orc.output_gates(out.cpu(), ref)
    assert orc.gates_pass(gates, min_sqnr_db=40.0), gates
    rounded = orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, swiglu_limit=limit, act_bits=8)
    # and it is the unrounded statement it matches, not the MXFP8 one
    assert orc.sqnr_db(out.cpu().float(), orc.bf16_round(ref)) > orc.sqnr_db(out.cpu().float(), orc.bf16_round(rounded)) + 6.0


@pytest.mark.parametrize("shape", [(256, 128, 6, 2, 40), (512, 256, 8, 4, 150), (1024, 384, 4, 2, 300)])
def test_mxfp4_experts_with_mxfp4_activations_match_the_oracle(shape):
    """The reference op's default: activations and the gated product quantised to MXFP4 (act_quant 4).  The same
    codes as the oracle except where the second quantisation sits on a tie (a grid step there is a quarter of the
    value), so the SQNR floor is the reference's own for this format family, 13 dB (aklr/ops/fused_moe/contract.py),
    with the measured value far above it."""
    from aklr_b200.moe import fused_experts_mxfp4

    hidden, inter, experts, topk, tokens = shape
    x, ids, wts, w1, s1, w2, s2 = case(hidden, inter, experts, topk, tokens, seed=200 + tokens)
    d = dev()
    out, ws = fused_experts_mxfp4(x.to(d), ids.to(d), wts.to(d), w1.to(d), s1.to(d), w2.to(d), s2.to(d), return_workspace=True, act_bits=4)
    ws.check_status()
    ref = orc.mx_experts(x, ids.long(), wts, w1, s1, w2, s2, act_bits=4)
    gates = orc.output_gates(out.cpu(), ref)
    assert gates["sqnr_db"] >= 25.0 and gates["cosine"] >= 0.998, gates

