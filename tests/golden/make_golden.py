"""Writes the golden vectors under tests/golden/ by running the REFERENCE's own functions.

Run only where the reference project is importable (``--reference <its root>``); the
fixtures it writes are committed, so tests never need the reference at run time:

    python tests/golden/make_golden.py --reference /path/to/reference

Inputs are regenerated from seeds by ``aklr_b200.workloads`` (their SHA-256 is stored and
re-checked by the tests, so an RNG drift shows up as a fixture mismatch, not as a parity
failure); outputs of the reference functions are stored whole.
"""

from __future__ import annotations

import argparse
import pathlib
import sys
from types import SimpleNamespace

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from aklr_b200 import workloads as wl  # noqa: E402
from oracle.moe_oracle import sha256_of  # noqa: E402
from tests.golden import cases  # noqa: E402

FP8_DTYPES = {
    "hidden_states": "bfloat16",
    "router_weight": "bfloat16",
    "correction_bias": "bfloat16",
    "w1": "float8_e4m3fn",
    "w1_scale": "float32",
    "w2": "float8_e4m3fn",
    "w2_scale": "float32",
}


def f32(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.float32).contiguous().numpy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True

    from aklr.ops.fused_moe.reference import _mxfp4, _mxfp8, fused_moe_reference
    from aklr.ops.mega_moe.reference import mega_moe_reference
    from aklr.ops.quant.reference import per_group_quant_fp8_reference, per_group_quant_mxfp8_reference
    from aklr.ops.topk.reference import biased_grouped_topk_reference
    from aklr.plugins.sglang.models.deepseek_v2 import reference as ds
    from aklr.plugins.sglang.models.qwen3_moe import reference as qw

    torch.set_num_threads(1)  # one accumulation order for the stored float outputs
    out: dict[str, np.ndarray] = {}
    meta: dict[str, str] = {}

    # ---- the exact sigmoid bits of the reference's runtime over every bf16 value ---------
    every_bf16 = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    meta["sigmoid_table_sha256"] = sha256_of(torch.sigmoid(every_bf16))

    # ---- layer: tiny softmax config through the router GEMM -----------------------------
    cfg, rargs = cases.tiny_layer()
    hidden = rargs["hidden_states"]
    point = SimpleNamespace(dtypes=FP8_DTYPES, attrs={"topk": cfg.topk}, axes={})
    logits = qw._router_logits(point, rargs)
    weights, ids = qw._routed(logits, cfg.topk)
    out["tiny.logits"], out["tiny.ids"], out["tiny.weights"] = f32(logits), ids.numpy(), f32(weights)
    out["tiny.out"] = f32(qw.qwen3_moe_fp8_moe_reference(point, rargs))
    out["tiny.fp8_input"] = f32(qw._fp8_input(hidden.float()))
    for k, v in rargs.items():
        meta[f"tiny.{k}"] = sha256_of(v)

    # ---- layer: DeepSeek routing on a small layer ---------------------------------------
    cfg, rargs = cases.ds_small_layer()
    hidden, rw, bias = rargs["hidden_states"], rargs["router_weight"], rargs["correction_bias"]
    point = SimpleNamespace(
        dtypes=FP8_DTYPES,
        attrs={
            "topk": cfg.topk,
            "num_expert_group": cfg.num_expert_group,
            "topk_group": cfg.topk_group,
            "renormalize": True,
        },
        axes={"n_routed": cfg.n_routed},
    )
    logits = ds.rounded_to_bfloat16(hidden.float() @ rw.float().T)
    ids, weights = ds._grouped_routed(point, rargs, logits, bias.float())
    ids, weights = ds._with_shared_slot(point, ids, weights)
    out["ds_small.logits"], out["ds_small.ids"], out["ds_small.weights"] = f32(logits), ids.numpy(), f32(weights)
    out["ds_small.out"] = f32(ds.deepseek_v2_fp8_moe_reference(point, rargs))
    for k, v in rargs.items():
        if isinstance(v, torch.Tensor):
            meta[f"ds_small.{k}"] = sha256_of(v)

    # ---- layer: DeepSeek routing without groups over MXFP4 experts, activations not quantised ----------
    cfg, rargs = cases.ds_mx_layer()
    point = SimpleNamespace(
        dtypes={"hidden_states": "bfloat16", "router_weight": "bfloat16", "correction_bias": "float32", "w1": "float4_e2m1",
                "w1_scale": "float8_e8m0", "w2": "float4_e2m1", "w2_scale": "float8_e8m0"},
        attrs={"topk": cfg.topk, "num_expert_group": 1, "topk_group": 1, "renormalize": True},
        axes={"n_routed": cfg.n_routed},
    )
    out["ds_mx.out"] = f32(ds.deepseek_v2_mxfp4_moe_reference(point, rargs))
    for k, v in rargs.items():
        if isinstance(v, torch.Tensor):
            meta[f"ds_mx.{k}"] = sha256_of(v)

    # ---- layer: MiniMax-M2 (float32 gate, plain biased top-k, this rank holds 8 of 16 experts) ----
    from aklr.plugins.sglang.models.minimax_m2 import reference as mm

    cfg, rargs = cases.minimax_layer()
    point = SimpleNamespace(
        dtypes={**FP8_DTYPES, "router_weight": "float32", "correction_bias": "float32"},
        attrs={"topk": cfg.topk},
        axes={"n_experts": cfg.n_routed},
    )
    x32 = rargs["hidden_states"].float()
    ids, weights = mm._routed(point, x32, rargs["router_weight"], rargs["correction_bias"])
    out["minimax.ids"], out["minimax.weights"] = ids.numpy(), f32(weights)
    out["minimax.out"] = f32(mm.minimax_m2_fp8_moe_reference(point, rargs))
    for k, v in rargs.items():
        if isinstance(v, torch.Tensor):
            meta[f"minimax.{k}"] = sha256_of(v)

    # ---- layer: Qwen2-MoE (softmax top-k + shared expert gated by sigmoid(x . g)) ---------------
    from aklr.plugins.sglang.models.qwen2_moe import reference as q2

    cfg, rargs = cases.qwen2_layer()
    point = SimpleNamespace(
        dtypes={**FP8_DTYPES, "shared_gate_weight": "bfloat16", "topk_weights": "float32", "topk_ids": "int32"},
        attrs={"topk": cfg.topk},
        axes={"n_routed": cfg.n_routed, "n_experts": cfg.n_routed + 1, "topk": cfg.topk},
    )
    weights, ids = q2.qwen2_moe_router_reference(point, rargs)
    out["qwen2.ids"], out["qwen2.weights"] = ids.numpy(), f32(weights)
    out["qwen2.out"] = f32(q2.qwen2_moe_fp8_router_experts_reference(point, rargs))
    out["qwen2.experts_out"] = f32(q2.qwen2_moe_fp8_experts_reference(point, {**rargs, "topk_weights": weights, "topk_ids": ids}))
    for k, v in rargs.items():
        meta[f"qwen2.{k}"] = sha256_of(v)

    # ---- layers over MXFP4 experts with unquantised activations: MiniMax-M2 and Qwen2-MoE (bf16 shared expert apart)
    mx_dtypes = {"hidden_states": "bfloat16", "w1": "float4_e2m1", "w1_scale": "float8_e8m0", "w2": "float4_e2m1",
                 "w2_scale": "float8_e8m0"}
    cfg, rargs = cases.minimax_mx_layer()
    point = SimpleNamespace(
        dtypes={**mx_dtypes, "router_weight": "float32", "correction_bias": "float32"},
        attrs={"topk": cfg.topk},
        axes={"n_experts": cfg.n_routed},
    )
    out["minimax_mx.out"] = f32(mm.minimax_m2_mxfp4_moe_reference(point, rargs))
    for k, v in rargs.items():
        if isinstance(v, torch.Tensor):
            meta[f"minimax_mx.{k}"] = sha256_of(v)
    cfg, rargs = cases.qwen2_mx_layer()
    point = SimpleNamespace(
        dtypes={**mx_dtypes, "router_weight": "bfloat16", "shared_w1": "bfloat16", "shared_w2": "bfloat16",
                "shared_gate_weight": "bfloat16"},
        attrs={"topk": cfg.topk},
        axes={"n_routed": cfg.n_routed},
    )
    out["qwen2_mx.out"] = f32(q2.qwen2_moe_mxfp4_moe_reference(point, rargs))
    for k, v in rargs.items():
        meta[f"qwen2_mx.{k}"] = sha256_of(v)

    # ---- routing only, at the full expert counts -----------------------------------------
    logits, bias = cases.route_ds()
    point = SimpleNamespace(
        attrs={"topk": 8, "num_expert_group": 8, "topk_group": 4, "renormalize": True},
        axes={"n_routed": 256},
    )
    ids, weights = ds._grouped_routed(point, {"routed_scaling_factor": 2.5}, logits.float(), bias.float())
    out["route_ds.ids"], out["route_ds.weights"] = ids.numpy(), f32(weights)
    meta["route_ds.logits"], meta["route_ds.bias"] = sha256_of(logits), sha256_of(bias)
    point.attrs["renormalize"] = False
    ids, weights = ds._grouped_routed(point, {"routed_scaling_factor": 1.0}, logits.float(), bias.float())
    out["route_ds_norenorm.ids"], out["route_ds_norenorm.weights"] = ids.numpy(), f32(weights)
    # heavy ties: logits drawn from 5 distinct values, zero bias
    tied = cases.route_tied()
    point.attrs["renormalize"] = True
    ids, weights = ds._grouped_routed(point, {"routed_scaling_factor": 2.5}, tied.float(), torch.zeros(256))
    out["route_tied.ids"], out["route_tied.weights"] = ids.numpy(), f32(weights)
    meta["route_tied.logits"] = sha256_of(tied)

    qcfg, logits = cases.route_qwen3()
    weights, ids = qw._routed(logits.float(), qcfg.topk)
    out["route_qwen3.ids"], out["route_qwen3.weights"] = ids.numpy(), f32(weights)
    meta["route_qwen3.logits"] = sha256_of(logits)
    weights, ids = qw._routed(tied[:, :128].float(), 8)
    out["route_tied_softmax.ids"], out["route_tied_softmax.weights"] = ids.numpy(), f32(weights)

    # ---- standalone routing op ------------------------------------------------------------
    logits, bias = cases.bgt()
    point = SimpleNamespace(
        dtypes={"router_logits": "bfloat16", "correction_bias": "bfloat16", "topk_ids": "int32"},
        axes={"topk": 8},
        attrs={"renormalize": True},
    )
    weights, ids = biased_grouped_topk_reference(
        point, {"router_logits": logits, "correction_bias": bias, "routed_scaling_factor": 2.5}
    )
    out["bgt.ids"], out["bgt.weights"] = ids.numpy(), f32(weights)
    meta["bgt.logits"], meta["bgt.bias"] = sha256_of(logits), sha256_of(bias)

    # ---- standalone quant ops ----------------------------------------------------------------
    x = cases.quant_x()
    point = SimpleNamespace(dtypes={"x": "bfloat16", "scales": "uint8"})
    q, s = per_group_quant_fp8_reference(point, {"x": x})
    out["quant_fp8.q"], out["quant_fp8.s"] = f32(q), f32(s)
    q, s = per_group_quant_mxfp8_reference(point, {"x": x})
    out["quant_mxfp8.q"], out["quant_mxfp8.s"] = f32(q), s.view(torch.uint8).numpy()
    out["mxfp8_input"] = f32(_mxfp8(x.float()))
    grid = torch.tensor((0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0))
    out["mxfp4_input"] = f32(_mxfp4(x.float(), grid))
    meta["quant.x"] = sha256_of(x)

    # ---- MXFP4 experts given routing (fused_moe, act_quant 8) and the EP statement ----------
    rargs, group = cases.mega_group()
    point = SimpleNamespace(
        dtypes={"hidden_states": "bfloat16", "topk_weights": "float32"},
        attrs={
            "has_expert_mask": False,
            "has_num_local_tokens": False,
            "activation": "silu",
            "doweight_stage1": False,
            "gate_mode": "separated",
            "act_quant": 8,
        },
        axes={"n_tokens": 12},
    )
    out["mx_moe.out"] = f32(fused_moe_reference(point, rargs))
    point.attrs["act_quant"] = 4
    out["mx_moe_a4.out"] = f32(fused_moe_reference(point, rargs))
    for k, v in rargs.items():
        meta[f"mx_moe.{k}"] = sha256_of(v)
    # the op's other attributes at act_quant 8: activations, stage-1 weighting, rows not received
    for name, vargs, vattrs, _ in cases.mx_variants():
        point.attrs.update({"act_quant": 8, "activation": "silu", "doweight_stage1": False, "has_expert_mask": False,
                            "has_num_local_tokens": False, "gate_mode": "separated", **vattrs})
        point.axes["n_tokens"] = vargs["hidden_states"].shape[0]
        out[f"mx_moe_{name}.out"] = f32(fused_moe_reference(point, vargs))
        for k, v in vargs.items():
            if torch.is_tensor(v):
                meta[f"mx_moe_{name}.{k}"] = sha256_of(v)
    # two ranks, 3 experts each: global expert e = local e % 3 of rank e // 3
    point = SimpleNamespace(
        dtypes={"hidden_states": "bfloat16", "topk_weights": "float32"}, axes={"n_experts": 3}
    )
    for r in range(2):
        out[f"mega.rank{r}.out"] = f32(mega_moe_reference(point, group, r))

    np.savez_compressed(HERE / "moe_golden.npz", **out)
    with open(HERE / "moe_golden_inputs.sha256", "w") as fh:
        for k in sorted(meta):
            fh.write(f"{meta[k]}  {k}\n")
    print("wrote", len(out), "arrays,", len(meta), "hashes")


if __name__ == "__main__":
    main()
