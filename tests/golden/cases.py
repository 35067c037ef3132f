"""Seeded inputs of the golden cases, shared by the fixture writer and the tests."""

from __future__ import annotations

import torch

from aklr_b200 import workloads as wl

ROUTE_SHAPE = wl.MoEConfig("route256", 128, 128, 256, 8, "sigmoid")


def tiny_layer():
    cfg, seed, tokens = wl.CONFIGS["tiny"], 1234, 64
    hidden, _, _ = wl.router_inputs(cfg, tokens, seed)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed)
    return cfg, dict(
        hidden_states=hidden, router_weight=wl.router_weight(cfg, seed), w1=w1, w1_scale=s1, w2=w2, w2_scale=s2
    )


def ds_small_layer():
    cfg, seed, tokens = wl.CONFIGS["deepseek_small"], 4321, 48
    hidden, _, bias = wl.router_inputs(cfg, tokens, seed)
    # x40 spreads the logits so the sigmoid scores are not all near 0.5
    rw = (wl.router_weight(cfg, seed) * 40).to(torch.bfloat16)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed)
    return cfg, dict(
        hidden_states=hidden,
        router_weight=rw,
        correction_bias=bias,
        w1=w1,
        w1_scale=s1,
        w2=w2,
        w2_scale=s2,
        routed_scaling_factor=cfg.routed_scaling_factor,
    )


def minimax_layer():
    """MiniMax-M2-style layer: float32 gate over 16 routed experts, this rank holds experts 4..11."""
    cfg, seed, tokens = wl.MoEConfig("minimax_small", hidden=256, inter=128, n_routed=8, topk=4, scoring="sigmoid"), 2468, 40
    n_routed, offset = 16, 4
    hidden, _, _ = wl.router_inputs(cfg, tokens, seed)
    g = torch.Generator().manual_seed(seed + 5)
    router = torch.randn(n_routed, cfg.hidden, generator=g) * (3.0 / cfg.hidden**0.5)
    bias = 8.0 + 0.02 * torch.randn(n_routed, generator=g)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed)
    return cfg, dict(
        hidden_states=hidden, router_weight=router, correction_bias=bias, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2,
        expert_offset=offset,
    )


def qwen2_layer():
    """Qwen2-MoE-style layer: 12 routed experts, top-4 softmax, a gated shared expert in the last slot."""
    cfg, seed, tokens = wl.MoEConfig("qwen2_small", hidden=256, inter=128, n_routed=12, topk=4, n_shared=1), 1357, 36
    hidden, _, _ = wl.router_inputs(cfg, tokens, seed)
    g = torch.Generator().manual_seed(seed + 3)
    rw = (wl.router_weight(cfg, seed) * 30).to(torch.bfloat16)
    gate = (torch.randn(1, cfg.hidden, generator=g) * (2.0 / cfg.hidden**0.5)).to(torch.bfloat16)
    w1, s1, w2, s2 = wl.expert_weights(cfg, seed)
    return cfg, dict(hidden_states=hidden, router_weight=rw, shared_gate_weight=gate, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2)


def ds_mx_layer():
    """deepseek_v2_mxfp4_moe: ungrouped sigmoid routing with a float32 bias near 8 (the contract's spread), 16 routed
    MXFP4 experts + the shared one, unquantised activations."""
    cfg = wl.MoEConfig("ds_mx", hidden=256, inter=256, n_routed=16, topk=4, scoring="sigmoid", n_shared=1, routed_scaling_factor=2.5)
    seed, tokens = 977, 40
    hidden = wl.normal(seed, "hidden", (tokens, cfg.hidden), 1.0, dtype=torch.bfloat16)
    rw = (wl.router_weight(cfg, seed) * 40).to(torch.bfloat16)
    bias = 8.0 + wl.normal(seed, "bias", (cfg.n_routed,), 0.05)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed)
    return cfg, dict(hidden_states=hidden, router_weight=rw, correction_bias=bias, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2,
                     routed_scaling_factor=2.5)


def minimax_mx_layer():
    """minimax_m2_mxfp4_moe: float32 gate over 16 routed experts, this rank holds the MXFP4 experts 4..11."""
    cfg = wl.MoEConfig("minimax_mx", hidden=256, inter=256, n_routed=8, topk=4, scoring="sigmoid")
    seed, tokens, n_routed, offset = 8642, 40, 16, 4
    hidden = wl.normal(seed, "hidden", (tokens, cfg.hidden), 1.0, dtype=torch.bfloat16)
    router = wl.normal(seed, "router", (n_routed, cfg.hidden), 3.0 / cfg.hidden**0.5)
    bias = 8.0 + wl.normal(seed, "bias", (n_routed,), 0.02)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed)
    return cfg, dict(hidden_states=hidden, router_weight=router, correction_bias=bias, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2,
                     expert_offset=offset)


def qwen2_mx_layer():
    """qwen2_moe_mxfp4_moe: 12 routed MXFP4 experts, top-4 softmax, a bf16 shared expert (inter 384) apart from them,
    its down projection drawn 8 times a Lecun normal's spread as the reference's contract draws it."""
    cfg = wl.MoEConfig("qwen2_mx", hidden=256, inter=256, n_routed=12, topk=4)
    seed, tokens, shared_inter = 7531, 36, 384
    hidden = wl.normal(seed, "hidden", (tokens, cfg.hidden), 1.0, dtype=torch.bfloat16)
    rw = (wl.router_weight(cfg, seed) * 30).to(torch.bfloat16)
    gate = wl.normal(seed, "shared_gate", (1, cfg.hidden), 2.0 / cfg.hidden**0.5, dtype=torch.bfloat16)
    sw1 = wl.normal(seed, "shared_w1", (2 * shared_inter, cfg.hidden), cfg.hidden**-0.5, dtype=torch.bfloat16)
    sw2 = wl.normal(seed, "shared_w2", (cfg.hidden, shared_inter), 8.0 * shared_inter**-0.5, dtype=torch.bfloat16)
    w1, s1, w2, s2 = wl.mx_expert_weights(cfg, seed)
    return cfg, dict(hidden_states=hidden, router_weight=rw, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2, shared_w1=sw1,
                     shared_w2=sw2, shared_gate_weight=gate)


def route_ds():
    _, logits, bias = wl.router_inputs(ROUTE_SHAPE, 192, 77)
    return logits, bias


def route_tied():
    """Heavy ties: logits take 5 distinct values."""
    g = torch.Generator().manual_seed(5)
    return (torch.randint(0, 5, (64, 256), generator=g).float() * 0.5 - 1.0).to(torch.bfloat16)


def route_qwen3():
    cfg = wl.CONFIGS["qwen3"]
    _, logits, _ = wl.router_inputs(cfg, 160, 99)
    return cfg, logits


def bgt():
    _, logits, bias = wl.router_inputs(ROUTE_SHAPE, 96, 78)
    return logits, bias


def quant_x():
    x = wl.normal(31, "quant.x", (24, 512), 1.0, dtype=torch.bfloat16)
    x[3] = 0  # an all-zero row: the amax floor
    x[5, :128] *= 1e-30
    return x


def mx_case(seed: int, tokens: int = 12, hidden: int = 128, inter: int = 64, experts: int = 6, topk: int = 2):
    """Random MXFP4 expert weights (random nibbles, e8m0 exponents 118..123) + routing."""
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(tokens, hidden, generator=g)).to(torch.bfloat16)
    w1 = torch.randint(0, 256, (experts, 2 * inter, hidden // 2), generator=g, dtype=torch.uint8)
    w2 = torch.randint(0, 256, (experts, hidden, inter // 2), generator=g, dtype=torch.uint8)
    s1 = torch.randint(118, 124, (experts, 2 * inter, hidden // 32), generator=g, dtype=torch.uint8)
    s2 = torch.randint(118, 124, (experts, hidden, inter // 32), generator=g, dtype=torch.uint8)
    ids = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)]).to(torch.int32)
    wts = torch.rand(tokens, topk, generator=g)
    return dict(hidden_states=x, w1=w1, w1_scale=s1, w2=w2, w2_scale=s2, topk_ids=ids, topk_weights=wts)


def mx_variants():
    """The other attributes of the experts-only op, one case each: (name, inputs, reference attrs, oracle
    keywords).  gpt-oss's swiglu has 256 tokens: below that the reference leaves activations unquantised."""
    mask = torch.tensor([1, 0, 1, 1, 0, 1], dtype=torch.int32)
    local = mx_case(13)
    held = {k: local[k][:4] for k in ("w1", "w1_scale", "w2", "w2_scale")}
    return [
        ("gelu", mx_case(11), {"activation": "gelu"}, {"activation": "gelu"}),
        ("swiglu", {**mx_case(12, tokens=256), "swiglu_limit": 7.0}, {"activation": "swiglu"},
         {"activation": "swiglu", "swiglu_limit": 7.0}),
        ("situv2", {**mx_case(14), "beta": 3.0, "linear_beta": 5.0}, {"activation": "situv2"},
         {"activation": "situv2", "beta": 3.0, "linear_beta": 5.0}),
        ("stage1", mx_case(15), {"doweight_stage1": True}, {"weight_in_stage1": True}),
        ("local", {**local, **held, "expert_mask": mask, "num_local_tokens": torch.tensor([9], dtype=torch.int32)},
         {"has_expert_mask": True, "has_num_local_tokens": True}, {"num_local_tokens": 9}),
        # activations kept in bf16: DeepSeek-V4's clamped SwiGLU (gate_mode 'interleave', with the expert mask and
        # the rows-received bound its published workload has), and gpt-oss swiglu below 256 rows
        ("interleave", {**mx_case(16, tokens=40), **{k: mx_case(16, tokens=40)[k][:4] for k in ("w1", "w1_scale", "w2", "w2_scale")},
                        "expert_mask": mask, "num_local_tokens": torch.tensor([33], dtype=torch.int32), "swiglu_limit": 7.0},
         {"gate_mode": "interleave", "has_expert_mask": True, "has_num_local_tokens": True},
         {"act_bits": 16, "swiglu_limit": 7.0, "num_local_tokens": 33}),
        ("swiglu_bf16", {**mx_case(17, tokens=70), "swiglu_limit": 7.0}, {"activation": "swiglu"},
         {"activation": "swiglu", "swiglu_limit": 7.0, "act_bits": 16}),
    ]


def mega_group():
    """Two ranks, 3 experts each: global expert e = local e % 3 of rank e // 3."""
    base = mx_case(7)
    group = []
    for r in range(2):
        mine = mx_case(100 + r)
        group.append(
            dict(
                hidden_states=mine["hidden_states"],
                topk_ids=mine["topk_ids"],
                topk_weights=mine["topk_weights"],
                w1=base["w1"][3 * r : 3 * r + 3],
                w1_scale=base["w1_scale"][3 * r : 3 * r + 3],
                w2=base["w2"][3 * r : 3 * r + 3],
                w2_scale=base["w2_scale"][3 * r : 3 * r + 3],
                swiglu_limit=10.0,
            )
        )
    return base, group
