"""Seeded synthetic inputs shaped like the benchmark configurations of the fused-MoE path.

They stand in for the public model shapes (Mixtral-8x7B, Qwen3-30B-A3B, DeepSeek-V3): no
checkpoint is read.  Everything is drawn from one ``torch.Generator`` seeded per tensor
name, on the device asked for (CPU for parity cases small enough for the CPU checker, the
GPU for full-size layers whose 11 GB of expert weights would take minutes on the host).
"""

from __future__ import annotations

import dataclasses
import hashlib
import math

import torch

FP8 = torch.float8_e4m3fn
BLOCK = 128


@dataclasses.dataclass(frozen=True)
class MoEConfig:
    """One fused-MoE layer shape.  ``n_shared`` experts sit after the routed ones in w1/w2."""

    name: str
    hidden: int
    inter: int
    n_routed: int
    topk: int
    scoring: str = "softmax"  # "softmax" | "sigmoid"
    n_shared: int = 0
    num_expert_group: int = 1
    topk_group: int = 1
    renormalize: bool = True
    routed_scaling_factor: float = 1.0
    zipf_s: float = 0.0  # > 0: log-Zipf popularity bias added to the router logits

    @property
    def n_experts(self) -> int:
        return self.n_routed + self.n_shared

    @property
    def routes_per_token(self) -> int:
        return self.topk + self.n_shared

    @property
    def expert_weight_bytes(self) -> int:
        """FP8 bytes of one expert's w1 + w2 plus their float32 block scales."""
        h, i = self.hidden, self.inter
        return 3 * h * i + 4 * ((2 * i // BLOCK) * (h // BLOCK) + (h // BLOCK) * (i // BLOCK))

    @property
    def flops_per_route(self) -> int:
        return 6 * self.hidden * self.inter


CONFIGS = {
    "tiny": MoEConfig("tiny", hidden=256, inter=512, n_routed=8, topk=2),
    "mixtral": MoEConfig("mixtral", hidden=4096, inter=14336, n_routed=8, topk=2),
    "qwen3": MoEConfig("qwen3", hidden=2048, inter=768, n_routed=128, topk=8, zipf_s=1.1),
    "deepseek_v3": MoEConfig(
        "deepseek_v3",
        hidden=7168,
        inter=2048,
        n_routed=256,
        topk=8,
        scoring="sigmoid",
        n_shared=1,
        num_expert_group=8,
        topk_group=4,
        renormalize=True,
        routed_scaling_factor=2.5,
    ),
    # DeepSeek-V3 routing on a layer small enough for the CPU checker
    "deepseek_small": MoEConfig(
        "deepseek_small",
        hidden=512,
        inter=256,
        n_routed=64,
        topk=8,
        scoring="sigmoid",
        n_shared=1,
        num_expert_group=8,
        topk_group=4,
        renormalize=True,
        routed_scaling_factor=2.5,
    ),
}


def _generator(seed: int, name: str, device) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def normal(seed: int, name: str, shape, std: float, device="cpu", dtype=torch.float32) -> torch.Tensor:
    g = _generator(seed, name, device)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


def quantize_block_fp8(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """float32 [..., rows, cols] -> (e4m3 codes, float32 scale per 128 x 128 block = amax/448)."""
    *lead, rows, cols = w.shape
    rb, cb = rows // BLOCK, cols // BLOCK
    blocks = w.reshape(*lead, rb, BLOCK, cb, BLOCK)
    amax = blocks.abs().amax(dim=(-3, -1), keepdim=True)
    scale = (amax / 448.0).clamp_min(torch.finfo(torch.float32).tiny)
    codes = (blocks / scale).to(FP8).reshape(*lead, rows, cols)
    return codes, scale.reshape(*lead, rb, cb).contiguous()


E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def quantize_mxfp4(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """float32 [..., rows, cols] -> (packed e2m1 uint8 [..., rows, cols/2], low nibble first;
    e8m0 scale bytes uint8 [..., rows, cols/32]).  Per 1 x 32 block the scale is the power of two
    that puts amax in (3, 6]; codes are the nearest grid value, ties to the even code."""
    grid = torch.tensor(E2M1_GRID, dtype=torch.float32, device=w.device)
    blocks = w.unflatten(-1, (-1, 32))
    amax = blocks.abs().amax(dim=-1, keepdim=True).clamp_min(1e-10)
    mantissa, exponent = torch.frexp(amax)
    exponent = (exponent - 3 + (mantissa > 0.75).int()).clamp(-127, 127)
    scaled = blocks / torch.exp2(exponent.float())
    m = scaled.abs()
    lo = torch.bucketize(m, grid, right=True) - 1
    hi = (lo + 1).clamp_max(7)
    below, above = m - grid[lo], grid[hi] - m
    up = (above < below) | ((above == below) & (hi % 2 == 0))
    code = torch.where(up, hi, lo) | ((scaled < 0).long() << 3)
    code = code.flatten(-2).to(torch.uint8)
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    return packed.contiguous(), (exponent.squeeze(-1) + 127).to(torch.uint8).contiguous()


def mx_expert_weights(cfg: MoEConfig, seed: int, device="cpu", experts=None):
    """(w1 e2m1x2 uint8 [E,2I,H/2], w1_scale e8m0 uint8 [E,2I,H/32], w2 [E,H,I/2], w2_scale [E,H,I/32]):
    N(0,0.02) quantised to MXFP4, each expert from its own seed."""
    ids = list(range(cfg.n_experts)) if experts is None else list(experts)
    h, i = cfg.hidden, cfg.inter
    w1 = torch.empty((len(ids), 2 * i, h // 2), dtype=torch.uint8, device=device)
    s1 = torch.empty((len(ids), 2 * i, h // 32), dtype=torch.uint8, device=device)
    w2 = torch.empty((len(ids), h, i // 2), dtype=torch.uint8, device=device)
    s2 = torch.empty((len(ids), h, i // 32), dtype=torch.uint8, device=device)
    for slot, e in enumerate(ids):
        w1[slot], s1[slot] = quantize_mxfp4(normal(seed, f"w1.{e}", (2 * i, h), 0.02, device))
        w2[slot], s2[slot] = quantize_mxfp4(normal(seed, f"w2.{e}", (h, i), 0.02, device))
    return w1, s1, w2, s2


def one_expert_weights(cfg: MoEConfig, seed: int, expert: int, device="cpu"):
    """(w1 e4m3 [2I,H], w1_scale, w2 e4m3 [H,I], w2_scale) of one expert: N(0,0.02) quantised per
    128 x 128 block.  Each expert has its own seed, so any subset can be drawn alone."""
    h, i = cfg.hidden, cfg.inter
    w1, s1 = quantize_block_fp8(normal(seed, f"w1.{expert}", (2 * i, h), 0.02, device))
    w2, s2 = quantize_block_fp8(normal(seed, f"w2.{expert}", (h, i), 0.02, device))
    return w1, s1, w2, s2


def expert_weights(cfg: MoEConfig, seed: int, device="cpu", experts=None):
    """(w1 e4m3 [E,2I,H], w1_scale f32 [E,2I/128,H/128], w2 e4m3 [E,H,I], w2_scale) for the expert
    slots ``experts`` (default: all, the shared ones last)."""
    ids = list(range(cfg.n_experts)) if experts is None else list(experts)
    h, i = cfg.hidden, cfg.inter
    w1 = torch.empty((len(ids), 2 * i, h), dtype=FP8, device=device)
    w2 = torch.empty((len(ids), h, i), dtype=FP8, device=device)
    s1 = torch.empty((len(ids), 2 * i // BLOCK, h // BLOCK), dtype=torch.float32, device=device)
    s2 = torch.empty((len(ids), h // BLOCK, i // BLOCK), dtype=torch.float32, device=device)
    for slot, e in enumerate(ids):
        w1[slot], s1[slot], w2[slot], s2[slot] = one_expert_weights(cfg, seed, e, device)
    return w1, s1, w2, s2


def router_inputs(cfg: MoEConfig, n_tokens: int, seed: int, device="cpu"):
    """(hidden bf16 [T,H], logits bf16 [T,E_routed], correction_bias bf16 [E_routed] or None).

    Logits are seeded N(0,1) rounded to bf16; with ``zipf_s`` a per-expert popularity bias
    ``-s * ln(rank)`` (ranks a seeded permutation of 1..E) is added before rounding."""
    hidden = normal(seed, "hidden", (n_tokens, cfg.hidden), 1.0, device, torch.bfloat16)
    logits = normal(seed, "logits", (n_tokens, cfg.n_routed), 1.0, device)
    if cfg.zipf_s > 0:
        g = _generator(seed, "zipf", "cpu")
        ranks = (torch.randperm(cfg.n_routed, generator=g) + 1).to(torch.float32)
        logits = logits + (-cfg.zipf_s * torch.log(ranks)).to(device)
    logits = logits.to(torch.bfloat16)
    bias = None
    if cfg.scoring == "sigmoid":
        bias = normal(seed, "bias", (cfg.n_routed,), 0.01, device, torch.bfloat16)
    return hidden, logits, bias


def router_weight(cfg: MoEConfig, seed: int, device="cpu") -> torch.Tensor:
    """bf16 [E_routed, H] router projection, N(0,0.02)."""
    return normal(seed, "router", (cfg.n_routed, cfg.hidden), 0.02, device, torch.bfloat16)


def roofline_work(cfg: MoEConfig, n_tokens: int, distinct_experts: int) -> tuple[float, float]:
    """(flops, algorithmic HBM bytes) of one layer call: every route costs 6*H*I flops; each
    distinct expert hit is read once; activations in, out and the logits once."""
    routes = n_tokens * cfg.routes_per_token
    flops = float(routes) * cfg.flops_per_route
    act = n_tokens * cfg.hidden * 2 * 2 + n_tokens * cfg.n_routed * 2
    return flops, float(distinct_experts) * cfg.expert_weight_bytes + act


def expected_distinct_experts(cfg: MoEConfig, n_tokens: int) -> float:
    """Expected number of distinct routed experts hit under uniform routing (+ shared)."""
    p_miss = (1.0 - cfg.topk / cfg.n_routed) ** n_tokens
    return cfg.n_routed * (1.0 - p_miss) + cfg.n_shared


def zipf_note() -> str:
    return "per-expert logit bias -s*ln(rank), ranks a seeded permutation (Zipf(s) popularity)"


__all__ = [
    "CONFIGS",
    "MoEConfig",
    "expert_weights",
    "expected_distinct_experts",
    "mx_expert_weights",
    "normal",
    "one_expert_weights",
    "quantize_mxfp4",
    "quantize_block_fp8",
    "roofline_work",
    "router_inputs",
    "router_weight",
]
_ = math
