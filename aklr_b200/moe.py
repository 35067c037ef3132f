"""Host-side calls into the sm_100a fused-MoE kernels (through the C ABI, ``_lib``).

torch is used for device memory and the current stream only.  Every function here requires a
CUDA device of compute capability 10.0 and the built library; none has a CPU path.
"""

from __future__ import annotations

import ctypes
import dataclasses

import torch

from aklr_b200 import _lib
from aklr_b200._lib import MoeConfig, WorkspaceLayout

FP8 = torch.float8_e4m3fn
_SIGMOID_TABLES: dict[torch.device, torch.Tensor] = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    device = tensors[0].device
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.device != device:
            raise ValueError("the fused-MoE kernels take CUDA tensors on one device; there is no CPU path")
        if not t.is_contiguous():
            raise ValueError("the fused-MoE kernels take contiguous tensors")
    return device


def sigmoid_table(device: torch.device) -> torch.Tensor:
    """float32[65536]: sigmoid of every bf16 bit pattern, as torch computes it on the host.

    The reference ranks experts by ``logits.sigmoid() + bias`` evaluated by torch on the CPU
    (aklr/plugins/sglang/models/deepseek_v2/reference.py:133-134); its low bits are
    implementation-defined, so the routing kernel looks the score up in this table to give the
    same expert ids bit for bit.  Built once per device."""
    device = torch.device(device)
    table = _SIGMOID_TABLES.get(device)
    if table is None:
        every = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
        table = torch.sigmoid(every).to(device)
        _SIGMOID_TABLES[device] = table
    return table


@dataclasses.dataclass
class Routing:
    """How a layer routes: mirrors the attrs of the reference contracts
    (aklr/plugins/sglang/models/deepseek_v2/contract.py:206-220)."""

    topk: int
    scoring: str = "softmax"
    n_shared: int = 0
    num_expert_group: int = 1
    topk_group: int = 1
    renormalize: bool = True
    routed_scaling_factor: float = 1.0


def _config(n_tokens, hidden, inter, n_routed, r: Routing, logits=None, bias=None, block_m=0, n_global=0, variant=0) -> MoeConfig:
    def code(t):
        if t is None or t.dtype == torch.bfloat16:
            return _lib.DTYPE_BF16
        if t.dtype == torch.float32:
            return _lib.DTYPE_F32
        raise ValueError(f"router logits / bias must be bfloat16 or float32, got {t.dtype}")

    return MoeConfig(
        n_tokens=n_tokens,
        hidden=hidden,
        inter=inter,
        n_routed=n_routed,
        n_shared=r.n_shared,
        topk=r.topk,
        scoring=_lib.SCORING[r.scoring],
        num_expert_group=r.num_expert_group,
        topk_group=r.topk_group,
        renormalize=int(bool(r.renormalize)),
        routed_scaling_factor=float(r.routed_scaling_factor),
        logits_dtype=code(logits),
        bias_dtype=code(bias),
        block_m=block_m,
        n_experts_global=n_global,
        variant=variant,
    )


def workspace_layout(cfg: MoeConfig) -> WorkspaceLayout:
    layout = WorkspaceLayout()
    _lib.check(_lib.load().aklr_moe_fp8_workspace(ctypes.byref(cfg), ctypes.byref(layout)))
    return layout


class Workspace:
    """The scratch buffer of one layer call and typed views of its intermediates."""

    def __init__(self, cfg: MoeConfig, device: torch.device):
        self.cfg = cfg
        self.layout = workspace_layout(cfg)
        self.buffer = torch.empty(self.layout.total_bytes + 1024, dtype=torch.uint8, device=device)
        shift = (-self.buffer.data_ptr()) % 1024
        self.base = self.buffer[shift : shift + self.layout.total_bytes]

    def _view(self, offset: int, count: int, dtype: torch.dtype) -> torch.Tensor:
        size = torch.empty((), dtype=dtype).element_size()
        return self.base[offset : offset + count * size].view(dtype)

    def check_status(self) -> None:
        """Waits for the stream and raises if a device-side wait gave up."""
        status = (ctypes.c_int32 * 2)()
        _lib.check(_lib.load().aklr_moe_read_status(self.base.data_ptr(), status, _stream()))

    @property
    def routes_per_token(self) -> int:
        return self.cfg.topk + self.cfg.n_shared

    def topk_ids(self) -> torch.Tensor:
        n = self.cfg.n_tokens * self.routes_per_token
        return self._view(self.layout.topk_ids, n, torch.int32).view(self.cfg.n_tokens, -1)

    def topk_weights(self) -> torch.Tensor:
        n = self.cfg.n_tokens * self.routes_per_token
        return self._view(self.layout.topk_weights, n, torch.float32).view(self.cfg.n_tokens, -1)

    def counts(self) -> torch.Tensor:
        return self._view(self.layout.counts, self.layout.n_experts, torch.int32)

    def num_blocks(self) -> int:
        return int(self._view(self.layout.num_blocks, 2, torch.int32)[0])

    def sorted_ids(self) -> torch.Tensor:
        return self._view(self.layout.sorted_ids, self.num_blocks() * self.layout.block_m, torch.int32)

    def block_expert(self) -> torch.Tensor:
        return self._view(self.layout.block_expert, self.num_blocks(), torch.int32)

    def _row_scales(self, offset: int, groups: int) -> torch.Tensor:
        """Scales stored [block, group, row-in-block], returned as [row, group]."""
        blocks, bm = self.layout.max_blocks, self.layout.block_m
        stored = self._view(offset, blocks * groups * bm, torch.float32).view(blocks, groups, bm)
        return stored.permute(0, 2, 1).reshape(blocks * bm, groups)

    def xq(self) -> tuple[torch.Tensor, torch.Tensor]:
        rows, h = self.layout.capacity, self.cfg.hidden
        return self._view(self.layout.xq, rows * h, FP8).view(rows, h), self._row_scales(self.layout.xs, h // 128)

    def hq(self) -> tuple[torch.Tensor, torch.Tensor]:
        rows, i = self.layout.capacity, self.cfg.inter
        return self._view(self.layout.hq, rows * i, FP8).view(rows, i), self._row_scales(self.layout.hs, i // 128)

    def route_rows(self) -> torch.Tensor:
        n = self.cfg.n_tokens * self.routes_per_token
        return self._view(self.layout.rows, n * self.cfg.hidden, torch.bfloat16).view(n, self.cfg.hidden)


def _weights_variant(w1, w2) -> int:
    """VARIANT_TILED_WEIGHTS when both weight tensors carry ``is_b200_tiled`` (aklr_b200.layouts), 0 when neither."""
    tiled = [bool(getattr(w, "is_b200_tiled", False)) for w in (w1, w2)]
    if tiled[0] != tiled[1]:
        raise ValueError("w1 and w2 must be in the same layout: both row-major or both tile-contiguous")
    return _lib.VARIANT_TILED_WEIGHTS if tiled[0] else 0


def require_row_major(*weights) -> None:
    """Paths without a tile-contiguous form (MXFP4 experts, expert parallelism) refuse such tensors."""
    if any(getattr(w, "is_b200_tiled", False) for w in weights):
        raise ValueError("tile-contiguous weights are served by the FP8 single-GPU entry points only")


def _check_weights(hidden_states, w1, w1_scale, w2, w2_scale):
    e, two_i, h = w1.shape
    inter = two_i // 2
    if hidden_states.dtype != torch.bfloat16 or hidden_states.shape[-1] != h:
        raise ValueError("hidden_states must be bfloat16 [tokens, hidden] matching w1's last dim")
    if w1.dtype != FP8 or w2.dtype != FP8 or tuple(w2.shape) != (e, h, inter):
        raise ValueError("w1 [E,2I,H] and w2 [E,H,I] must be float8_e4m3fn")
    if w1_scale.dtype != torch.float32 or tuple(w1_scale.shape) != (e, two_i // 128, h // 128):
        raise ValueError("w1_scale must be float32 [E, 2I/128, H/128]")
    if w2_scale.dtype != torch.float32 or tuple(w2_scale.shape) != (e, h // 128, inter // 128):
        raise ValueError("w2_scale must be float32 [E, H/128, I/128]")
    return e, inter, h


def fused_moe_fp8(
    hidden_states: torch.Tensor,
    logits: torch.Tensor,
    bias: torch.Tensor | None,
    w1: torch.Tensor,
    w1_scale: torch.Tensor,
    w2: torch.Tensor,
    w2_scale: torch.Tensor,
    routing: Routing,
    out: torch.Tensor | None = None,
    block_m: int = 0,
    workspace: Workspace | None = None,
    return_workspace: bool = False,
    variant: int = 0,
):
    """The whole FP8 layer from router logits: routing, sort, quant, gate_up, down, combine.
    ``variant``: ``_lib.VARIANT_*`` bits overriding a kernel choice for this call (tests)."""
    device = _need_cuda(hidden_states, logits, bias, w1, w1_scale, w2, w2_scale, out)
    e, inter, h = _check_weights(hidden_states, w1, w1_scale, w2, w2_scale)
    n_tokens, n_routed = logits.shape
    if n_routed + routing.n_shared != e or hidden_states.shape[0] != n_tokens:
        raise ValueError("w1 must hold the routed experts followed by the shared ones")
    cfg = _config(n_tokens, h, inter, n_routed, routing, logits, bias, block_m, variant=variant | _weights_variant(w1, w2))
    ws = workspace or Workspace(cfg, device)
    if out is None:
        out = torch.empty_like(hidden_states)
    table = sigmoid_table(device) if routing.scoring == "sigmoid" and logits.dtype == torch.bfloat16 else None
    _lib.check(
        _lib.load().aklr_moe_fp8_forward(
            ctypes.byref(cfg),
            _ptr(hidden_states),
            _ptr(logits),
            _ptr(bias),
            _ptr(table),
            _ptr(w1),
            _ptr(w1_scale),
            _ptr(w2),
            _ptr(w2_scale),
            _ptr(out),
            ws.base.data_ptr(),
            ws.layout.total_bytes,
            _stream(),
        )
    )
    return (out, ws) if return_workspace else out


def fused_experts_fp8(
    hidden_states: torch.Tensor,
    topk_ids: torch.Tensor,
    topk_weights: torch.Tensor,
    w1: torch.Tensor,
    w1_scale: torch.Tensor,
    w2: torch.Tensor,
    w2_scale: torch.Tensor,
    expert_map: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    block_m: int = 0,
    return_workspace: bool = False,
):
    """Experts only, routing given.  ``expert_map`` (int32 [global experts] -> local slot or -1)
    makes it one rank's share under expert parallelism with replicated tokens."""
    device = _need_cuda(hidden_states, topk_ids, topk_weights, w1, w1_scale, w2, w2_scale, expert_map, out)
    e, inter, h = _check_weights(hidden_states, w1, w1_scale, w2, w2_scale)
    if topk_ids.dtype != torch.int32 or topk_weights.dtype != torch.float32 or topk_ids.shape != topk_weights.shape:
        raise ValueError("topk_ids int32 and topk_weights float32 must share the shape [tokens, routes]")
    n_tokens, routes = topk_ids.shape
    n_global = 0 if expert_map is None else expert_map.numel()
    cfg = _config(n_tokens, h, inter, e, Routing(topk=routes), None, None, block_m, n_global, variant=_weights_variant(w1, w2))
    ws = Workspace(cfg, device)
    if out is None:
        out = torch.empty_like(hidden_states)
    _lib.check(
        _lib.load().aklr_moe_fp8_experts(
            ctypes.byref(cfg),
            _ptr(hidden_states),
            _ptr(topk_ids),
            _ptr(topk_weights),
            _ptr(expert_map),
            _ptr(w1),
            _ptr(w1_scale),
            _ptr(w2),
            _ptr(w2_scale),
            _ptr(out),
            ws.base.data_ptr(),
            ws.layout.total_bytes,
            _stream(),
        )
    )
    return (out, ws) if return_workspace else out


def _check_mx_weights(hidden_states, w1, w1_scale, w2, w2_scale):
    e, two_i, half_h = w1.shape
    h, inter = half_h * 2, two_i // 2
    if hidden_states.dtype != torch.bfloat16 or hidden_states.shape[-1] != h:
        raise ValueError("hidden_states must be bfloat16 [tokens, hidden] matching w1's unpacked last dim")
    for t in (w1, w1_scale, w2, w2_scale):
        if t.dtype != torch.uint8:
            raise ValueError("MXFP4 weights (packed e2m1) and their e8m0 scales are uint8 tensors")
    if tuple(w2.shape) != (e, h, inter // 2) or tuple(w1_scale.shape) != (e, two_i, h // 32) or tuple(w2_scale.shape) != (e, h, inter // 32):
        raise ValueError("expected w1 [E,2I,H/2], w1_scale [E,2I,H/32], w2 [E,H,I/2], w2_scale [E,H,I/32]")
    return e, inter, h


def _act_bits_variant(act_bits: int) -> int:
    """The numerics mode of the MXFP4 entry points for the bits the activations keep: 4 MXFP4, 8 MXFP8, 16 bf16."""
    try:
        return {4: _lib.VARIANT_MXFP4_ACTIVATIONS, 8: 0, 16: _lib.VARIANT_BF16_ACTIVATIONS}[act_bits]
    except KeyError:
        raise ValueError("act_bits: 4 (MXFP4 activations), 8 (MXFP8) or 16 (kept in bf16)") from None


# the AKLR_ACT_* values of the public header, by the reference's attribute names
ACTIVATIONS = {"silu": 0, "gelu": 1, "swiglu": 2, "situv2": 3}


def fused_experts_mxfp4(
    hidden_states: torch.Tensor,
    topk_ids: torch.Tensor,
    topk_weights: torch.Tensor,
    w1: torch.Tensor,
    w1_scale: torch.Tensor,
    w2: torch.Tensor,
    w2_scale: torch.Tensor,
    expert_map: torch.Tensor | None = None,
    swiglu_limit: float | None = None,
    out: torch.Tensor | None = None,
    return_workspace: bool = False,
    activation: str = "silu",
    weight_in_stage1: bool = False,
    beta: float | None = None,
    linear_beta: float | None = None,
    num_local_tokens: torch.Tensor | None = None,
    variant: int = 0,
    act_bits: int = 8,
):
    """MXFP4-weight experts, routing given (block-scaled tcgen05 MMA).  ``act_bits`` 8: activations
    quantised to MXFP8 per 1 x 32; 4: to MXFP4 (the reference op's default); 16: kept in bf16 (each value enters the MMAs as two e4m3 terms whose
    sum is the bf16 value) -- the reference's gate_mode 'interleave' and gpt-oss swiglu below 256 rows.
    ``activation`` one of ACTIVATIONS; ``weight_in_stage1`` applies the route weight to the gate_up
    projection instead of the output; ``num_local_tokens`` (int32 device scalar) zeroes the rows at
    or past it (aklr/ops/fused_moe/reference.py:85-127)."""
    device = _need_cuda(hidden_states, topk_ids, topk_weights, w1, w1_scale, w2, w2_scale, expert_map, out, num_local_tokens)
    variant |= _act_bits_variant(act_bits)
    options = _lib.MxOptions(
        ACTIVATIONS[activation], int(weight_in_stage1), float(swiglu_limit or 0.0), float(beta or 0.0),
        float(linear_beta or 0.0), _ptr(num_local_tokens),
    )
    require_row_major(w1, w2)
    e, inter, h = _check_mx_weights(hidden_states, w1, w1_scale, w2, w2_scale)
    if topk_ids.dtype != torch.int32 or topk_weights.dtype != torch.float32 or topk_ids.shape != topk_weights.shape:
        raise ValueError("topk_ids int32 and topk_weights float32 must share the shape [tokens, routes]")
    n_tokens, routes = topk_ids.shape
    n_global = 0 if expert_map is None else expert_map.numel()
    cfg = _config(n_tokens, h, inter, e, Routing(topk=routes), None, None, 128, n_global, variant)
    ws = Workspace(cfg, device)
    if out is None:
        out = torch.empty_like(hidden_states)
    _lib.check(
        _lib.load().aklr_moe_mxfp4_experts_ex(
            ctypes.byref(cfg), _ptr(hidden_states), _ptr(topk_ids), _ptr(topk_weights), _ptr(expert_map), _ptr(w1),
            _ptr(w1_scale), _ptr(w2), _ptr(w2_scale), ctypes.byref(options), _ptr(out), ws.base.data_ptr(),
            ws.layout.total_bytes, _stream(),
        )
    )
    return (out, ws) if return_workspace else out


def fused_moe_mxfp4(
    hidden_states: torch.Tensor,
    logits: torch.Tensor,
    bias: torch.Tensor | None,
    w1: torch.Tensor,
    w1_scale: torch.Tensor,
    w2: torch.Tensor,
    w2_scale: torch.Tensor,
    routing: Routing,
    swiglu_limit: float | None = None,
    out: torch.Tensor | None = None,
    workspace: Workspace | None = None,
    return_workspace: bool = False,
    act_bits: int = 8,
):
    """The whole MXFP4 layer from router logits (the routing of ``fused_moe_fp8``).  ``act_bits`` as in
    ``fused_experts_mxfp4``: 8 MXFP8 activations, 16 activations kept in bf16."""
    device = _need_cuda(hidden_states, logits, bias, w1, w1_scale, w2, w2_scale, out)
    require_row_major(w1, w2)
    e, inter, h = _check_mx_weights(hidden_states, w1, w1_scale, w2, w2_scale)
    n_tokens, n_routed = logits.shape
    if n_routed + routing.n_shared != e or hidden_states.shape[0] != n_tokens:
        raise ValueError("w1 must hold the routed experts followed by the shared ones")
    cfg = _config(n_tokens, h, inter, n_routed, routing, logits, bias, 128, variant=_act_bits_variant(act_bits))
    ws = workspace or Workspace(cfg, device)
    if out is None:
        out = torch.empty_like(hidden_states)
    table = sigmoid_table(device) if routing.scoring == "sigmoid" and logits.dtype == torch.bfloat16 else None
    _lib.check(
        _lib.load().aklr_moe_mxfp4_forward(
            ctypes.byref(cfg), _ptr(hidden_states), _ptr(logits), _ptr(bias), _ptr(table), _ptr(w1), _ptr(w1_scale),
            _ptr(w2), _ptr(w2_scale), float(swiglu_limit or 0.0), _ptr(out), ws.base.data_ptr(), ws.layout.total_bytes,
            _stream(),
        )
    )
    return (out, ws) if return_workspace else out


def route(logits: torch.Tensor, bias: torch.Tensor | None, routing: Routing, topk_ids=None, topk_weights=None):
    """(topk_ids int32, topk_weights float32), both [tokens, topk + n_shared]."""
    device = _need_cuda(logits, bias, topk_ids, topk_weights)
    n_tokens, n_routed = logits.shape
    width = routing.topk + routing.n_shared
    if topk_ids is None:
        topk_ids = torch.empty((n_tokens, width), dtype=torch.int32, device=device)
    if topk_weights is None:
        topk_weights = torch.empty((n_tokens, width), dtype=torch.float32, device=device)
    cfg = _config(n_tokens, 128, 128, n_routed, routing, logits, bias)
    table = sigmoid_table(device) if routing.scoring == "sigmoid" and logits.dtype == torch.bfloat16 else None
    _lib.check(
        _lib.load().aklr_moe_route(
            ctypes.byref(cfg), _ptr(logits), _ptr(bias), _ptr(table), _ptr(topk_ids), _ptr(topk_weights), _stream()
        )
    )
    return topk_ids, topk_weights


def moe_align(topk_ids: torch.Tensor, n_experts: int, block_m: int, expert_map: torch.Tensor | None = None):
    """(sorted_route_ids, block_expert, counts, num_blocks): the stable padded sort by expert.
    Reads ``num_blocks`` back, so it synchronises: a test and tooling helper."""
    device = _need_cuda(topk_ids, expert_map)
    lib = _lib.load()
    n_routes = topk_ids.numel()
    max_blocks = max(1, lib.aklr_moe_align_max_blocks(n_routes, n_experts, block_m))
    sorted_ids = torch.empty(max_blocks * block_m, dtype=torch.int32, device=device)
    block_expert = torch.empty(max_blocks, dtype=torch.int32, device=device)
    counts = torch.empty(n_experts, dtype=torch.int32, device=device)
    num_blocks = torch.zeros(2, dtype=torch.int32, device=device)
    scratch = torch.empty(max(1, (n_routes + 1023) // 1024) * n_experts, dtype=torch.int32, device=device)
    n_global = n_experts if expert_map is None else expert_map.numel()
    _lib.check(
        lib.aklr_moe_align(
            _ptr(topk_ids),
            _ptr(expert_map),
            n_routes,
            n_experts,
            n_global,
            block_m,
            _ptr(sorted_ids),
            _ptr(block_expert),
            _ptr(counts),
            _ptr(num_blocks),
            _ptr(scratch),
            _stream(),
        )
    )
    nb = int(num_blocks[0])
    return sorted_ids[: nb * block_m], block_expert[:nb], counts, nb


def router_logits(hidden_states: torch.Tensor, router_weight: torch.Tensor) -> torch.Tensor:
    """bf16 [tokens, experts] = bf16(hidden_states @ router_weight^T), float32 accumulation."""
    device = _need_cuda(hidden_states, router_weight)
    if hidden_states.dtype != torch.bfloat16 or router_weight.dtype != torch.bfloat16:
        raise ValueError("router inputs must be bfloat16")
    n_tokens, h = hidden_states.shape
    n_routed = router_weight.shape[0]
    logits = torch.empty((n_tokens, n_routed), dtype=torch.bfloat16, device=device)
    _lib.check(
        _lib.load().aklr_router_gemm_bf16(
            _ptr(hidden_states), _ptr(router_weight), _ptr(logits), n_tokens, h, n_routed, _stream()
        )
    )
    return logits


def with_gated_shared_slot(hidden_states, shared_gate_weight, topk_ids, topk_weights, shared_slot: int, copy_from=None):
    """Slot K of the [tokens, K+1] routing tables <- expert ``shared_slot`` at sigmoid(x . gate).
    ``copy_from`` = (ids [tokens, K] int32, weights [tokens, K] float32) fills the first K slots too."""
    _need_cuda(hidden_states, shared_gate_weight, topk_ids, topk_weights)
    n_tokens, h = hidden_states.shape
    ids_in, w_in = copy_from if copy_from is not None else (None, None)
    _lib.check(
        _lib.load().aklr_moe_shared_gate(
            _ptr(hidden_states), _ptr(shared_gate_weight), _ptr(ids_in), _ptr(w_in), _ptr(topk_ids), _ptr(topk_weights),
            n_tokens, h, topk_ids.shape[1] - 1, shared_slot, _stream(),
        )
    )
    return topk_ids, topk_weights


def add_bf16_shared_expert(hidden_states, shared_w1, shared_w2, shared_gate_weight, out):
    """out += sigmoid(x . shared_gate_weight) * down(silu(gate(x)) * up(x)) of a shared expert held in bf16 apart
    from the routed ones (aklr/plugins/sglang/models/qwen2_moe/reference.py:160-185).  The two projections are plain
    dense GEMMs (torch.mm: the library GEMM); the gated product and the weighted add are this library's kernels."""
    _need_cuda(hidden_states, shared_w1, shared_w2, shared_gate_weight, out)
    n_tokens, h = hidden_states.shape
    inter = shared_w2.shape[1]
    if tuple(shared_w1.shape) != (2 * inter, h) or tuple(shared_w2.shape) != (h, inter) or shared_gate_weight.numel() != h:
        raise ValueError("shared_w1 [2*inter, hidden], shared_w2 [hidden, inter], shared_gate_weight [1, hidden]")
    lib = _lib.load()
    gate_up = torch.mm(hidden_states, shared_w1.t())
    gated = torch.empty((n_tokens, inter), dtype=torch.bfloat16, device=hidden_states.device)
    _lib.check(lib.aklr_silu_mul_bf16(_ptr(gate_up), _ptr(gated), n_tokens, inter, _stream()))
    rows = torch.mm(gated, shared_w2.t())
    _lib.check(lib.aklr_moe_add_gated_rows(_ptr(hidden_states), _ptr(shared_gate_weight), _ptr(rows), _ptr(out), n_tokens, h, _stream()))
    return out


def router_logits_f32(hidden_states: torch.Tensor, router_weight: torch.Tensor) -> torch.Tensor:
    """float32 [tokens, experts] = hidden_states (bf16) @ router_weight (float32)^T, nothing rounded."""
    device = _need_cuda(hidden_states, router_weight)
    if hidden_states.dtype != torch.bfloat16 or router_weight.dtype != torch.float32:
        raise ValueError("hidden_states must be bfloat16 and router_weight float32")
    n_tokens, h = hidden_states.shape
    n_routed = router_weight.shape[0]
    logits = torch.empty((n_tokens, n_routed), dtype=torch.float32, device=device)
    _lib.check(
        _lib.load().aklr_router_gemm_f32(_ptr(hidden_states), _ptr(router_weight), _ptr(logits), n_tokens, h, n_routed, _stream())
    )
    return logits


def per_group_quant_fp8(x: torch.Tensor, quantized=None, scales=None):
    """(e4m3 [T,H], float32 scales [H/128, T]) -- the standalone op's scheme."""
    device = _need_cuda(x, quantized, scales)
    rows, h = x.shape
    if quantized is None:
        quantized = torch.empty((rows, h), dtype=FP8, device=device)
    if scales is None:
        scales = torch.empty((h // 128, rows), dtype=torch.float32, device=device)
    _lib.check(_lib.load().aklr_per_group_quant_fp8(_ptr(x), _ptr(quantized), _ptr(scales), rows, h, _stream()))
    return quantized, scales


def per_group_quant_mxfp8(x: torch.Tensor, quantized=None, scales=None):
    """(e4m3 [T,H], e8m0 exponent bytes uint8 [T,H/32])."""
    device = _need_cuda(x, quantized, scales)
    rows, h = x.shape
    if quantized is None:
        quantized = torch.empty((rows, h), dtype=FP8, device=device)
    if scales is None:
        scales = torch.empty((rows, h // 32), dtype=torch.uint8, device=device)
    _lib.check(_lib.load().aklr_per_group_quant_mxfp8(_ptr(x), _ptr(quantized), _ptr(scales), rows, h, _stream()))
    return quantized, scales


def act_quant_fp8(x: torch.Tensor):
    """(e4m3 [T,H], float32 scales [T,H/128]) -- the MoE layer's own scheme (true divisions)."""
    device = _need_cuda(x)
    rows, h = x.shape
    quantized = torch.empty((rows, h), dtype=FP8, device=device)
    scales = torch.empty((rows, h // 128), dtype=torch.float32, device=device)
    _lib.check(_lib.load().aklr_moe_act_quant_fp8(_ptr(x), _ptr(quantized), _ptr(scales), rows, h, _stream()))
    return quantized, scales
