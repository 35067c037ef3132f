"""Expert parallelism for the fused-MoE layer: tokens stay on their home rank, experts are sharded,
one NCCL all-to-all carries quantised token rows out and one carries bf16 rows back.

Ownership is the reference's (aklr/ops/mega_moe/contract.py:42-51, reference.py:25,38): with
``n_local`` routed experts per rank, global expert ``e`` is local expert ``e % n_local`` of rank
``e // n_local``.  Shared experts are replicated and applied to a rank's own tokens on a side
stream while the dispatch is in flight.  No kernel waits on another rank: every exchange is a
host-ordered collective whose payload lands in local HBM before a kernel reads it.

What travels is one row per (token, destination rank), not one per route: a token whose routes name
several experts of one rank sends that rank its quantised row once, with the list of (local expert,
weight) pairs; the rank runs them all and returns ONE row, their weighted sum.  With DeepSeek-V3's
group-limited routing (8 groups, 4 kept) a token reaches at most 4 of 8 ranks, so both all-to-alls
carry half of what one row per route would.  The row, its scales and the pairs are one packed buffer
(``RowLayout``), so a direction is one collective.

One step of one rank is three phases, so that a test can drive several ranks in one process:

    state = layer.prepare(hidden, logits, bias)          # route, plan, quantise, pack
    received = exchange(state.packed, ...)               # all-to-all by destination rank
    rows = layer.compute(received)                       # local experts over the rows received
    back = exchange back                                 # all-to-all, same splits reversed
    out = layer.finish(state, back)                      # sum at home + shared experts

``ExpertParallelMoE.forward`` runs them over ``torch.distributed``.  It reads the split sizes of the
uneven all-to-all on the host once per step, so it cannot be captured in a CUDA graph.
"""

from __future__ import annotations

import ctypes
import dataclasses

import torch

from aklr_b200 import _lib
from aklr_b200.moe import (
    Routing,
    Workspace,
    _config,
    _ptr,
    _stream,
    fused_experts_fp8,
    fused_experts_mxfp4,
    require_row_major,
    route,
)


@dataclasses.dataclass(frozen=True)
class RowLayout:
    """Bytes of one travelling row: [hidden e4m3 codes][scales][topk int32 local expert ids][topk float32
    weights], padded to 16 bytes.  Scales: float32 per 128 values (FP8 experts) or one e8m0 byte per 32
    (MXFP4 experts).  ``aklr_ep_row_bytes`` computes the same size."""

    hidden: int
    topk: int
    mx: bool

    @property
    def scale_bytes(self) -> int:
        return self.hidden // 32 if self.mx else self.hidden // 128 * 4

    @property
    def meta_offset(self) -> int:
        return self.hidden + self.scale_bytes

    @property
    def row_bytes(self) -> int:
        return (self.meta_offset + 8 * self.topk + 15) // 16 * 16


@dataclasses.dataclass
class StepState:
    packed: torch.Tensor             # uint8 [capacity, row_bytes]; the first sum(counts) rows are sent
    counts: torch.Tensor             # int32 [world] rows per destination rank (device)
    position_of_route: torch.Tensor  # int32 [n_tokens * topk]: send position of a (token, rank)'s first slot, else -1
    shared_rows: torch.Tensor | None
    shared_done: torch.cuda.Event | None
    n_tokens: int
    layout: RowLayout


class CudaKernels:
    """The device side of the phases: libaklr_b200.so through the C ABI.

    ``fmt`` "fp8": e4m3 experts with 128 x 128 block scales, rows travel as FP8 + float32 scales per
    1 x 128.  "mxfp4": e2m1 experts with e8m0 scales, rows travel as MXFP8 (one e8m0 byte per 32);
    ``swiglu_limit`` then clamps gate and up as the reference's mega_moe does."""

    def __init__(self, fmt: str = "fp8", swiglu_limit: float | None = None):
        if fmt not in ("fp8", "mxfp4"):
            raise ValueError(f"unknown expert format {fmt!r}")
        self.fmt, self.swiglu_limit = fmt, swiglu_limit

    @property
    def mx(self) -> bool:
        return self.fmt == "mxfp4"

    def route(self, logits, bias, routing):
        return route(logits, bias, routing)

    def plan(self, ids, n_local, world):
        """(first slots sorted by destination rank int32 [T*K] -- the first sum(counts) entries count --,
        rows per rank int32 [world], position_of_route int32 [T*K] filled with -1)."""
        lib = _lib.load()
        device = ids.device
        n_tokens, topk = ids.shape
        n_routes = ids.numel()
        first_rank = torch.empty(n_routes, dtype=torch.int32, device=device)
        position = torch.empty(n_routes, dtype=torch.int32, device=device)
        _lib.check(lib.aklr_ep_plan(_ptr(ids), n_tokens, topk, n_local, _ptr(first_rank), _ptr(position), _stream()))
        sorted_ids = torch.empty(n_routes + world, dtype=torch.int32, device=device)
        block_rank = torch.empty(n_routes + world, dtype=torch.int32, device=device)
        counts = torch.empty(world, dtype=torch.int32, device=device)
        num_blocks = torch.empty(2, dtype=torch.int32, device=device)
        scratch = torch.empty(max(1, (n_routes + 1023) // 1024) * world, dtype=torch.int32, device=device)
        _lib.check(
            lib.aklr_moe_align(
                _ptr(first_rank), None, n_routes, world, world, 1, _ptr(sorted_ids), _ptr(block_rank), _ptr(counts),
                _ptr(num_blocks), _ptr(scratch), _stream(),
            )
        )
        return sorted_ids, counts, position, num_blocks

    def pack(self, hidden, ids, weights, plan, n_local, layout: RowLayout):
        """The packed send rows (uint8 [T*K, row_bytes]; the rows past sum(counts) are not written)."""
        lib = _lib.load()
        sorted_ids, _, position, num_blocks = plan
        device = hidden.device
        n_tokens, h = hidden.shape
        topk = ids.shape[1]
        tokens_q = torch.empty((n_tokens, h), dtype=torch.uint8, device=device)
        tokens_scale = torch.empty((n_tokens, layout.scale_bytes), dtype=torch.uint8, device=device)
        if self.mx:
            identity = torch.arange(n_tokens, dtype=torch.int32, device=device)
            _lib.check(lib.aklr_ep_gather_quant_mxfp8(_ptr(hidden), _ptr(identity), n_tokens, h, 1, _ptr(tokens_q), _ptr(tokens_scale), _stream()))
        else:
            _lib.check(lib.aklr_moe_act_quant_fp8(_ptr(hidden), _ptr(tokens_q), _ptr(tokens_scale), n_tokens, h, _stream()))
        packed = torch.empty((n_tokens * topk, layout.row_bytes), dtype=torch.uint8, device=device)
        _lib.check(
            lib.aklr_ep_pack(
                _ptr(tokens_q), _ptr(tokens_scale), _ptr(sorted_ids), _ptr(ids), _ptr(weights), n_tokens * topk, n_tokens, topk, h,
                n_local, int(self.mx), num_blocks[1:].data_ptr(), _ptr(packed), _ptr(position), _stream(),
            )
        )
        return packed

    def experts(self, received, layout: RowLayout, w1, s1, w2, s2):
        """bf16 [n, H]: for each row received, the weighted sum of the local experts its pairs name."""
        lib = _lib.load()
        device = received.device
        n, h, topk = received.shape[0], layout.hidden, layout.topk
        out = torch.empty((n, h), dtype=torch.bfloat16, device=device)
        if n == 0:
            return out
        ids = torch.empty((n, topk), dtype=torch.int32, device=device)
        weights = torch.empty((n, topk), dtype=torch.float32, device=device)
        _lib.check(lib.aklr_ep_unpack_meta(_ptr(received), n, h, topk, int(self.mx), _ptr(ids), _ptr(weights), _stream()))
        e, two_i = w1.shape[0], w1.shape[1]
        base = received.data_ptr()
        if self.mx:
            cfg = _config(n, h, two_i // 2, e, Routing(topk=topk), block_m=128)
            ws = Workspace(cfg, device)
            _lib.check(
                lib.aklr_moe_mxfp4_experts_rows(
                    ctypes.byref(cfg), base, layout.row_bytes, base + h, layout.row_bytes, _ptr(ids), _ptr(weights), _ptr(w1), _ptr(s1),
                    _ptr(w2), _ptr(s2), float(self.swiglu_limit or 0.0), _ptr(out), ws.base.data_ptr(), ws.layout.total_bytes, _stream(),
                )
            )
            return out
        cfg = _config(n, h, two_i // 2, e, Routing(topk=topk))
        ws = Workspace(cfg, device)
        _lib.check(
            lib.aklr_moe_fp8_experts_rows(
                ctypes.byref(cfg), base, layout.row_bytes, base + h, layout.row_bytes, _ptr(ids), _ptr(weights), _ptr(w1), _ptr(s1),
                _ptr(w2), _ptr(s2), _ptr(out), ws.base.data_ptr(), ws.layout.total_bytes, _stream(),
            )
        )
        return out

    def shared(self, hidden, w1, s1, w2, s2):
        """Sum of the shared experts on the rank's own tokens (each at weight 1), bf16 [T, H]."""
        n_tokens, n_shared = hidden.shape[0], w1.shape[0]
        ids = torch.arange(n_shared, dtype=torch.int32, device=hidden.device).repeat(n_tokens, 1).contiguous()
        ones = torch.ones((n_tokens, n_shared), dtype=torch.float32, device=hidden.device)
        if self.mx:
            return fused_experts_mxfp4(hidden, ids, ones, w1, s1, w2, s2, swiglu_limit=self.swiglu_limit)
        return fused_experts_fp8(hidden, ids, ones, w1, s1, w2, s2)

    def combine(self, rows, position, shared_rows, n_tokens, topk, hidden):
        out = torch.empty((n_tokens, hidden), dtype=torch.bfloat16, device=position.device)
        _lib.check(_lib.load().aklr_ep_combine(_ptr(rows), _ptr(position), _ptr(shared_rows), _ptr(out), n_tokens, topk, hidden, _stream()))
        return out

    def side_stream(self, device):
        return torch.cuda.Stream(device=device)


class ExpertParallelMoE:
    """One rank's share of an expert-parallel MoE layer.

    ``w1``/``w2`` (+ scales) hold this rank's ``n_local`` routed experts followed by the layer's
    shared experts (replicated).  ``routing`` describes the whole layer (global expert count =
    ``n_local * world``)."""

    def __init__(self, routing: Routing, w1, w1_scale, w2, w2_scale, rank: int, world: int, kernels=None):
        self.routing = dataclasses.replace(routing, n_shared=0)
        self.n_shared = routing.n_shared
        require_row_major(w1, w2)  # the rank's slices below are views: a tile-contiguous tensor cannot be sliced this way
        self.n_local = w1.shape[0] - self.n_shared
        if self.n_local < 1:
            raise ValueError("w1 must hold at least one routed expert before the shared ones")
        self.rank, self.world = rank, world
        self.kernels = kernels or CudaKernels()
        split = self.n_local
        self.routed = (w1[:split], w1_scale[:split], w2[:split], w2_scale[:split])
        self.shared = (w1[split:], w1_scale[split:], w2[split:], w2_scale[split:]) if self.n_shared else None
        self._side = None

    # ---- phase 1: on the home rank --------------------------------------------------------------
    def prepare(self, hidden: torch.Tensor, logits: torch.Tensor | None, bias: torch.Tensor | None, routed=None) -> StepState:
        """``routed`` = (topk_ids int32 [T,K] global ids, topk_weights float32 [T,K]) skips the routing
        (the reference's mega_moe takes the routing as input)."""
        k = self.kernels
        if routed is None and logits.shape[1] != self.n_local * self.world:
            raise ValueError(f"router has {logits.shape[1]} experts, the group holds {self.n_local * self.world}")
        shared_rows = shared_done = None
        if self.shared is not None:  # overlaps the dispatch: own tokens through the replicated shared experts
            if hidden.is_cuda:
                if self._side is None:
                    self._side = k.side_stream(hidden.device)
                self._side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._side):
                    shared_rows = k.shared(hidden, *self.shared)
                    shared_done = torch.cuda.Event()
                    shared_done.record(self._side)
                hidden.record_stream(self._side)
            else:
                shared_rows = k.shared(hidden, *self.shared)
        ids, weights = routed if routed is not None else k.route(logits, bias, self.routing)
        self.routing = dataclasses.replace(self.routing, topk=ids.shape[1])
        layout = RowLayout(hidden.shape[1], ids.shape[1], bool(getattr(k, "mx", False)))
        plan = k.plan(ids, self.n_local, self.world)
        packed = k.pack(hidden, ids, weights, plan, self.n_local, layout)
        return StepState(packed, plan[1], plan[2], shared_rows, shared_done, hidden.shape[0], layout)

    # ---- phase 2: on the rank that holds the experts ---------------------------------------------
    def compute(self, received: torch.Tensor, layout: RowLayout) -> torch.Tensor:
        return self.kernels.experts(received, layout, *self.routed)

    # ---- phase 3: back home ------------------------------------------------------------------------
    def finish(self, state: StepState, back_rows: torch.Tensor) -> torch.Tensor:
        if state.shared_done is not None:
            torch.cuda.current_stream().wait_event(state.shared_done)
        return self.kernels.combine(back_rows, state.position_of_route, state.shared_rows, state.n_tokens, state.layout.topk, state.layout.hidden)

    def _counts_buffer(self) -> torch.Tensor:
        """Pinned int32 [2, world] for one part's split sizes; a small ring, so that a buffer is not rewritten
        while the host may still be reading the one of a few parts ago."""
        ring = getattr(self, "_counts_ring", None)
        if ring is None:
            ring = self._counts_ring = [torch.zeros((2, self.world), dtype=torch.int32).pin_memory() for _ in range(8)]
            self._counts_next = 0
        self._counts_next = (self._counts_next + 1) % len(ring)
        return ring[self._counts_next]

    # ---- all three over torch.distributed ------------------------------------------------------------
    def forward(self, hidden, logits, bias, group=None, routed=None, micro_batches: int = 1) -> torch.Tensor:
        """``micro_batches`` > 1 splits the tokens into that many consecutive parts whose steps are
        interleaved: all parts are prepared and their counts exchanged first, so that while the host
        reads one part's counts and enqueues its exchange and experts, the GPU still has the other
        parts' work.  Every token's result is the same as with one part."""
        import torch.distributed as dist

        n = hidden.shape[0]
        parts = max(1, min(int(micro_batches), n))
        bounds = [n * i // parts for i in range(parts + 1)]
        pending = []
        for lo, hi in zip(bounds[:-1], bounds[1:]):
            part_routed = None if routed is None else (routed[0][lo:hi], routed[1][lo:hi])
            state = self.prepare(hidden[lo:hi], None if logits is None else logits[lo:hi], bias, part_routed)
            recv_counts_dev = torch.empty_like(state.counts)
            dist.all_to_all_single(recv_counts_dev, state.counts, group=group)
            if recv_counts_dev.is_cuda:
                # the one host read of the part, waited for below: a kernel stores the counts into pinned host
                # memory (a device-to-host copy would queue behind any large copy on the copy engine)
                host = self._counts_buffer()
                _lib.check(_lib.load().aklr_ep_counts_to_host(_ptr(state.counts), _ptr(recv_counts_dev), self.world, host.data_ptr(), _stream()))
                ready = torch.cuda.Event()
                ready.record()
            else:
                host, ready = torch.stack([state.counts, recv_counts_dev]), None
            pending.append((state, host, ready))
        outs = []
        for state, host, ready in pending:
            if ready is not None:
                ready.synchronize()
            send_counts, recv_counts = host[0].tolist(), host[1].tolist()
            n_send, n_recv = sum(send_counts), sum(recv_counts)
            received = torch.empty((n_recv, state.layout.row_bytes), dtype=torch.uint8, device=hidden.device)
            dist.all_to_all_single(received, state.packed[:n_send], output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
            rows = self.compute(received, state.layout)
            back = torch.empty((n_send, rows.shape[1]), dtype=rows.dtype, device=rows.device)
            dist.all_to_all_single(back, rows, output_split_sizes=send_counts, input_split_sizes=recv_counts, group=group)
            outs.append(self.finish(state, back))
        return outs[0] if len(outs) == 1 else torch.cat(outs)


def exchange_in_process(states: list[StepState]) -> tuple[list[torch.Tensor], list[list[int]]]:
    """The dispatch among ranks that live in one process (tests, single-GPU emulation): what each rank
    receives (rows ordered by source rank) and each rank's send counts."""
    world = len(states)
    counts = [s.counts.cpu().tolist() for s in states]
    starts = [[sum(c[:d]) for d in range(world)] for c in counts]
    received = []
    for dst in range(world):
        parts = [states[src].packed[starts[src][dst] : starts[src][dst] + counts[src][dst]] for src in range(world)]
        received.append(torch.cat(parts))
    return received, counts


def exchange_back_in_process(rows_per_rank: list[torch.Tensor], counts: list[list[int]]) -> list[torch.Tensor]:
    """Rows computed on each rank returned to the ranks that sent them, in their send order."""
    world = len(rows_per_rank)
    back = []
    for home in range(world):
        parts = []
        for holder in range(world):
            start = sum(counts[src][holder] for src in range(home))
            parts.append(rows_per_rank[holder][start : start + counts[home][holder]])
        back.append(torch.cat(parts))
    return back


def run_in_process(layers: list[ExpertParallelMoE], inputs: list[tuple]) -> list[torch.Tensor]:
    """All ranks' steps in one process: phase by phase, never two ranks' kernels waiting on each other."""
    states = [layer.prepare(*inp) for layer, inp in zip(layers, inputs)]
    received, counts = exchange_in_process(states)
    rows = [layer.compute(r, s.layout) for layer, r, s in zip(layers, received, states)]
    back = exchange_back_in_process(rows, counts)
    return [layer.finish(s, b) for layer, s, b in zip(layers, states, back)]
