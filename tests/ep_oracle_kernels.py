"""CPU stand-in for the device side of the expert-parallel phases, built on the oracle: lets the
host logic (ownership, one row per (token, rank), the packed row layout, split sizes, the exchanges)
run over gloo without a GPU."""

from __future__ import annotations

import torch

from oracle import moe_oracle as orc


class OracleKernels:
    mx = False

    def route(self, logits, bias, routing):
        if routing.scoring == "sigmoid":
            ids, w = orc.grouped_sigmoid_topk(
                logits.float(), bias.float(), routing.topk, routing.num_expert_group, routing.topk_group,
                routing.renormalize, routing.routed_scaling_factor,
            )
        else:
            ids, w = orc.softmax_topk(logits.float(), routing.topk)
        return ids.to(torch.int32), w.float()

    def plan(self, ids, n_local, world):
        n_tokens, topk = ids.shape
        ranks = ids.long() // n_local
        first = torch.ones_like(ranks, dtype=torch.bool)
        for s in range(1, topk):  # a slot is a first slot when no earlier slot of its token goes to the same rank
            first[:, s] = ~(ranks[:, :s] == ranks[:, s : s + 1]).any(dim=1)
        first &= ids >= 0
        first_rank = torch.where(first, ranks, torch.full_like(ranks, -1)).reshape(-1)
        routes = first.reshape(-1).nonzero().flatten()
        order = routes[torch.sort(first_rank[routes], stable=True).indices].to(torch.int32)
        sorted_ids = torch.full((n_tokens * topk + world,), -1, dtype=torch.int32)
        sorted_ids[: order.numel()] = order
        counts = torch.bincount(first_rank[routes], minlength=world).to(torch.int32)
        position = torch.full((n_tokens * topk,), -1, dtype=torch.int32)
        return sorted_ids, counts, position, torch.tensor([order.numel(), order.numel()], dtype=torch.int32)

    def pack(self, hidden, ids, weights, plan, n_local, layout):
        sorted_ids, _, position, num_blocks = plan
        n_send, topk, h = int(num_blocks[1]), ids.shape[1], hidden.shape[1]
        rids = sorted_ids[:n_send].long()
        tokens = rids // topk
        codes, scales = orc.fp8_group_quant(hidden.float())
        packed = torch.zeros((ids.numel(), layout.row_bytes), dtype=torch.uint8)
        packed[:n_send, :h] = codes.view(torch.uint8)[tokens]
        packed[:n_send, h : layout.meta_offset] = scales.contiguous().view(torch.uint8).reshape(hidden.shape[0], -1)[tokens]
        rank = (ids.reshape(-1)[rids].long() // n_local).unsqueeze(1)
        here = (ids[tokens].long() // n_local == rank) & (ids[tokens] >= 0)
        local = torch.where(here, ids[tokens] % n_local, torch.full_like(ids[tokens], -1)).to(torch.int32)
        w = torch.where(here, weights[tokens], torch.zeros_like(weights[tokens])).float()
        packed[:n_send, layout.meta_offset : layout.meta_offset + 4 * topk] = local.contiguous().view(torch.uint8).reshape(n_send, -1)
        packed[:n_send, layout.meta_offset + 4 * topk : layout.meta_offset + 8 * topk] = w.contiguous().view(torch.uint8).reshape(n_send, -1)
        position[rids] = torch.arange(n_send, dtype=torch.int32)
        return packed

    @staticmethod
    def _mlp_rows(xq, w1, s1, w2, s2, expert_ids):
        out = torch.zeros_like(xq)
        for e in expert_ids.unique().tolist():
            rows = (expert_ids == e).nonzero().flatten()
            gate, up = (xq[rows] @ orc.dequant_block_weight(w1[e], s1[e]).T).chunk(2, dim=-1)
            out[rows] = orc.fp8_input(torch.nn.functional.silu(gate) * up) @ orc.dequant_block_weight(w2[e], s2[e]).T
        return out

    def experts(self, received, layout, w1, s1, w2, s2):
        n, h, topk = received.shape[0], layout.hidden, layout.topk
        codes = received[:, :h].contiguous().view(orc.FP8).float()
        scales = received[:, h : layout.meta_offset].contiguous().view(torch.float32)
        ids = received[:, layout.meta_offset : layout.meta_offset + 4 * topk].contiguous().view(torch.int32)
        weights = received[:, layout.meta_offset + 4 * topk : layout.meta_offset + 8 * topk].contiguous().view(torch.float32)
        xq = (codes.unflatten(-1, (-1, 128)) * scales.unsqueeze(-1)).flatten(-2)
        total = torch.zeros((n, h))
        for s in range(topk):  # slot order, each route's row rounded to bf16 before the float32 sum, as the kernels do
            live = (ids[:, s] >= 0).nonzero().flatten()
            if live.numel():
                y = self._mlp_rows(xq[live], w1, s1, w2, s2, ids[live, s].long())
                total[live] += (y * weights[live, s : s + 1]).to(torch.bfloat16).float()
        return total.to(torch.bfloat16)

    def shared(self, hidden, w1, s1, w2, s2):
        xq = orc.fp8_input(hidden.float())
        total = torch.zeros_like(xq)
        for e in range(w1.shape[0]):
            total += self._mlp_rows(xq, w1, s1, w2, s2, torch.full((hidden.shape[0],), e)).to(torch.bfloat16).float()
        return total.to(torch.bfloat16)

    def combine(self, rows, position, shared_rows, n_tokens, topk, hidden):
        picked = rows.float()[position.long().clamp_min(0)] * (position >= 0).unsqueeze(-1)
        out = picked.view(n_tokens, topk, hidden).sum(dim=1)
        if shared_rows is not None:
            out = out + shared_rows.float()
        return out.to(torch.bfloat16)
