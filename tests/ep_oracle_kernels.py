"""CPU stand-in for the device side of the expert-parallel phases, built on the oracle: lets the
host logic (ownership, split sizes, ordering, the exchanges) run over gloo without a GPU."""

from __future__ import annotations

import torch

from oracle import moe_oracle as orc


class OracleKernels:
    def route(self, logits, bias, routing):
        if routing.scoring == "sigmoid":
            ids, w = orc.grouped_sigmoid_topk(
                logits.float(), bias.float(), routing.topk, routing.num_expert_group, routing.topk_group,
                routing.renormalize, routing.routed_scaling_factor,
            )
        else:
            ids, w = orc.softmax_topk(logits.float(), routing.topk)
        return ids.to(torch.int32), w.float()

    def order_by_rank(self, ids, n_local, world):
        ranks = (ids.reshape(-1).long() // n_local)
        order = torch.sort(ranks, stable=True).indices.to(torch.int32)
        return order, torch.bincount(ranks, minlength=world).to(torch.int32)

    def pack(self, hidden, ids, weights, sorted_ids, n_local):
        tokens = sorted_ids.long() // ids.shape[1]
        codes, scales = orc.fp8_group_quant(hidden.float()[tokens])
        flat_ids, flat_w = ids.reshape(-1)[sorted_ids.long()], weights.reshape(-1)[sorted_ids.long()]
        meta = torch.stack([(flat_ids % n_local).to(torch.int32), flat_w.contiguous().view(torch.int32)], dim=1).contiguous()
        position = torch.full((ids.numel(),), -1, dtype=torch.int32)
        position[sorted_ids.long()] = torch.arange(sorted_ids.numel(), dtype=torch.int32)
        return codes.view(torch.uint8), scales, meta, position

    @staticmethod
    def _mlp_rows(xq, w1, s1, w2, s2, expert_ids):
        out = torch.zeros_like(xq)
        for e in expert_ids.unique().tolist():
            rows = (expert_ids == e).nonzero().flatten()
            gate, up = (xq[rows] @ orc.dequant_block_weight(w1[e], s1[e]).T).chunk(2, dim=-1)
            out[rows] = orc.fp8_input(torch.nn.functional.silu(gate) * up) @ orc.dequant_block_weight(w2[e], s2[e]).T
        return out

    def experts(self, rows_q, rows_scale, expert_ids, weights, w1, s1, w2, s2):
        codes = rows_q.view(orc.FP8).float()
        xq = (codes.unflatten(-1, (-1, 128)) * rows_scale.unsqueeze(-1)).flatten(-2)
        y = self._mlp_rows(xq, w1, s1, w2, s2, expert_ids.long())
        return (y * weights.unsqueeze(-1)).to(torch.bfloat16)

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
