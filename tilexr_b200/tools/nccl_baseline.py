"""The baseline this repository is measured against: the same MoE dispatch + combine written
with stock PyTorch ops and NCCL ``all_to_all_single`` (routing, fp8 1x128 quantisation, sort by
expert, count exchange, payload exchange, dequantisation, exchange back, weighted un-permute).
None of this repository's kernels run on this path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class NcclMoEBaseline:
    def __init__(self, world: int, rank: int, num_experts: int, top_k: int, device):
        self.world, self.rank, self.E, self.K, self.dev = world, rank, num_experts, top_k, device
        self.per = num_experts // world

    def _a2a(self, send, send_counts, recv_counts):
        if self.world == 1:
            return send
        out = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
        dist.all_to_all_single(out, send, output_split_sizes=recv_counts, input_split_sizes=send_counts)
        return out

    @torch.no_grad()
    def step(self, x: torch.Tensor, logits: torch.Tensor, ev=None):
        T, H = x.shape
        if ev is not None:
            ev[0].record()
        scores = torch.sigmoid(logits)
        w, ids = torch.topk(scores, self.K, dim=-1)
        w = w / w.sum(dim=-1, keepdim=True)
        # fp8 1x128 quantisation
        g = x.float().view(T, H // 128, 128)
        amax = g.abs().amax(dim=-1).clamp_min(1e-4)
        q = (g * (448.0 / amax).unsqueeze(-1)).to(torch.float8_e4m3fn).view(T, H)
        scales = amax / 448.0
        # permute routes by expert (stable), exchange counts, then payload
        flat = ids.reshape(-1)
        order = torch.argsort(flat, stable=True)
        token = order // self.K
        per_expert = torch.bincount(flat, minlength=self.E)
        send_counts = per_expert.view(self.world, self.per).sum(dim=1)
        if self.world > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts)
        else:
            recv_counts = send_counts
        sc, rc = send_counts.tolist(), recv_counts.tolist()      # the host sync NCCL's API forces
        payload = self._a2a(q[token].view(torch.uint8), sc, rc).view(torch.float8_e4m3fn)
        rscales = self._a2a(scales[token], sc, rc)
        if ev is not None:
            ev[1].record()
        rows = (payload.float().view(-1, H // 128, 128) * rscales.unsqueeze(-1)).view(-1, H).to(torch.bfloat16)
        if ev is not None:
            ev[2].record()
        back = self._a2a(rows, rc, sc)
        y = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        y.index_add_(0, token, back.float() * w.reshape(-1)[order].unsqueeze(1))
        y = y.to(torch.bfloat16)
        if ev is not None:
            ev[3].record()
        return y
