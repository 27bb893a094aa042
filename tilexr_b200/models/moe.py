"""Expert-parallel MoE layer built on the fused dispatch / combine kernels.

The reference ships no model code; its harness drives dispatch -> expert FFN (grouped GEMM,
SwiGLU, grouped GEMM) -> combine with synthetic experts (tools/moonep/expert_forward.py).  This
module is the same workload as a reusable layer, shaped like a DeepSeek-V3 MoE block: sigmoid
router with top-k renormalisation, fp8 (e4m3, 1x128 scales) token transport, bf16 combine.
The expert feed-forward is two launches of this repository's grouped tcgen05 GEMM over all local experts at
once -- the first with the SwiGLU activation in its epilogue -- driven by the per-expert row counts that dispatch
left on the device, so nothing is read back to the host between dispatch and combine; the communication, routing,
quantisation and the gate-weighted reduction are this repository's kernels too.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..ops import ep, gemm, quant


@dataclasses.dataclass
class MoEConfig:
    hidden: int = 7168
    ffn: int = 2048
    num_experts: int = 256
    top_k: int = 8
    score_func: int = quant.SCORE_SIGMOID
    renormalize: bool = True
    routed_scale: float = 1.0
    fp8_dispatch: bool = True
    dtype: torch.dtype = torch.bfloat16


class ExpertParallelMoE(torch.nn.Module):
    """One MoE block whose experts are sharded over the ranks of ``comm``."""

    def __init__(self, comm, cfg: MoEConfig, device="cuda", seed: int = 0, with_experts: bool = True):
        super().__init__()
        self.comm = comm
        self.cfg = cfg
        assert cfg.num_experts % comm.world_size == 0
        self.local_experts = cfg.num_experts // comm.world_size
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.gate = torch.nn.Parameter((torch.randn(cfg.num_experts, cfg.hidden, generator=g) * 0.02).to(torch.float32).to(device))
        if with_experts:
            ge = torch.Generator(device="cpu").manual_seed(seed + 1 + comm.rank)
            self.w13 = torch.nn.Parameter(
                (torch.randn(self.local_experts, 2 * cfg.ffn, cfg.hidden, generator=ge) * 0.02).to(cfg.dtype).to(device))
            self.w2 = torch.nn.Parameter(
                (torch.randn(self.local_experts, cfg.hidden, cfg.ffn, generator=ge) * 0.02).to(cfg.dtype).to(device))
        else:
            self.w13 = None
            self.w2 = None

    def route_logits(self, x: torch.Tensor) -> torch.Tensor:
        return torch.matmul(x.float(), self.gate.t()).contiguous()

    def experts(self, rows: torch.Tensor, token_nums: torch.Tensor) -> torch.Tensor:
        """SwiGLU feed-forward over rows that arrive grouped by local expert; ``token_nums`` (int64, on the device) holds
        the rows per expert.  ``w13[e]`` is [2 * ffn, hidden] with gate row i at 2i and up row i at 2i + 1."""
        if self.w13 is None:
            return rows.clone()
        mid = gemm.grouped_matmul(rows, self.w13, token_nums, epilogue=gemm.EPILOGUE_SWIGLU)
        return gemm.grouped_matmul(mid, self.w2, token_nums)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, gate_logits: Optional[torch.Tensor] = None, max_recv_rows: Optional[int] = None,
                expand_x_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        cfg = self.cfg
        if gate_logits is None:
            gate_logits = self.route_logits(x)
        d = ep.dispatch(self.comm, x, gate_logits=gate_logits, num_experts=cfg.num_experts, top_k=cfg.top_k,
                        quant_mode=ep.QUANT_FP8_1X128 if cfg.fp8_dispatch else ep.QUANT_NONE, score_func=cfg.score_func,
                        renormalize=cfg.renormalize, routed_scale=cfg.routed_scale, max_recv_rows=max_recv_rows,
                        expand_x_out=expand_x_out)
        rows = quant.fp8_dequant_1x128(d.expand_x, d.dynamic_scales, cfg.dtype) if cfg.fp8_dispatch else d.expand_x
        out = self.experts(rows, d.expert_token_nums) if self.w13 is not None else rows
        return ep.combine(self.comm, out, d, expert_scales=d.topk_weights)
