"""Grouped expert FFN on dispatched rows: GEMM -> SwiGLU -> GEMM per expert segment (reference:
tools/moonep/expert_forward.py).  `cu_seqlens[j]` is the end row of segment j; segments `[0, E/R)` are the
rank's own experts and `[E/R, E/R + B)` the prefetch slots, whose weights sit at the same row index of the
projection tensors."""
from __future__ import annotations

import torch


def expert_forward(rows: torch.Tensor, cu_seqlens: torch.Tensor, gate: torch.Tensor, up: torch.Tensor,
                   down: torch.Tensor) -> torch.Tensor:
    """rows [NvS, H]; gate/up [segments, F, H]; down [segments, F, H] (used transposed).  Rows past the last
    segment end stay zero."""
    out = torch.zeros_like(rows)
    ends = cu_seqlens.to(torch.int64).tolist()
    start = 0
    for j, end in enumerate(ends[: gate.shape[0]]):
        if end > start:
            seg = rows[start:end].to(gate.dtype)
            g = seg @ gate[j].t()
            u = seg @ up[j].t()
            out[start:end] = ((torch.nn.functional.silu(g.float()) * u.float()).to(gate.dtype) @ down[j]).to(rows.dtype)
        start = max(start, end)
    return out
