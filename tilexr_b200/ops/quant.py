"""Quantisation, routing and normalisation kernels (local ops, no communicator)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _C

SCORE_SOFTMAX = 0
SCORE_SIGMOID = 1


def fp8_quant_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 values and fp32 scales ``[rows, h/128]``; ``x ~= y.float() * scale``."""
    return _C.fp8_quant_1x128(x.contiguous())


def fp8_dequant_1x128(y: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return _C.fp8_dequant_1x128(y, scales, dtype)


def mxfp8_quant(x: torch.Tensor, e5m2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """OCP MXFP8: 32-element blocks with a shared E8M0 exponent (uint8, bias 127)."""
    return _C.mxfp8_quant(x.contiguous(), e5m2)


def mxfp8_dequant(y: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return _C.mxfp8_dequant(y, scales, dtype)


def routing_topk(gate_logits: torch.Tensor, top_k: int, score_func: int = SCORE_SOFTMAX, renormalize: bool = True,
                 routed_scale: float = 1.0, selection_bias: Optional[torch.Tensor] = None):
    return _C.routing_topk(gate_logits.contiguous(), selection_bias, top_k, score_func, renormalize, routed_scale)


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = norm(x (+ residual)) * gamma``; with ``residual`` the sum is written back into it."""
    return _C.rmsnorm(x.contiguous(), residual, gamma, eps)
