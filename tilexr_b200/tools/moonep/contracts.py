"""Data contracts of the MoonEP harness (reference: tools/moonep/contracts.py).

A *case* fixes the problem shape and the seed; *inputs* are one rank's tensors; a *backend* runs the five
stages for one rank; *artifacts* are what the correctness runner compares, stage by stage.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Protocol

import torch


@dataclasses.dataclass(frozen=True)
class MoonEPCase:
    name: str
    ranks: int            # R
    tokens: int           # S per rank
    hidden: int           # H
    top_k: int            # K
    experts: int          # E (global)
    prefetch_slots: int   # B
    token_padding: int = 1
    ffn: int = 0          # expert FFN width for the projection tensors (0: no prefetch / reduce-grad stages)
    skew: float = 10.0    # weight of the hot experts in the routing distribution (1.0 = uniform)
    seed: int = 0
    dtype: str = "bfloat16"

    @property
    def routes(self) -> int:
        return self.tokens * self.top_k

    @property
    def local_experts(self) -> int:
        return self.experts // self.ranks

    @property
    def nvs(self) -> int:
        return self.routes + (self.token_padding - 1) * 2 * self.local_experts

    def torch_dtype(self) -> torch.dtype:
        return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[self.dtype]

    def validate(self) -> None:
        if self.experts % self.ranks != 0:
            raise ValueError("E must divide by R")
        if not 1 <= self.prefetch_slots <= self.local_experts:
            raise ValueError("1 <= B <= E/R")
        if self.top_k > 32:
            raise ValueError("K <= 32")
        if self.ranks * self.nvs >= 2 ** 31:
            raise ValueError("R * NvS must fit 31 bits")


@dataclasses.dataclass
class RankInputs:
    """One rank's inputs.  Backends must not modify them (the runner checks)."""
    hidden_sh: torch.Tensor              # [S, H]
    route_weights_sk: torch.Tensor       # [S, K] fp32
    topk_experts_sk: torch.Tensor        # [S, K] int32
    gate: Optional[torch.Tensor] = None  # [E/R, ffn, H]   own experts' projection rows
    up: Optional[torch.Tensor] = None
    down: Optional[torch.Tensor] = None
    grad_rows: Optional[torch.Tensor] = None   # [E/R + B, ffn, H] fp32: gradients incl. the borrowed slots


@dataclasses.dataclass
class StageArtifacts:
    """What one rank produced, keyed the same way by every backend."""
    plan: Dict[str, torch.Tensor]
    dispatched_hidden: torch.Tensor              # [NvS, H]
    dispatched_weights: torch.Tensor             # [NvS]
    prefetched_gate: Optional[torch.Tensor]      # [E/R + B, ...]
    combined_hidden: torch.Tensor                # [S, H]
    combined_weights: torch.Tensor               # [S, K]
    reduced_grad: Optional[torch.Tensor]         # [E/R + B, ...] fp32

    STAGES = ("plan", "dispatched_hidden", "dispatched_weights", "prefetched_gate", "combined_hidden",
              "combined_weights", "reduced_grad")


class MoonEPBackend(Protocol):
    """One rank of an implementation of the five stages."""

    name: str

    def run(self, case: MoonEPCase, inputs: RankInputs) -> StageArtifacts: ...

    def close(self) -> None: ...
