"""Token-dispatcher adapter for Megatron-Core style MoE layers (the role of the reference's MindSpeed adapter,
tools/moonep/mindspeed/tilexr_mindspeed_adapter.py:1-722, which bridges MindSpeed's private Buffer contracts to the
TileXR stages).

Megatron-Core's ``MoETokenDispatcher`` contract is two calls around the experts:

    dispatched, tokens_per_expert = dispatcher.token_permutation(hidden_states, probs, top_indices)
    expert_out = experts(dispatched, tokens_per_expert)            # grouped GEMMs over rows sorted by local expert
    output, _ = dispatcher.token_unpermutation(expert_out)

This adapter serves it with the fused kernels: ``token_permutation`` is one dispatch kernel (rows arrive sorted by
local expert, exactly the layout grouped GEMMs want), ``token_unpermutation`` is one combine kernel (gate-weighted sum in
fp32 and un-permutation).  No all-to-all, sort, or index_select runs in PyTorch.  The context of a step (what the
reference's adapter keeps in its ``ctx`` dict) is the ``DispatchResult`` held between the two calls; ``ctx()`` exposes
it for code that wants to run its own backward.

The adapter does not import Megatron or MindSpeed: it has the same method names and tensor conventions, so a
``MoELayer`` can be given it as its ``token_dispatcher``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ops import ep


class TileXRTokenDispatcher:
    def __init__(self, comm, num_experts: int, top_k: int, hidden_size: int, *, quant_mode: int = ep.QUANT_NONE,
                 max_tokens_per_rank: Optional[int] = None, dedup: Optional[bool] = None):
        if num_experts % comm.world_size != 0:
            raise ValueError("num_experts must be a multiple of the expert-parallel world size")
        self.comm = comm
        self.num_experts = num_experts
        self.num_local_experts = num_experts // comm.world_size
        self.top_k = top_k
        self.hidden_size = hidden_size
        self.quant_mode = quant_mode
        self.max_tokens_per_rank = max_tokens_per_rank
        self.dedup = dedup
        self._ctx: Optional[ep.DispatchResult] = None
        self._shape: Optional[torch.Size] = None
        self._probs: Optional[torch.Tensor] = None

    # ---- Megatron-Core names ---------------------------------------------------------------------------------
    def token_permutation(self, hidden_states: torch.Tensor, probs: torch.Tensor,
                          top_indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``hidden_states`` [s, b, h] or [tokens, h]; ``probs`` and ``top_indices`` [tokens, top_k].

        Returns the rows this rank's experts compute, sorted by local expert ([capacity, h]; rows past the sum of
        ``tokens_per_expert`` are unused), and ``tokens_per_expert`` [num_local_experts] (int64, on the device)."""
        self._shape = hidden_states.shape
        x = hidden_states.reshape(-1, hidden_states.shape[-1]).contiguous()
        tokens = x.shape[0]
        if self.max_tokens_per_rank is not None and tokens > self.max_tokens_per_rank:
            raise ValueError(f"{tokens} tokens exceed max_tokens_per_rank={self.max_tokens_per_rank}")
        cap_tokens = self.max_tokens_per_rank if self.max_tokens_per_rank is not None else tokens
        max_rows = cap_tokens * self.comm.world_size * min(self.top_k, self.num_local_experts)
        self._probs = probs.to(torch.float32).contiguous()
        self._ctx = ep.dispatch(self.comm, x, num_experts=self.num_experts, top_k=self.top_k,
                                expert_ids=top_indices.to(torch.int32).contiguous(), expert_scales=self._probs,
                                quant_mode=self.quant_mode, max_recv_rows=max_rows, dedup=self.dedup)
        return self._ctx.expand_x, self._ctx.expert_token_nums

    def token_unpermutation(self, expert_output: torch.Tensor, bias: Optional[torch.Tensor] = None):
        """``expert_output`` [capacity, h] in the row order ``token_permutation`` returned.  Returns (output, None) with
        ``output`` in the shape of the original ``hidden_states``: sum over the token's experts of prob * expert row."""
        if self._ctx is None:
            raise RuntimeError("token_unpermutation without a preceding token_permutation")
        if bias is not None:
            raise NotImplementedError("expert bias is added by the expert, before the combine")
        y = ep.combine(self.comm, expert_output.contiguous(), self._ctx, expert_scales=self._probs)
        out = y.reshape(self._shape)
        self._ctx = None
        return out, None

    # ---- extras ------------------------------------------------------------------------------------------------
    def ctx(self) -> Optional[ep.DispatchResult]:
        """The step's routing context between the two calls (source rank, token, slot and expert of every row)."""
        return self._ctx

    def dispatched_scales(self) -> Optional[torch.Tensor]:
        """Per-row (or per-block) dequantisation scales when the dispatch quantised the rows."""
        return None if self._ctx is None else self._ctx.dynamic_scales
