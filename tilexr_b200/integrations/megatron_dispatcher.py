"""Token-dispatcher adapter for Megatron-Core style MoE layers (the role of the reference's MindSpeed adapter,
tools/moonep/mindspeed/tilexr_mindspeed_adapter.py:1-722, which bridges MindSpeed's private Buffer contracts to the
TileXR stages, with its stage barrier tools/moonep/mindspeed/mindspeed_stage_barrier.py and its route capture / replay
tools/moonep/mindspeed/build_route_replay.py).

Megatron-Core's ``MoETokenDispatcher`` contract is two calls around the experts:

    dispatched, tokens_per_expert = dispatcher.token_permutation(hidden_states, probs, top_indices)
    expert_out = experts(dispatched, tokens_per_expert)            # grouped GEMMs over rows sorted by local expert
    output, _ = dispatcher.token_unpermutation(expert_out)

This adapter serves it with the fused kernels: ``token_permutation`` is one dispatch kernel (rows arrive sorted by
local expert, exactly the layout grouped GEMMs want), ``token_unpermutation`` is one combine kernel (gate-weighted sum in
fp32 and un-permutation).  No all-to-all, sort, or index_select runs in PyTorch.

Training.  Both calls are ``torch.autograd.Function``s, so a loss behind the layer back-propagates through them with
the same two kernels in swapped roles:

    d loss / d expert_out[row]   = prob(row) * grad_y[token(row)]       a dispatch of grad_y; the gate weight of every
                                                                       row travels with it (``expand_scales``)
    d loss / d prob[token, k]    = < grad_y[token], expert_out[row(token, k)] >   the dot product is taken on the expert
                                                                       rank, where both vectors are, and returns through
                                                                       a combine of 2K-wide rows that hold it at column k
                                                                       as a bf16 (high, low) pair
    d loss / d hidden[token]     = sum over k of grad_rows[row(token, k)]          a combine with unit weights

The context of a step (what the reference's adapter keeps in its ``ctx`` dict) is the ``DispatchResult`` held between
the two calls; ``ctx()`` exposes it.

Tools around the two calls, as in the reference's adapter:

  * ``stage_barrier`` (or ``TILEXR_MEGATRON_STAGE_BARRIER=1``): a device synchronisation and a host barrier of the ranks
    in front of every stage, so that a per-stage timer measures the stage and not the skew its peers arrived with.
  * ``RouteRecorder`` / ``RouteReplay``: the routing of every step (top-k indices and probabilities) written to one file
    per rank, and a dispatcher fed from such a file instead of the router, so that two runs (or two implementations)
    see identical traffic.

The adapter does not import Megatron or MindSpeed: it has the same method names and tensor conventions, so a
``MoELayer`` can be given it as its ``token_dispatcher``.  The kernels are reached through ``ops`` (default
``tilexr_b200.ops.ep``), which a test can replace by any object with the same ``dispatch`` / ``combine``.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import List, Optional, Tuple

import torch

from ..ops import ep as _ep


class _Permute(torch.autograd.Function):
    """rows = dispatch(hidden); backward: grad_hidden = combine(grad_rows) with unit weights."""

    @staticmethod
    def forward(ctx, hidden, owner):
        d = owner._dispatch(hidden, owner._probs)
        ctx.owner, ctx.d = owner, d
        ctx.mark_non_differentiable(d.expert_token_nums)
        rows = d.expand_x
        if rows.dtype != hidden.dtype:          # quantised transport: the rows come back in the activation type
            rows = owner._dequantise(d, hidden.dtype)
        return rows, d.expert_token_nums

    @staticmethod
    def backward(ctx, grad_rows, _grad_counts):
        owner, d = ctx.owner, ctx.d
        owner._barrier()
        plain = dataclasses.replace(d, dedup=False)       # unit weights: the rows of a token are summed at the origin
        grad_hidden = owner.ops.combine(owner.comm, grad_rows.contiguous(), plain, expert_scales=None)
        return grad_hidden, None


class _Unpermute(torch.autograd.Function):
    """y = combine(expert_out, probs); backward: the two products of the rule y[t] = sum_k p[t, k] * out[row(t, k)]."""

    @staticmethod
    def forward(ctx, expert_out, probs, owner, d):
        ctx.owner, ctx.d = owner, d
        ctx.save_for_backward(expert_out, probs)
        return owner.ops.combine(owner.comm, expert_out.contiguous(), d, expert_scales=probs)

    @staticmethod
    def backward(ctx, grad_y):
        owner, d = ctx.owner, ctx.d
        expert_out, probs = ctx.saved_tensors
        owner._barrier()
        # grad_y goes where the tokens went; the gate weight of every row arrives beside it
        g = owner.ops.dispatch(owner.comm, grad_y.contiguous(), num_experts=owner.num_experts, top_k=owner.top_k,
                               expert_ids=owner._ids, expert_scales=probs, quant_mode=_ep.QUANT_NONE,
                               max_recv_rows=d.expand_x.shape[0], dedup=False, tp_world_size=owner.tp_world_size)
        rows = d.expand_x.shape[0]
        grad_out = (g.expand_x.float() * g.expand_scales[:rows].unsqueeze(1)).to(expert_out.dtype)
        grad_probs = None
        if ctx.needs_input_grad[1]:
            # <grad_y[token], out[row]> per row, placed at column k of a 2K-wide row as a (high, low) bf16 pair, summed at
            # the origin with unit weights: column k of the result is the dot product of route (token, k)
            K = owner.top_k * owner.tp_world_size
            width = max(256, (2 * K + 7) // 8 * 8)       # rows of at least 512 bytes, the width the kernels are tuned for
            dots = (g.expand_x.float() * expert_out.float()).sum(dim=1)
            high = dots.to(torch.bfloat16)
            low = (dots - high.float()).to(torch.bfloat16)
            slot = g.assist[:, 2].long().clamp(0, K - 1)
            wide = torch.zeros(rows, width, dtype=torch.bfloat16, device=dots.device)
            wide.scatter_(1, (2 * slot).unsqueeze(1), high.unsqueeze(1))
            wide.scatter_(1, (2 * slot + 1).unsqueeze(1), low.unsqueeze(1))
            back = owner.ops.combine(owner.comm, wide, dataclasses.replace(g, dedup=False), expert_scales=None).float()
            per_slot = back[:, 0:2 * K:2] + back[:, 1:2 * K:2]
            # tensor-parallel lanes hold slices of one route: their dot products add up
            grad_probs = per_slot.view(-1, owner.top_k, owner.tp_world_size).sum(dim=2).to(probs.dtype)
        return grad_out, grad_probs, None, None


class TileXRTokenDispatcher:
    def __init__(self, comm, num_experts: int, top_k: int, hidden_size: int, *, quant_mode: int = _ep.QUANT_NONE,
                 max_tokens_per_rank: Optional[int] = None, dedup: Optional[bool] = None, tp_world_size: int = 1,
                 stage_barrier: Optional[bool] = None, recorder: Optional["RouteRecorder"] = None, ops=None):
        groups = comm.world_size // tp_world_size
        if comm.world_size % tp_world_size != 0 or num_experts % groups != 0:
            raise ValueError("the tensor-parallel size must divide the ranks, and the expert groups the experts")
        self.comm = comm
        self.ops = ops if ops is not None else _ep
        self.num_experts = num_experts
        self.num_local_experts = num_experts // groups
        self.top_k = top_k
        self.hidden_size = hidden_size
        self.quant_mode = quant_mode
        self.max_tokens_per_rank = max_tokens_per_rank
        self.dedup = dedup
        self.tp_world_size = tp_world_size
        self.stage_barrier = os.environ.get("TILEXR_MEGATRON_STAGE_BARRIER", "0") == "1" if stage_barrier is None else stage_barrier
        self.recorder = recorder
        self._ctx: Optional[_ep.DispatchResult] = None
        self._shape: Optional[torch.Size] = None
        self._probs: Optional[torch.Tensor] = None
        self._ids: Optional[torch.Tensor] = None

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
        self._ids = top_indices.to(torch.int32).contiguous()
        self._probs = probs if probs.dtype == torch.float32 and probs.is_contiguous() else probs.to(torch.float32).contiguous()
        if self.recorder is not None:
            self.recorder.record(self._ids, self._probs)
        self._barrier()
        rows, counts = _Permute.apply(x, self)
        return rows, counts

    def token_unpermutation(self, expert_output: torch.Tensor, bias: Optional[torch.Tensor] = None):
        """``expert_output`` [capacity, h] in the row order ``token_permutation`` returned.  Returns (output, None) with
        ``output`` in the shape of the original ``hidden_states``: sum over the token's experts of prob * expert row."""
        if self._ctx is None:
            raise RuntimeError("token_unpermutation without a preceding token_permutation")
        if bias is not None:
            raise NotImplementedError("expert bias is added by the expert, before the combine")
        self._barrier()
        y = _Unpermute.apply(expert_output, self._probs, self, self._ctx)
        out = y.reshape(self._shape)
        self._ctx = None
        return out, None

    # ---- extras ------------------------------------------------------------------------------------------------
    def ctx(self) -> Optional[_ep.DispatchResult]:
        """The step's routing context between the two calls (source rank, token, slot and expert of every row)."""
        return self._ctx

    def dispatched_scales(self) -> Optional[torch.Tensor]:
        """Per-row (or per-block) dequantisation scales when the dispatch quantised the rows."""
        return None if self._ctx is None else self._ctx.dynamic_scales

    # ---- internals ---------------------------------------------------------------------------------------------
    def _dispatch(self, x: torch.Tensor, probs: torch.Tensor):
        tokens = x.shape[0]
        cap_tokens = self.max_tokens_per_rank if self.max_tokens_per_rank is not None else tokens
        max_rows = cap_tokens * self.comm.world_size * min(self.top_k, self.num_local_experts)
        self._ctx = self.ops.dispatch(self.comm, x, num_experts=self.num_experts, top_k=self.top_k, expert_ids=self._ids,
                                      expert_scales=probs.detach(), quant_mode=self.quant_mode, max_recv_rows=max_rows,
                                      dedup=self.dedup, tp_world_size=self.tp_world_size)
        return self._ctx

    def _dequantise(self, d, dtype):
        from ..ops import quant

        if self.quant_mode == _ep.QUANT_FP8_1X128:
            return quant.fp8_dequant_1x128(d.expand_x, d.dynamic_scales, dtype)
        if self.quant_mode in (_ep.QUANT_MXFP8_E4M3, _ep.QUANT_MXFP8_E5M2):
            return quant.mxfp8_dequant(d.expand_x, d.dynamic_scales).to(dtype)
        raise NotImplementedError("the int8 transports hand their rows to an int8 expert; there is no activation to return")

    def _barrier(self):
        if not self.stage_barrier:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        barrier = getattr(self.comm, "barrier", None)
        if barrier is not None:
            barrier()


class RouteRecorder:
    """Writes the routing of every step of one rank to ``<directory>/routes_rank<r>.jsonl``: one line per step with the
    top-k indices and probabilities (what a replay needs to reproduce the traffic of the run)."""

    def __init__(self, directory: str, rank: int, max_steps: int = 64):
        os.makedirs(directory, exist_ok=True)
        self.path = os.path.join(directory, f"routes_rank{rank}.jsonl")
        self.max_steps = max_steps
        self.steps = 0
        self._file = open(self.path, "w")

    def record(self, ids: torch.Tensor, probs: torch.Tensor) -> None:
        if self.steps >= self.max_steps:
            return
        self._file.write(json.dumps({"step": self.steps, "tokens": int(ids.shape[0]), "top_k": int(ids.shape[1]),
                                     "ids": ids.detach().cpu().reshape(-1).tolist(),
                                     "probs": probs.detach().float().cpu().reshape(-1).tolist()}) + "\n")
        self._file.flush()
        self.steps += 1

    def close(self) -> None:
        self._file.close()


class RouteReplay:
    """The routes a ``RouteRecorder`` wrote, step by step: ``next(device)`` returns (top_indices, probs) of the next
    recorded step, wrapping around at the end of the file."""

    def __init__(self, path: str):
        self.steps: List[dict] = [json.loads(line) for line in open(path) if line.strip()]
        if not self.steps:
            raise ValueError(f"{path} holds no recorded step")
        self._next = 0

    def __len__(self) -> int:
        return len(self.steps)

    def next(self, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
        s = self.steps[self._next % len(self.steps)]
        self._next += 1
        shape = (s["tokens"], s["top_k"])
        ids = torch.tensor(s["ids"], dtype=torch.int32).view(shape).to(device)
        probs = torch.tensor(s["probs"], dtype=torch.float32).view(shape).to(device)
        return ids, probs
