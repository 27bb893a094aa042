"""Expert-parallel dispatch / combine on torch tensors.

``dispatch`` returns a :class:`DispatchResult`; pass it to ``combine`` together with the
expert outputs.  Semantics are those of csrc/include/tilexr_ep.h.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from .. import _C

QUANT_NONE = 0
QUANT_STATIC_INT8 = 1    # q = rint(x * scales[expert]); `scales` [num_experts, h] required
QUANT_DYNAMIC_INT8 = 2   # per row: scale = amax(x * scales[expert]) / 127 in dynamic_scales [rows], q = rint(x / scale)
QUANT_MXFP8_E5M2 = 3     # 1x32 blocks, E8M0 exponent bytes; dynamic_scales is uint8 [rows, h/32]
QUANT_MXFP8_E4M3 = 4
QUANT_FP8_1X128 = 5
TOKEN_NUMS_PREFIX = 0
TOKEN_NUMS_COUNT = 1


@dataclasses.dataclass
class DispatchResult:
    expand_x: torch.Tensor            # [max_recv_rows, h]
    dynamic_scales: Optional[torch.Tensor]
    assist: torch.Tensor              # [max_recv_rows, 4] int32 {src_rank, token, k, expert}
    expert_token_nums: torch.Tensor   # [experts_per_rank] int64
    send_counts: torch.Tensor         # [experts_per_rank * world] int32, running sum
    recv_total: torch.Tensor          # [1] int32
    topk_ids: torch.Tensor            # [bs, k] int32 (negative = inactive)
    topk_weights: torch.Tensor        # [bs, k] fp32 (only meaningful with fused routing)
    route_rows: torch.Tensor          # [bs, k] int32 row of each route at its destination rank (-1 = inactive)
    assist_ext: torch.Tensor          # [max_recv_rows, 2] int32 {group link, gate weight bits} for combine
    expand_scales: torch.Tensor       # [max_recv_rows] fp32 gate weight of each received row
    tp_recv_counts: torch.Tensor      # [tp_world_size] int32 rows that came from the ranks of each tensor-parallel lane
    bs: int
    top_k: int
    num_experts: int
    dedup: bool = False
    shared_expert_num: int = 0
    shared_expert_rank_num: int = 0
    tp_world_size: int = 1


def dispatch(comm, x: torch.Tensor, *, num_experts: int, top_k: int, expert_ids: Optional[torch.Tensor] = None,
             gate_logits: Optional[torch.Tensor] = None, selection_bias: Optional[torch.Tensor] = None,
             active_mask: Optional[torch.Tensor] = None, quant_mode: int = QUANT_NONE, score_func: int = 0,
             renormalize: bool = True, routed_scale: float = 1.0, token_nums_type: int = TOKEN_NUMS_COUNT,
             max_recv_rows: Optional[int] = None, expand_x_out: Optional[torch.Tensor] = None,
             expert_scales: Optional[torch.Tensor] = None, dedup: Optional[bool] = None,
             scales: Optional[torch.Tensor] = None, shared_expert_num: int = 0,
             shared_expert_rank_num: int = 0, tp_world_size: int = 1) -> DispatchResult:
    """``tp_world_size`` T > 1: tensor parallelism inside expert parallelism.  The ranks form ``world / T`` groups of T
    consecutive ranks that hold the same ``num_experts / (world / T)`` experts, each a slice of their weights; every
    route is written to all T ranks of its expert's group in one hop, so each of them receives all the group's rows
    (sorted by local expert, ready for a grouped GEMM) and ``tp_recv_counts[l]`` says how many came from ranks of lane l.
    ``combine`` then adds the T partial outputs of every row on the way back.  Per-route tensors of the result have T
    slots per route (``route_rows`` is [bs, top_k * T], the k of an assist tuple is ``k * T + lane``).  Needs explicit
    ``expert_ids``.

    ``dedup`` (default: on when gate weights are known at dispatch time): a token with several experts on one
    remote rank crosses NVLink once in each direction; the expert rank replicates it after arrival and sums
    its outputs, gate-weighted in fp32, before sending them back.  The weights used for those sums are the ones
    given here (fused routing or ``expert_scales``), so pass the same ones to ``combine``."""
    bs = x.shape[0]
    if dedup is None:
        dedup = gate_logits is not None or expert_scales is not None
    if scales is not None:
        dedup = False        # per-expert smoothing scales make every route's row different
    if max_recv_rows is None:
        # the same on every rank (the window layout depends on it): all tokens of all ranks with every route here
        max_recv_rows = bs * comm.world_size * min(top_k, num_experts // (comm.world_size // tp_world_size - shared_expert_rank_num))
    out = _C.ep_dispatch(comm, x, expert_ids, gate_logits, selection_bias, active_mask, top_k, num_experts, quant_mode,
                         score_func, renormalize, routed_scale, token_nums_type, max_recv_rows, expand_x_out, expert_scales,
                         bool(dedup), scales, shared_expert_num, shared_expert_rank_num, tp_world_size)
    res = DispatchResult(*out, bs=bs, top_k=top_k, num_experts=num_experts, dedup=bool(dedup),
                         shared_expert_num=shared_expert_num, shared_expert_rank_num=shared_expert_rank_num,
                         tp_world_size=tp_world_size)
    if tp_world_size > 1:
        res.topk_ids = expert_ids          # the kernel ran on the widened routes and did not echo the ids
    return res


def combine(comm, expert_out: torch.Tensor, d: DispatchResult, *, expert_scales: Optional[torch.Tensor] = None,
            active_mask: Optional[torch.Tensor] = None, shared_expert_x: Optional[torch.Tensor] = None,
            y_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _C.ep_combine(comm, expert_out, d.assist, d.send_counts, d.topk_ids, expert_scales, active_mask, shared_expert_x,
                         d.bs, d.top_k, d.num_experts, y_out, d.route_rows, d.assist_ext, d.dedup, d.shared_expert_num,
                         d.shared_expert_rank_num, d.tp_world_size)
