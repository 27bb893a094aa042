"""Plain PyTorch (CPU, fp32) restatements of every operator: the correctness oracles.

Nothing here is on a hot path.  Each function states the arithmetic of one kernel in the most
direct way, so that tests can compare the CUDA result against it, and so that the semantics
are readable in one place.  The expert-parallel ordering rules follow the reference's own CPU
golden (tests/ep/demo/tilexr_ep_dispatch_demo.cpp:647-831): per destination rank, rows are
sorted local-expert-major, then by source rank, and keep source order (token, then k) within.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

FP8_MAX = 448.0
AMAX_FLOOR = 1e-4


# ---- routing ---------------------------------------------------------------------------------

def routing_topk_ref(logits: torch.Tensor, top_k: int, score_func: int = 0, renormalize: bool = True,
                     routed_scale: float = 1.0, selection_bias: Optional[torch.Tensor] = None):
    """score_func 0 = softmax, 1 = sigmoid.  Returns (ids int32 [bs,k], weights fp32 [bs,k])."""
    logits = logits.float().cpu()
    scores = torch.softmax(logits, dim=-1) if score_func == 0 else torch.sigmoid(logits)
    sel = scores if selection_bias is None else scores + selection_bias.float().cpu()
    # stable: ties go to the lower expert id
    order = torch.argsort(sel, dim=-1, descending=True, stable=True)[:, :top_k]
    w = torch.gather(scores, 1, order)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    w = w * routed_scale
    return order.to(torch.int32), w


# ---- quantisation ----------------------------------------------------------------------------

def fp8_quant_1x128_ref(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.float().cpu()
    rows, h = xf.shape
    g = xf.view(rows, h // 128, 128)
    amax = g.abs().amax(dim=-1).clamp_min(AMAX_FLOOR)
    # tensor / tensor: a true IEEE division (scalar / tensor is reciprocal-then-multiply in torch)
    inv = (torch.full_like(amax, FP8_MAX) / amax).unsqueeze(-1)
    q = (g * inv).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(rows, h)
    return q, amax / torch.full_like(amax, FP8_MAX)


def fp8_dequant_1x128_ref(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    rows, h = q.shape
    return (q.float().cpu().view(rows, h // 128, 128) * scales.float().cpu().unsqueeze(-1)).view(rows, h)


def mxfp8_quant_ref(x: torch.Tensor, e5m2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Shared exponent = floor(log2(amax)) - emax over 32 elements (emax 8 for e4m3, 15 for e5m2)."""
    xf = x.float().cpu()
    rows, h = xf.shape
    blocks = (h + 31) // 32
    pad = blocks * 32 - h
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    g = xf.view(rows, blocks, 32)
    amax = g.abs().amax(dim=-1)
    emax = 15 if e5m2 else 8
    exp = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp_min(1e-45))) - emax, torch.full_like(amax, -127.0))
    exp = exp.clamp(-127, 127)
    scaled = g * torch.exp2(-exp).unsqueeze(-1)
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    lim = 57344.0 if e5m2 else 448.0
    q = scaled.clamp(-lim, lim).to(dt).view(rows, blocks * 32)[:, :h].contiguous()
    return q, (exp + 127).to(torch.uint8)


def mxfp8_dequant_ref(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    rows, h = q.shape
    s = torch.exp2(scales.float().cpu() - 127.0)
    s = s.repeat_interleave(32, dim=1)[:, :h]
    return q.float().cpu() * s


def rmsnorm_ref(x: torch.Tensor, gamma: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """Returns (y, new_residual).  With a residual the sum is rounded to the storage dtype first."""
    if residual is not None:
        s = (x.float().cpu() + residual.float().cpu()).to(x.dtype)
        new_res = s
        xf = s.float()
    else:
        new_res = None
        xf = x.float().cpu()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * rstd * gamma.float().cpu()).to(x.dtype), new_res


# ---- expert parallel -------------------------------------------------------------------------

def ep_dispatch_ref(xs: Sequence[torch.Tensor], ids: Sequence[torch.Tensor], num_experts: int,
                    masks: Optional[Sequence[Optional[torch.Tensor]]] = None):
    """Global view of a dispatch.

    ``xs[r]`` is rank r's ``[bs, h]`` tokens, ``ids[r]`` its ``[bs, k]`` expert ids (negative =
    inactive).  ``masks[r]`` is an optional bool mask, ``[bs]`` or ``[bs, k]``.
    Returns one dict per destination rank with ``rows`` (list of (src, token, k, expert)),
    ``expand_x``, ``assist`` (int32 [n,4]), ``token_nums`` (count per local expert) and
    ``send_counts`` (running sums in (local expert, source) order).
    """
    world = len(xs)
    per = num_experts // world
    out = []
    for d in range(world):
        rows: List[Tuple[int, int, int, int]] = []
        token_nums = []
        send_counts = []
        running = 0
        for le in range(per):
            e = d * per + le
            n_e = 0
            for s in range(world):
                idt = ids[s].cpu()
                bs, k = idt.shape
                m = None if masks is None else masks[s]
                for t in range(bs):
                    for kk in range(k):
                        if int(idt[t, kk]) != e:
                            continue
                        if m is not None:
                            mm = m.cpu()
                            if (mm.dim() == 1 and not bool(mm[t])) or (mm.dim() == 2 and not bool(mm[t, kk])):
                                continue
                        rows.append((s, t, kk, e))
                        running += 1
                        n_e += 1
                send_counts.append(running)
            token_nums.append(n_e)
        if rows:
            expand = torch.stack([xs[s].cpu()[t] for (s, t, _, _) in rows])
        else:
            expand = xs[0].cpu()[:0]
        out.append({
            "rows": rows,
            "expand_x": expand,
            "assist": torch.tensor(rows, dtype=torch.int32).view(-1, 4),
            "token_nums": torch.tensor(token_nums, dtype=torch.int64),
            "send_counts": torch.tensor(send_counts, dtype=torch.int32),
        })
    return out


def ep_dispatch_assist_ref(ids: Sequence[torch.Tensor], num_experts: int) -> List[torch.Tensor]:
    """The assist tuples of :func:`ep_dispatch_ref` (no masks, no shared experts) computed with tensor ops, for
    batches where the loops above take too long: per destination rank, int32 ``[n, 4]`` rows
    ``(src, token, k, expert)`` sorted by expert, then source, then token, then k."""
    world = len(ids)
    per = num_experts // world
    rows = []
    for s, idt in enumerate(ids):
        idt = idt.cpu().long()
        bs, k = idt.shape
        t = torch.arange(bs).unsqueeze(1).expand(bs, k)
        kk = torch.arange(k).unsqueeze(0).expand(bs, k)
        keep = (idt >= 0) & (idt < num_experts)
        rows.append(torch.stack([torch.full_like(idt, s)[keep], t[keep], kk[keep], idt[keep]], dim=1))
    allrows = torch.cat(rows)
    key = ((allrows[:, 3] * world + allrows[:, 0]) * (allrows[:, 1].max() + 1) + allrows[:, 1]) * (allrows[:, 2].max() + 1) + allrows[:, 2]
    allrows = allrows[torch.argsort(key, stable=True)]
    dest = allrows[:, 3] // per
    return [allrows[dest == d].to(torch.int32) for d in range(world)]


def ep_combine_ref(dispatch, expert_outs: Sequence[torch.Tensor], ids: Sequence[torch.Tensor],
                   weights: Sequence[Optional[torch.Tensor]], out_dtype, shared: Optional[Sequence[torch.Tensor]] = None):
    """``expert_outs[d]`` are the processed rows of rank d in dispatch order.  Each token sums its
    K rows in k order in fp32 with fused multiply-adds, then rounds once."""
    world = len(ids)
    h = expert_outs[0].shape[1]
    ys = []
    slot = {}
    for d in range(world):
        rows_d = expert_outs[d].float().cpu()                  # once per rank: a per-row conversion would keep a copy per row
        for i, (s, t, k, _) in enumerate(dispatch[d]["rows"]):
            slot[(s, t, k)] = rows_d[i]
    shared_cpu = None if shared is None else [x.float().cpu() for x in shared]
    for s in range(world):
        bs, k = ids[s].shape
        y = torch.zeros(bs, h, dtype=torch.float32)
        w = None if weights[s] is None else weights[s].float().cpu()
        for t in range(bs):
            acc = torch.zeros(h, dtype=torch.float64)
            acc32 = torch.zeros(h, dtype=torch.float32)
            for kk in range(k):
                if (s, t, kk) not in slot:
                    continue
                wt = 1.0 if w is None else float(w[t, kk])
                # fma(w, row, acc) in fp32: emulate with one rounding from a float64 product-sum
                acc = acc32.double() + torch.tensor(wt, dtype=torch.float32).double() * slot[(s, t, kk)].double()
                acc32 = acc.float()
            if shared is not None:
                acc32 = acc32 + shared_cpu[s][t]
            y[t] = acc32
        ys.append(y.to(out_dtype))
    return ys


# ---- collectives -----------------------------------------------------------------------------

def all_gather_ref(xs):
    return torch.cat([x.cpu().reshape(-1) for x in xs])


def all_to_all_ref(xs):
    world = len(xs)
    chunks = [x.cpu().reshape(world, -1) for x in xs]
    return [torch.cat([chunks[s][d] for s in range(world)]) for d in range(world)]


def all_reduce_ref(xs, op: str = "sum"):
    """Rank-order accumulation in fp32 (integers natively), one final rounding."""
    first = xs[0].cpu()
    if first.dtype.is_floating_point:
        acc = first.float()
        for x in xs[1:]:
            v = x.cpu().float()
            acc = {"sum": acc + v, "prod": acc * v, "max": torch.maximum(acc, v), "min": torch.minimum(acc, v)}[op]
        return acc.to(first.dtype)
    acc = first.clone()
    for x in xs[1:]:
        v = x.cpu()
        acc = {"sum": acc + v, "prod": acc * v, "max": torch.maximum(acc, v), "min": torch.minimum(acc, v)}[op]
    return acc
