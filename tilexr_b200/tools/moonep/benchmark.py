"""Full-protocol timing of the MoonEP stages (reference: tools/moonep/benchmark.py): CUDA events around each
stage on the launching stream, warm-up first; every iteration's sample of every rank is kept, a stage's time in
an iteration is the slowest rank's, and the report gives P50 / P99 of that with the bytes of the reference's own
formula (tools/moonep/benchmark.py:433-462):

* dispatch, combine: remote routes x (2 x hidden row bytes + route weight bytes);
* prefetch_weight: remote_stats[0] x (gate + up + down row bytes);
* reduce_grad: remote_stats[1] x (gate + up + down gradient row bytes).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence

import torch
import torch.distributed as dist

from ...integrations.moonep import ProjectionBuffers, TileXRMoonEPBuffer
from . import report
from .case_factory import make_inputs
from .contracts import MoonEPCase


def gather_samples(samples: Mapping[str, Sequence[float]]) -> Dict[str, List[List[float]]]:
    """{stage: [rank][iteration]} on every rank."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return {s: [list(v)] for s, v in samples.items()}
    world = dist.get_world_size()
    everybody: List[Optional[dict]] = [None] * world
    dist.all_gather_object(everybody, {s: list(v) for s, v in samples.items()})
    return {s: [everybody[r][s] for r in range(world)] for s in samples}


def algorithm_bytes(plan, rank: int, hidden_row_bytes: int, weight_bytes: int, projection_row_bytes: int,
                    gradient_row_bytes: int) -> Dict[str, int]:
    """Bytes per stage for one rank from its plan.  A negative destination is a route that sends nothing of its own
    (-(v) - 1 decodes the raw value: the planner of the second generation marks duplicates that way)."""
    dst = plan.dst.to(torch.int64).cpu()
    raw = torch.where(dst < 0, -dst - 1, dst)
    dest_rank = raw // int(plan.NvS)
    remote = int(((dest_rank != rank) & (dest_rank >= 0) & (dest_rank < int(plan.R))).sum())
    stats = plan.remote_stats.cpu().reshape(-1).tolist()
    route_bytes = remote * (2 * hidden_row_bytes + weight_bytes)
    return {"dispatch": route_bytes, "combine": route_bytes, "prefetch_weight": int(stats[0]) * projection_row_bytes,
            "reduce_grad": int(stats[1]) * gradient_row_bytes}


def _row_bytes(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t[0].numel() * t.element_size()


def summarise(case: MoonEPCase, samples: Mapping[str, Sequence[float]], bytes_by_stage: Mapping[str, float], iters: int,
              warmup: int, device) -> Dict[str, object]:
    """Cross-rank statistics of one case; the byte count of a stage is the largest over ranks."""
    gathered = gather_samples(samples)
    stats = {s: report.aggregate_rank_samples(v) for s, v in gathered.items()}
    nbytes = {}
    for s in samples:
        b = float(bytes_by_stage.get(s, 0.0))
        if dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([b], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            b = float(t.item())
        nbytes[s] = b
    stage_us = {s: stats[s]["cross_rank_max"]["p50"] for s in samples}
    return {"case": case.name, "ranks": case.ranks, "stage_us": stage_us, "stage_stats": stats, "stage_bytes": nbytes,
            "stage_gbps": {s: report.bandwidth_gbps(nbytes[s], stage_us[s]) for s in samples if nbytes[s] > 0},
            "iters": iters, "warmup": warmup,
            "shape": {"S": case.tokens, "K": case.top_k, "E": case.experts, "H": case.hidden, "Hf": case.ffn,
                      "B": case.prefetch_slots, "dtype": case.dtype}}


def nccl_stage_baseline(plan, hidden_sh: torch.Tensor, iters: int, warmup: int) -> Dict[str, float]:
    """The same dispatch and combine as a torch + NCCL program, timed on this rank (us, median): rows gathered in destination
    order, `all_to_all_single` with the plan's split sizes, an indexed store into the [NvS, H] buffer; and back: an indexed load,
    `all_to_all_single`, a per-token `index_add_` in fp32 and a cast.  Split sizes and the receivers' slot lists are exchanged
    once outside the timed region (they are fixed for a plan), so nothing in the timed region waits for the host."""
    R, NvS, K = int(plan.R), int(plan.NvS), int(plan.K)
    dst = plan.dst.to(torch.int64)
    raw = torch.where(dst < 0, -dst - 1, dst)
    dest_rank = raw // NvS
    order = torch.argsort(dest_rank, stable=True)
    send_tokens = (order // K)
    send_slots = (raw % NvS)[order].contiguous()
    send_counts = torch.bincount(dest_rank, minlength=R)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts)
    send_splits, recv_splits = send_counts.tolist(), recv_counts.tolist()
    recv_slots = torch.empty(sum(recv_splits), dtype=torch.int64, device=dst.device)
    dist.all_to_all_single(recv_slots, send_slots, recv_splits, send_splits)
    rows_nvs = torch.zeros(NvS, hidden_sh.shape[1], dtype=hidden_sh.dtype, device=hidden_sh.device)
    arrived = torch.empty(sum(recv_splits), hidden_sh.shape[1], dtype=hidden_sh.dtype, device=hidden_sh.device)
    back = torch.empty(order.numel(), hidden_sh.shape[1], dtype=hidden_sh.dtype, device=hidden_sh.device)

    def dispatch():
        dist.all_to_all_single(arrived, hidden_sh.index_select(0, send_tokens), recv_splits, send_splits)
        rows_nvs.index_copy_(0, recv_slots, arrived)

    def combine():
        dist.all_to_all_single(back, rows_nvs.index_select(0, recv_slots), send_splits, recv_splits)
        acc = torch.zeros(hidden_sh.shape[0], hidden_sh.shape[1], dtype=torch.float32, device=hidden_sh.device)
        acc.index_add_(0, send_tokens, back.float())
        return acc.to(hidden_sh.dtype)

    out = {}
    for name, fn in (("dispatch", dispatch), ("combine", combine)):
        times = []
        for it in range(warmup + iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(e0.elapsed_time(e1) * 1e3)
        times.sort()
        t = torch.tensor([times[len(times) // 2]], dtype=torch.float64, device=hidden_sh.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = float(t.item())
    return out


def benchmark_case(comm, case: MoonEPCase, iters: int = 20, warmup: int = 5, sample_dir: str = "", trace: bool = False, nccl_baseline: bool = False,
                   stage_barrier: bool = False) -> Dict[str, object]:
    """``trace``: one more dispatch after the timed loop records the kernel's event trace; the result then carries this
    rank's per-phase summary (``dispatch_phases``: count, mean and longest duration, bytes) beside the stage times."""
    # ``stage_barrier``: a device synchronisation and a host barrier of the ranks in front of every stage (the reference's
    # mindspeed_stage_barrier): a stage's time is then the kernel's own and not the skew its peers arrived with.
    def align():
        if stage_barrier:
            torch.cuda.synchronize()
            comm.barrier()

    rank = comm.rank
    buf = TileXRMoonEPBuffer(comm, case.tokens, case.hidden, case.top_k, case.experts, token_padding=case.token_padding,
                             B=case.prefetch_slots, dtype=case.torch_dtype())
    dev = buf.hidden_nvsh.device
    inp = make_inputs(case, rank, str(dev))
    L = case.local_experts
    proj = grads = None
    if case.ffn > 0:
        proj = buf.register_projection_buffers(inp.gate.shape[1:], inp.gate.shape[1:], inp.gate.shape[1:], dtype=inp.gate.dtype)
        for t, src in ((proj.gate, inp.gate), (proj.up, inp.up), (proj.down, inp.down)):
            t.zero_()
            t[:L].copy_(src)
        grads = buf.prepare_reduce_grad(proj)
        torch.cuda.synchronize()
        comm.barrier()
    stages = ["planning", "dispatch", "combine"] + (["prefetch_weight", "reduce_grad"] if proj is not None else [])
    samples = {s: [] for s in stages}
    plan = None
    for it in range(warmup + iters):
        ev = {s: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for s in stages}
        align()
        ev["planning"][0].record()
        plan = buf.planning(inp.topk_experts_sk)
        ev["planning"][1].record()
        align()
        ev["dispatch"][0].record()
        rows, w = buf.dispatch(inp.hidden_sh, inp.route_weights_sk, plan)
        ev["dispatch"][1].record()
        if proj is not None:
            align()
            ev["prefetch_weight"][0].record()
            buf.prefetch_weight(plan, proj)
            ev["prefetch_weight"][1].record()
        align()
        ev["combine"][0].record()
        buf.combine(plan, rows, w)
        ev["combine"][1].record()
        if grads is not None:
            align()
            ev["reduce_grad"][0].record()
            buf.reduce_grad(plan, ProjectionBuffers(grads.gate, grads.up, grads.down))
            ev["reduce_grad"][1].record()
        buf.synchronize()
        if it >= warmup:
            for s in stages:
                samples[s].append(ev[s][0].elapsed_time(ev[s][1]) * 1e3)
    esize = torch.tensor([], dtype=case.torch_dtype()).element_size()
    proj_row = 0 if proj is None else _row_bytes(proj.gate) + _row_bytes(proj.up) + _row_bytes(proj.down)
    grad_row = 0 if grads is None else _row_bytes(grads.gate) + _row_bytes(grads.up) + _row_bytes(grads.down)
    nbytes = algorithm_bytes(plan, rank, case.hidden * esize, 4, proj_row, grad_row)
    out = summarise(case, samples, nbytes, iters, warmup, dev)
    if nccl_baseline and dist.is_initialized() and dist.get_world_size() > 1:
        out["nccl_baseline_us"] = nccl_stage_baseline(plan, inp.hidden_sh, max(3, iters // 2), 2)
    if trace:
        from .dispatch_trace import phase_summary

        recorder = buf.dispatch_trace(iterations=1, event_capacity=64, blocks=256)
        buf.dispatch(inp.hidden_sh, inp.route_weights_sk, plan, trace=recorder)
        buf.synchronize()
        out["dispatch_phases"] = phase_summary(recorder.decode())
    if sample_dir:
        report.write_jsonl(f"{sample_dir}/rank{rank}.jsonl", report.rank_sample_rows(case.name, rank, samples, nbytes))
    buf.close()
    return out
