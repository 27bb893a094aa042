"""Full-protocol timing of the MoonEP stages (reference: tools/moonep/benchmark.py,
prefetch_weight_benchmark.py, reduce_grad_benchmark.py): CUDA events around each stage on the launching
stream, warm-up first, max over ranks."""
from __future__ import annotations

import statistics
from typing import Dict

import torch
import torch.distributed as dist

from ...integrations.moonep import ProjectionBuffers, TileXRMoonEPBuffer
from .case_factory import make_inputs
from .contracts import MoonEPCase


def _max_over_ranks(v: float, device) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def benchmark_case(comm, case: MoonEPCase, iters: int = 20, warmup: int = 5) -> Dict[str, object]:
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
    for it in range(warmup + iters):
        ev = {s: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for s in stages}
        ev["planning"][0].record()
        plan = buf.planning(inp.topk_experts_sk)
        ev["planning"][1].record()
        ev["dispatch"][0].record()
        rows, w = buf.dispatch(inp.hidden_sh, inp.route_weights_sk, plan)
        ev["dispatch"][1].record()
        if proj is not None:
            ev["prefetch_weight"][0].record()
            buf.prefetch_weight(plan, proj)
            ev["prefetch_weight"][1].record()
        ev["combine"][0].record()
        buf.combine(plan, rows, w)
        ev["combine"][1].record()
        if grads is not None:
            ev["reduce_grad"][0].record()
            buf.reduce_grad(plan, ProjectionBuffers(grads.gate, grads.up, grads.down))
            ev["reduce_grad"][1].record()
        buf.synchronize()
        if it >= warmup:
            for s in stages:
                samples[s].append(ev[s][0].elapsed_time(ev[s][1]) * 1e3)
    stage_us = {s: _max_over_ranks(statistics.median(v), dev) for s, v in samples.items()}
    esize = torch.tensor([], dtype=case.torch_dtype()).element_size()
    moved = case.routes * case.hidden * esize
    stage_gbps = {"dispatch": moved / stage_us["dispatch"] / 1e3, "combine": moved / stage_us["combine"] / 1e3}
    buf.close()
    return {"case": case.name, "ranks": case.ranks, "stage_us": stage_us, "stage_gbps": stage_gbps,
            "bytes_per_rank": moved, "iters": iters, "warmup": warmup}
