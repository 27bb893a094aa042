"""Capture the routing of a model's MoE layers once, replay the MoonEP operator sequence from the capture, and
compare two replays (reference: tools/moonep/model_flow.py and model_replay_{cache,meta,compare,
orchestrator,cli}.py).

A capture is a directory with `meta.json` (shape of every layer, in call order) and one `.pt` file per layer
and rank holding the `[S, K]` expert ids.  Replaying needs no model: the harness re-issues planning, dispatch,
combine (forward) and dispatch, combine (backward) per layer with synthetic activations of the recorded shape.
"""
from __future__ import annotations

import json
import pathlib
import statistics
from typing import Dict, List, Optional

import torch

from .contracts import MoonEPCase

META = "meta.json"


class RouteRecorder:
    """Call `record(layer_name, topk_experts_sk, hidden)` from the model's router; `save()` at the end."""

    def __init__(self, out_dir: str, rank: int, ranks: int, experts: int, prefetch_slots: int, token_padding: int = 1):
        self.dir = pathlib.Path(out_dir)
        self.rank, self.ranks = rank, ranks
        self.experts, self.prefetch_slots, self.token_padding = experts, prefetch_slots, token_padding
        self.layers: List[Dict[str, object]] = []

    def record(self, name: str, topk_experts_sk: torch.Tensor, hidden: int, dtype: str = "bfloat16") -> None:
        idx = len(self.layers)
        self.dir.mkdir(parents=True, exist_ok=True)
        torch.save(topk_experts_sk.to(torch.int32).cpu(), self.dir / f"layer{idx:04d}_rank{self.rank}.pt")
        self.layers.append({"index": idx, "name": name, "tokens": int(topk_experts_sk.shape[0]),
                            "top_k": int(topk_experts_sk.shape[1]), "hidden": int(hidden), "dtype": dtype})

    def save(self) -> None:
        if self.rank == 0:
            meta = {"schema": "tilexr-moonep-replay-v1", "ranks": self.ranks, "experts": self.experts,
                    "prefetch_slots": self.prefetch_slots, "token_padding": self.token_padding, "layers": self.layers}
            (self.dir / META).write_text(json.dumps(meta, indent=1))


def load_meta(capture_dir: str) -> Dict[str, object]:
    meta = json.loads((pathlib.Path(capture_dir) / META).read_text())
    if meta.get("schema") != "tilexr-moonep-replay-v1":
        raise ValueError("not a MoonEP replay capture")
    return meta


def layer_case(meta: Dict[str, object], layer: Dict[str, object]) -> MoonEPCase:
    return MoonEPCase(name=str(layer["name"]), ranks=int(meta["ranks"]), tokens=int(layer["tokens"]), hidden=int(layer["hidden"]),
                      top_k=int(layer["top_k"]), experts=int(meta["experts"]), prefetch_slots=int(meta["prefetch_slots"]),
                      token_padding=int(meta["token_padding"]), dtype=str(layer["dtype"]))


def replay(capture_dir: str, comm, iters: int = 3, layers: Optional[int] = None) -> Dict[str, object]:
    """Re-issues every captured layer's forward and backward communication `iters` times; returns per-layer
    median microseconds (max over nothing: this rank's own timing) of each operator."""
    from ...integrations.moonep import TileXRMoonEPBuffer

    meta = load_meta(capture_dir)
    out = []
    buffers: Dict[tuple, TileXRMoonEPBuffer] = {}
    for layer in meta["layers"][: layers or len(meta["layers"])]:
        case = layer_case(meta, layer)
        key = (case.tokens, case.hidden, case.top_k, case.dtype)
        if key not in buffers:
            buffers[key] = TileXRMoonEPBuffer(comm, case.tokens, case.hidden, case.top_k, case.experts,
                                              token_padding=case.token_padding, B=case.prefetch_slots, dtype=case.torch_dtype())
        buf = buffers[key]
        dev = buf.hidden_nvsh.device
        topk = torch.load(pathlib.Path(capture_dir) / f"layer{int(layer['index']):04d}_rank{comm.rank}.pt").to(dev)
        hidden = torch.randn(case.tokens, case.hidden, device=dev).to(case.torch_dtype())
        weights = torch.rand(case.tokens, case.top_k, device=dev)
        times: Dict[str, List[float]] = {"planning": [], "dispatch_fwd": [], "combine_fwd": [], "dispatch_bwd": [], "combine_bwd": []}
        for _ in range(iters):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
            ev[0].record()
            plan = buf.planning(topk)
            ev[1].record()
            rows, w = buf.dispatch(hidden, weights, plan)
            ev[2].record()
            y, _ = buf.combine(plan, rows)
            ev[3].record()
            grows, _ = buf.dispatch(y, None, plan)
            ev[4].record()
            buf.combine(plan, grows)
            ev[5].record()
            buf.synchronize()
            for i, k in enumerate(times):
                times[k].append(ev[i].elapsed_time(ev[i + 1]) * 1e3)
        out.append({"layer": layer["name"], "tokens": case.tokens, "us": {k: statistics.median(v) for k, v in times.items()}})
    for b in buffers.values():
        b.close()
    total = {k: sum(l["us"][k] for l in out) for k in out[0]["us"]} if out else {}
    return {"schema": "tilexr-moonep-replay-result-v1", "ranks": meta["ranks"], "layers": out, "total_us": total}


def replay_host(capture_dir: str, comm, iters: int = 3, layers: Optional[int] = None) -> Dict[str, object]:
    """The same operator sequence on a host-memory communicator (gloo ranks, no GPU): planning from the exchanged routing,
    dispatch, combine, and both again for the backward pass, through host-memory windows.  Times are wall clock; every
    layer is also verified: an unweighted combine of what the dispatch delivered returns each token times its number of
    active routes, exactly."""
    import time

    from ... import _C
    from .host_backend import HostMemoryBackend
    from .planner_reference import dst_local_from_plans, reference_plan

    meta = load_meta(capture_dir)
    gather = HostMemoryBackend(comm)._all_gather
    out = []
    for layer in meta["layers"][: layers or len(meta["layers"])]:
        case = layer_case(meta, layer)
        topk = torch.load(pathlib.Path(capture_dir) / f"layer{int(layer['index']):04d}_rank{comm.rank}.pt").to(torch.int32).reshape(case.tokens, case.top_k)
        g = torch.Generator().manual_seed(int(layer["index"]) * 131 + comm.rank)
        hidden = torch.randn(case.tokens, case.hidden, generator=g).to(case.torch_dtype()).float().contiguous()
        weights = torch.rand(case.routes, generator=g)
        times: Dict[str, List[float]] = {"planning": [], "dispatch_fwd": [], "combine_fwd": [], "dispatch_bwd": [], "combine_bwd": []}
        verified = True
        for _ in range(iters):
            t = [time.perf_counter()]
            dst = reference_plan(case, gather(topk), comm.rank)["dst"].to(torch.int32).contiguous()
            dst_local = dst_local_from_plans(case, gather(dst), comm.rank).to(torch.int32)
            t.append(time.perf_counter())
            rows, w = _C.host_moon_dispatch(comm, hidden, weights, dst, dst_local, case.top_k)
            t.append(time.perf_counter())
            y, wback = _C.host_moon_combine(comm, rows, w, dst, dst_local, case.tokens, case.top_k)
            t.append(time.perf_counter())
            grows, _ = _C.host_moon_dispatch(comm, y.contiguous(), None, dst, dst_local, case.top_k)
            t.append(time.perf_counter())
            _C.host_moon_combine(comm, grows, None, dst, dst_local, case.tokens, case.top_k)
            t.append(time.perf_counter())
            for i, k in enumerate(times):
                times[k].append((t[i + 1] - t[i]) * 1e6)
            active = (dst.view(case.tokens, case.top_k) >= 0).sum(1, keepdim=True).float()
            sent = (dst >= 0).reshape(-1)
            verified &= bool(torch.equal(y, hidden * active)) and bool(torch.equal(wback.reshape(-1)[sent], weights[sent]))
        out.append({"layer": layer["name"], "tokens": case.tokens, "verified": verified, "us": {k: statistics.median(v) for k, v in times.items()}})
    total = {k: sum(l["us"][k] for l in out) for k in out[0]["us"]} if out else {}
    return {"schema": "tilexr-moonep-replay-result-v1", "ranks": meta["ranks"], "layers": out, "total_us": total, "backend": "host-memory",
            "verified": all(l["verified"] for l in out)}


def compare_replays(a: Dict[str, object], b: Dict[str, object]) -> List[Dict[str, object]]:
    """Per operator: total microseconds of both replays and b's speed-up over a."""
    rows = []
    for k, va in a["total_us"].items():
        vb = b["total_us"].get(k)
        rows.append({"operator": k, "a_us": va, "b_us": vb, "speedup_b_over_a": None if not vb else va / vb})
    return rows
