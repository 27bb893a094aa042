"""The MoonEP operator sequence of a training step with activation recomputation, timed operator by operator
(reference: tools/moonep/model_flow.py; its published result is
tools/moonep/model_replay_meta/model-replay-s4096-k8-h7168-ep8-r8/performance.json).

A step over L MoE layers issues, per rank:

    initial forward      layer 0 .. L-1:   planning, dispatch (forward), prefetch-weight, combine (forward)
    backward, recompute  layer L-1 .. 0:   the same four again (the forward is recomputed), then
                                           dispatch (backward), combine (backward), reduce-grad

so 2L forward calls and L backward calls: with L = 5 the 55 operators of the reference's replay (ten of each forward
stage, five of each backward stage).  Every operator is
bracketed by events on the stream, the document that comes out has the reference's layout (`ranks.<r>.operators[]` with
`sequence`, `phase`, `layer`, `stage`, `latency_us`, `algorithm_bytes`), and `compare_with_published` sets the medians
beside the reference's Ascend950 EP8 numbers.

The routing of a layer is either synthetic (the case's skewed distribution) or rebuilt from per-expert route counts that a
model run recorded (`routes_from_expert_counts`: a histogram is all that has to be kept of a layer's routing to replay its
communication).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m tilexr_b200.tools.moonep.launcher \\
        --mode model-flow --cases perf --layers 5 --iters 5 --json performance.json
    python -m tilexr_b200.tools.moonep.model_flow compare before.json after.json     (also reads the reference's performance.json)
"""
from __future__ import annotations

import heapq
import json
import statistics
import time
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from .contracts import MoonEPCase

FORWARD_STAGES = ("planning", "dispatch_forward", "prefetch_weight", "combine_forward")
BACKWARD_STAGES = ("dispatch_backward", "combine_backward", "reduce_grad")
SCHEMA = "tilexr-moonep-model-flow-v1"

# Medians of the reference's published EP8 replay (S 4096, K 8, H 7168, bf16, 8 x Ascend950), microseconds.
PUBLISHED_EP8_US = {"planning": 16750.0, "dispatch_forward": 2646.0, "dispatch_backward": 2232.0, "prefetch_weight": 573.0,
                    "combine_forward": 3021.0, "combine_backward": 4495.0, "reduce_grad": 2760.0}


def operator_order(layers: int = 5, recompute: bool = True) -> List[dict]:
    """The operators of one step in issue order; `stage_occurrence` counts the earlier operators of the same stage."""
    out: List[dict] = []
    seen: Dict[str, int] = {}

    def add(phase: str, layer: int, stage: str) -> None:
        out.append({"sequence": len(out), "phase": phase, "layer": layer, "stage": stage, "stage_occurrence": seen.get(stage, 0)})
        seen[stage] = seen.get(stage, 0) + 1

    for layer in range(layers):
        for stage in FORWARD_STAGES:
            add("initial_forward", layer, stage)
    for layer in reversed(range(layers)):
        if recompute:
            for stage in FORWARD_STAGES:
                add("recompute_backward", layer, stage)
        for stage in BACKWARD_STAGES:
            add("recompute_backward" if recompute else "backward", layer, stage)
    return out


def routes_from_expert_counts(counts: Iterable[int], tokens: int, top_k: int) -> torch.Tensor:
    """[tokens, top_k] int32 expert ids whose histogram is `counts` and whose rows hold distinct experts: every token takes
    the `top_k` experts with the most routes left (ties to the lower id), which keeps the remaining counts feasible."""
    counts = [int(c) for c in counts]
    if tokens <= 0 or top_k <= 0 or len(counts) < top_k:
        raise ValueError("tokens and top_k must be positive and there must be at least top_k experts")
    if any(c < 0 or c > tokens for c in counts):
        raise ValueError("an expert can be routed to at most once per token: every count must be in [0, tokens]")
    if sum(counts) != tokens * top_k:
        raise ValueError("the counts must sum to tokens * top_k")
    heap = [(-c, e) for e, c in enumerate(counts) if c > 0]
    heapq.heapify(heap)
    rows: List[int] = []
    for _ in range(tokens):
        if len(heap) < top_k:
            raise ValueError("the histogram cannot give every token top_k distinct experts")
        picked = [heapq.heappop(heap) for _ in range(top_k)]
        rows.extend(e for _, e in picked)
        for neg, e in picked:
            if neg + 1 < 0:
                heapq.heappush(heap, (neg + 1, e))
    return torch.tensor(rows, dtype=torch.int32).view(tokens, top_k)


def operator_bytes(stage: str, case: MoonEPCase, remote_stats: Optional[Sequence[int]], projection_row_bytes: int) -> Optional[int]:
    """Bytes an operator has to move by its definition (the reference's accounting): a row per route for dispatch and
    combine, plus the fp32 route weight where it travels; a projection row set per borrowed expert for the weight stages."""
    elem = {"bfloat16": 2, "float16": 2, "float32": 4}[case.dtype]
    hidden = case.routes * case.hidden * elem
    weights = case.routes * 4
    if stage == "planning":
        return None
    if stage in ("dispatch_forward", "combine_backward"):
        return hidden + weights
    if stage in ("dispatch_backward", "combine_forward"):
        return hidden
    if remote_stats is None:
        return None
    if stage == "prefetch_weight":
        return int(remote_stats[0]) * projection_row_bytes
    if stage == "reduce_grad":
        return int(remote_stats[1]) * projection_row_bytes
    raise ValueError(f"unknown stage {stage}")


class _HostEvent:
    def __init__(self):
        self.t = 0.0

    def record(self):
        self.t = time.perf_counter()

    def elapsed_time(self, other: "_HostEvent") -> float:
        return (other.t - self.t) * 1e3


def _event(cuda: bool):
    return torch.cuda.Event(enable_timing=True) if cuda else _HostEvent()


class ModelFlow:
    """Issues the operator sequence on `buffer` (a `TileXRMoonEPBuffer`, or anything with its stage methods).

    `topk_per_layer[l]` is the `[S, K]` routing of layer l, `hidden` / `weights` the activations (one set, reused by every
    layer: the communication does not depend on their values), `projections` / `grads` the weight and gradient buffers of
    the prefetch and reduce-grad stages (None: those two stages are skipped, as for cases without an FFN width).
    `expert` maps the dispatched rows to the rows that combine returns (default: the rows themselves)."""

    def __init__(self, buffer, case: MoonEPCase, topk_per_layer: Sequence[torch.Tensor], hidden: torch.Tensor, weights: torch.Tensor,
                 projections=None, grads=None, expert: Optional[Callable] = None, recompute: bool = True, cuda: Optional[bool] = None,
                 between_operators: Optional[Callable[[], None]] = None):
        self.buffer, self.case = buffer, case
        self.topk, self.hidden, self.weights = list(topk_per_layer), hidden, weights
        self.projections, self.grads = projections, grads
        self.expert = expert or (lambda rows, plan: rows)
        self.order = operator_order(len(self.topk), recompute)
        self.cuda = hidden.is_cuda if cuda is None else cuda
        self.between = between_operators

    def run_iteration(self) -> List[dict]:
        """One step; returns the operator records with `latency_us` (and `skipped` for the stages that did not run)."""
        plans: Dict[int, object] = {}
        rows: Dict[int, torch.Tensor] = {}
        marks = []
        buf = self.buffer
        for op in self.order:
            layer, stage = op["layer"], op["stage"]
            if self.between is not None:
                self.between()
            start, stop = _event(self.cuda), _event(self.cuda)
            skipped = False
            start.record()
            if stage == "planning":
                plans[layer] = buf.planning(self.topk[layer])
            elif stage == "dispatch_forward":
                rows[layer], _ = buf.dispatch(self.hidden, self.weights, plans[layer])
            elif stage == "prefetch_weight":
                if self.projections is None:
                    skipped = True
                else:
                    buf.prefetch_weight(plans[layer], self.projections)
            elif stage == "combine_forward":
                buf.combine(plans[layer], self.expert(rows[layer], plans[layer]))
            elif stage == "dispatch_backward":
                rows[layer], _ = buf.dispatch(self.hidden, None, plans[layer])
            elif stage == "combine_backward":
                buf.combine(plans[layer], self.expert(rows[layer], plans[layer]), getattr(buf, "weights_nvs", None))
            elif stage == "reduce_grad":
                if self.grads is None:
                    skipped = True
                else:
                    buf.reduce_grad(plans[layer], self.grads)
            stop.record()
            marks.append((op, start, stop, skipped, plans.get(layer)))
        if self.cuda:
            torch.cuda.synchronize()
        out = []
        for op, start, stop, skipped, plan in marks:
            rec = dict(op)
            rec["skipped"] = skipped
            rec["latency_us"] = None if skipped else start.elapsed_time(stop) * 1e3
            rec["remote_stats"] = None
            stats = getattr(plan, "remote_stats", None)
            if stats is not None and op["stage"] in ("prefetch_weight", "reduce_grad") and not skipped:
                rec["remote_stats"] = [int(v) for v in stats.cpu().tolist()]
            out.append(rec)
        return out


def performance_document(case: MoonEPCase, rank: int, iterations: List[List[dict]], projection_row_bytes: int = 0, backend: str = "tilexr") -> dict:
    """Folds the iterations of one rank: per operator the median and the largest latency, bytes and bandwidth."""
    operators = []
    for i, op in enumerate(iterations[0]):
        samples = [it[i]["latency_us"] for it in iterations if it[i]["latency_us"] is not None]
        rec = {k: op[k] for k in ("sequence", "phase", "layer", "stage", "stage_occurrence")}
        rec["backend"] = backend
        if not samples:
            rec.update(latency_us=None, latency_max_us=None, algorithm_bytes=None, algorithm_bandwidth_GBps=None, skipped=True)
        else:
            med = statistics.median(samples)
            nbytes = operator_bytes(op["stage"], case, op.get("remote_stats"), projection_row_bytes)
            rec.update(latency_us=med, latency_max_us=max(samples), algorithm_bytes=nbytes,
                       algorithm_bandwidth_GBps=None if not nbytes or med <= 0 else nbytes / med / 1e3, skipped=False)
        operators.append(rec)
    return {"schema": SCHEMA, "case": case.name, "world_size": case.ranks, "iterations": len(iterations), "backend": backend,
            "shape": {"tokens": case.tokens, "hidden": case.hidden, "top_k": case.top_k, "experts": case.experts,
                      "prefetch_slots": case.prefetch_slots, "token_padding": case.token_padding, "dtype": case.dtype, "ffn": case.ffn},
            "timing_source": "wall clock around every (blocking) operator" if "host" in backend else "events on the issuing stream around every operator", "operator_order": [o["stage"] for o in iterations[0]],
            "ranks": {str(rank): {"operators": operators}}}


def merge_rank_documents(docs: Sequence[dict]) -> dict:
    """One document for all ranks (every rank contributes its `ranks` entry)."""
    merged = dict(docs[0])
    merged["ranks"] = {}
    for d in docs:
        merged["ranks"].update(d["ranks"])
    return merged


def stage_medians(doc: dict) -> Dict[str, dict]:
    """Per stage: the median over operators of the slowest rank's latency (an operator ends when its last rank ends)."""
    per_op: Dict[int, List[float]] = {}
    stage_of: Dict[int, str] = {}
    nbytes: Dict[int, Optional[int]] = {}
    for entry in doc["ranks"].values():
        for op in entry["operators"]:
            if op["latency_us"] is None:
                continue
            per_op.setdefault(op["sequence"], []).append(op["latency_us"])
            stage_of[op["sequence"]] = op["stage"]
            nbytes[op["sequence"]] = op.get("algorithm_bytes")
    out: Dict[str, dict] = {}
    for stage in FORWARD_STAGES + BACKWARD_STAGES:
        seqs = [s for s, st in stage_of.items() if st == stage]
        if not seqs:
            continue
        slowest = [max(per_op[s]) for s in seqs]
        med = statistics.median(slowest)
        sizes = [nbytes[s] for s in seqs if nbytes[s]]
        out[stage] = {"operators": len(seqs), "median_us": med, "max_us": max(slowest),
                      "median_GBps": None if not sizes or med <= 0 else statistics.median(sizes) / med / 1e3}
    return out


def compare_with_published(doc: dict, published: Optional[Dict[str, float]] = None) -> List[dict]:
    """Rows `{stage, this_us, published_us, speedup}` against the reference's published medians (other hardware: context,
    not a like-for-like comparison)."""
    published = PUBLISHED_EP8_US if published is None else published
    rows = []
    for stage, s in stage_medians(doc).items():
        ref = published.get(stage)
        rows.append({"stage": stage, "this_us": s["median_us"], "published_us": ref, "speedup": None if not ref else ref / s["median_us"]})
    return rows


def run_case(comm, case: MoonEPCase, layers: int = 5, iters: int = 5, warmup: int = 1, recompute: bool = True,
             route_counts: Optional[Sequence[Sequence[int]]] = None) -> dict:
    """The flow of `case` on this rank of `comm`; `route_counts[l]` (per-expert route counts of this rank in layer l)
    replaces the synthetic routing.  Returns this rank's performance document."""
    from ...integrations.moonep import ProjectionBuffers, TileXRMoonEPBuffer
    from .case_factory import make_inputs, routing

    buf = TileXRMoonEPBuffer(comm, case.tokens, case.hidden, case.top_k, case.experts, token_padding=case.token_padding,
                             B=case.prefetch_slots, dtype=case.torch_dtype())
    dev = buf.hidden_nvsh.device
    inputs = make_inputs(case, comm.rank, dev)
    topk = []
    for layer in range(layers):
        if route_counts is not None:
            topk.append(routes_from_expert_counts(route_counts[layer], case.tokens, case.top_k).to(dev))
        else:
            topk.append(routing(dataclass_replace_seed(case, case.seed + layer), comm.rank).to(dev))
    projections = grads = None
    row_bytes = 0
    if case.ffn > 0:
        L = case.local_experts
        shape = inputs.gate.shape[1:]
        projections = buf.register_projection_buffers(shape, shape, shape, dtype=inputs.gate.dtype)
        for t, src in ((projections.gate, inputs.gate), (projections.up, inputs.up), (projections.down, inputs.down)):
            t.zero_()
            t[:L].copy_(src)
        g = buf.prepare_reduce_grad(projections)
        g.gate.copy_(inputs.grad_rows)
        grads = ProjectionBuffers(g.gate, None, None)
        row_bytes = 3 * inputs.gate[0].numel() * inputs.gate.element_size()
        torch.cuda.synchronize()
        comm.barrier()
    flow = ModelFlow(buf, case, topk, inputs.hidden_sh, inputs.route_weights_sk, projections, grads, recompute=recompute)
    for _ in range(warmup):
        flow.run_iteration()
    runs = [flow.run_iteration() for _ in range(iters)]
    buf.synchronize()
    buf.close()
    return performance_document(case, comm.rank, runs, row_bytes)


def run_case_host(comm, case: MoonEPCase, layers: int = 5, iters: int = 2, warmup: int = 0, recompute: bool = True) -> dict:
    """The same operator sequence on a host-memory communicator (gloo ranks, no GPU): every operator through host-memory
    windows, timed by wall clock.  The document has the layout of the device run with `backend` = "tilexr-host-memory"."""
    import types

    from .case_factory import make_inputs, routing
    from .host_backend import HostStageBuffer

    buf = HostStageBuffer(comm, case)
    inputs = make_inputs(case, comm.rank)
    topk = [routing(dataclass_replace_seed(case, case.seed + layer), comm.rank) for layer in range(layers)]
    projections = grads = None
    row_bytes = 0
    if case.ffn > 0:
        L, B = case.local_experts, case.prefetch_slots

        def slots(src):
            t = torch.zeros((L + B,) + tuple(src.shape[1:]), dtype=src.dtype)
            t[:L] = src
            return t

        projections = types.SimpleNamespace(gate=slots(inputs.gate), up=slots(inputs.up), down=slots(inputs.down))
        grads = types.SimpleNamespace(gate=inputs.grad_rows.clone().float(), up=None, down=None)
        row_bytes = 3 * inputs.gate[0].numel() * inputs.gate.element_size()
    flow = ModelFlow(buf, case, topk, inputs.hidden_sh, inputs.route_weights_sk, projections, grads, recompute=recompute, cuda=False)
    for _ in range(warmup):
        flow.run_iteration()
    runs = [flow.run_iteration() for _ in range(iters)]
    return performance_document(case, comm.rank, runs, row_bytes, backend="tilexr-host-memory")


def dataclass_replace_seed(case: MoonEPCase, seed: int) -> MoonEPCase:
    import dataclasses

    return dataclasses.replace(case, seed=seed)


def markdown(doc: dict) -> str:
    lines = [f"### {doc['case']}: {len(doc['operator_order'])} operators per step, {doc['iterations']} iterations, {doc['world_size']} ranks", "",
             "| stage | operators | median us (slowest rank) | longest us | GB/s at the median | published Ascend950 EP8 us | ratio |", "|---|---|---|---|---|---|---|"]
    cmp_rows = {r["stage"]: r for r in compare_with_published(doc)}
    on_device = "host" not in str(doc.get("backend", ""))                 # wall-clock times of the host plumbing compare with nothing published
    for stage, s in stage_medians(doc).items():
        c = cmp_rows[stage] if on_device else {"speedup": None, "published_us": None}
        gb = "-" if s["median_GBps"] is None else f"{s['median_GBps']:.1f}"
        ratio = "-" if c["speedup"] is None else f"{c['speedup']:.1f}x"
        lines.append(f"| {stage} | {s['operators']} | {s['median_us']:.1f} | {s['max_us']:.1f} | {gb} | {c['published_us'] or '-'} | {ratio} |")
    return "\n".join(lines)


def compare_documents(a: dict, b: dict) -> List[dict]:
    """Stage by stage: the slowest rank's median of two runs and b's speed-up over a (reference:
    tools/moonep/model_replay_compare.py).  The documents may come from different builds, machines or backends; stages
    that only one of them timed are listed with the other side empty."""
    ma, mb = stage_medians(a), stage_medians(b)
    rows = []
    for stage in FORWARD_STAGES + BACKWARD_STAGES:
        sa, sb = ma.get(stage), mb.get(stage)
        if sa is None and sb is None:
            continue
        rows.append({"stage": stage, "a_us": None if sa is None else sa["median_us"], "b_us": None if sb is None else sb["median_us"],
                     "a_operators": 0 if sa is None else sa["operators"], "b_operators": 0 if sb is None else sb["operators"],
                     "speedup_b_over_a": None if not sa or not sb or sb["median_us"] <= 0 else sa["median_us"] / sb["median_us"]})
    total_a = sum(r["a_us"] * r["a_operators"] for r in rows if r["a_us"] is not None and r["b_us"] is not None)
    total_b = sum(r["b_us"] * r["b_operators"] for r in rows if r["a_us"] is not None and r["b_us"] is not None)
    rows.append({"stage": "step (stages both runs timed, median x operators)", "a_us": total_a, "b_us": total_b, "a_operators": None, "b_operators": None,
                 "speedup_b_over_a": None if total_b <= 0 else total_a / total_b})
    return rows


def load_document(path: str) -> dict:
    """A document written by the launcher's model-flow mode (`--json` holds a list with one document per case; the first is
    taken), or one in the reference's layout (`ranks.<r>.operators[]` with `stage` and `latency_us`)."""
    with open(path) as f:
        doc = json.load(f)
    if isinstance(doc, list):
        doc = doc[0]
    if "ranks" not in doc:
        raise ValueError(f"{path}: no per-rank operator list")
    for entry in doc["ranks"].values():
        for op in entry["operators"]:
            op.setdefault("algorithm_bytes", None)
            op.setdefault("sequence", entry["operators"].index(op))
    return doc


def main(argv=None) -> int:
    import argparse

    p = argparse.ArgumentParser(description="Compare two model-flow documents stage by stage, or show one against the published medians.")
    sub = p.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    s1 = sub.add_parser("show")
    s1.add_argument("doc")
    args = p.parse_args(argv)
    if args.cmd == "show":
        doc = load_document(args.doc)
        doc.setdefault("case", args.doc)
        doc.setdefault("operator_order", [o["stage"] for o in next(iter(doc["ranks"].values()))["operators"]])
        doc.setdefault("iterations", 1)
        doc.setdefault("world_size", len(doc["ranks"]))
        print(markdown(doc))
        return 0
    rows = compare_documents(load_document(args.a), load_document(args.b))
    print("| stage | a us | b us | b over a |\n|---|---|---|---|")
    for r in rows:
        fmt = lambda v: "-" if v is None else f"{v:.1f}"
        sp = "-" if r["speedup_b_over_a"] is None else f"{r['speedup_b_over_a']:.2f}x"
        print(f"| {r['stage']} | {fmt(r['a_us'])} | {fmt(r['b_us'])} | {sp} |")
    return 0


def write_json(path: str, doc: dict) -> None:
    with open(path, "w") as f:
        json.dump(doc, f, indent=1)


if __name__ == "__main__":
    raise SystemExit(main())
