"""A Mermaid flowchart of one rank's MoonEP stages drawn from a tensor dump (tensor_dump.py): every stage as a node with what it
does and what to check, every tensor that flows between stages as an edge label with its shape, dtype and first values
(reference: tools/moonep/flowcharts.py, which draws one chart per stage from stage snapshots).

    python -m tilexr_b200.tools.moonep.flowcharts DUMP_DIR --case smoke_r2 --rank 0 --out flow.mmd

The text renders in any Mermaid viewer (GitHub shows ```mermaid blocks inline).
"""
from __future__ import annotations

import argparse
import html
import pathlib
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import tensor_dump

# stage id, title, what it does, what a reader should check in its outputs
STAGES: Sequence[Tuple[str, str, str, str]] = (
    ("planning", "Planning", "gathers every rank's routes per expert, balances the load between ranks and lays out the receive rows",
     "dst encodes rank * NvS + row; cu_seqlens is non-decreasing and padded; experts_to_copy lists the borrowed experts"),
    ("dispatch", "Dispatch", "writes each route's hidden row and route weight into its destination row on the destination rank",
     "a row holds the hidden state of the route that the plan sends there; rows nobody fills are zero"),
    ("prefetch_weight", "PrefetchWeight", "pulls the projection rows of borrowed experts from their owners into the weight slots",
     "own expert rows unchanged; slot b equals the owner's rows of experts_to_copy[b]"),
    ("combine", "Combine", "sends every row back to its source token and adds a token's K rows in fp32, route order, one rounding",
     "combined_hidden is the K-row sum; route weights return bit for bit"),
    ("reduce_grad", "ReduceGrad", "adds the gradients of borrowed experts into their owners' rows and clears the slots",
     "each borrowed gradient is added once, at the owner only; slot rows are zero afterwards"),
)

# tensors of a dump (flat names) that enter and leave each stage
FLOWS: Dict[str, Tuple[Sequence[str], Sequence[str]]] = {
    "planning": (("input.topk_experts_sk",), ("plan.dst", "plan.cu_seqlens", "plan.experts_to_copy", "plan.zero_fill_ranges", "plan.remote_stats")),
    "dispatch": (("input.hidden_sh", "input.route_weights_sk", "plan.dst"), ("dispatched_hidden", "dispatched_weights")),
    "prefetch_weight": (("input.gate", "plan.experts_to_copy"), ("prefetched_gate",)),
    "combine": (("dispatched_hidden", "dispatched_weights", "plan.dst"), ("combined_hidden", "combined_weights")),
    "reduce_grad": (("input.grad_rows", "plan.experts_to_copy"), ("reduced_grad",)),
}

MAX_VALUES = 8


def tensor_label(name: str, t: Optional[torch.Tensor]) -> str:
    if t is None:
        return f"{name}: not in this dump"
    head = t.reshape(-1)[:MAX_VALUES].tolist()
    values = ", ".join(f"{v:.4g}" if isinstance(v, float) else str(v) for v in head)
    more = ", ..." if t.numel() > MAX_VALUES else ""
    return f"{name} {list(t.shape)} {str(t.dtype).replace('torch.', '')}: {values}{more}"


def _node_text(lines: Sequence[str]) -> str:
    return "<br/>".join(html.escape(line, quote=True) for line in lines)


def mermaid(tensors: Dict[str, torch.Tensor], shape: Optional[dict] = None, title: str = "") -> str:
    """The chart of one rank.  Stages whose output tensors are all absent from the dump (a case without projection
    tensors has no prefetch or reduce-grad stage) are left out."""
    out: List[str] = ["flowchart TD"]
    if title or shape:
        dims = "" if not shape else ", ".join(f"{k}={v}" for k, v in shape.items())
        out.append(f'  head["{_node_text([title, dims])}"]')
    present = [s for s in STAGES if any(name in tensors for name in FLOWS[s[0]][1])]
    previous = "head" if (title or shape) else None
    for stage, stage_title, does, check in present:
        ins, outs = FLOWS[stage]
        out.append(f'  {stage}["{_node_text([stage_title, does, "check: " + check])}"]')
        in_id, out_id = f"{stage}_in", f"{stage}_out"
        out.append(f'  {in_id}(["{_node_text([tensor_label(n, tensors.get(n)) for n in ins])}"])')
        out.append(f'  {out_id}(["{_node_text([tensor_label(n, tensors.get(n)) for n in outs])}"])')
        if previous is not None:
            out.append(f"  {previous} --> {in_id}")
        out.append(f"  {in_id} --> {stage}")
        out.append(f"  {stage} --> {out_id}")
        previous = out_id
    return "\n".join(out) + "\n"


def chart_from_dump(root: str, case: str, rank: int = 0) -> str:
    tensors = tensor_dump.load_rank(root, case, rank)
    shape = None
    for m in tensor_dump.manifests(root):
        if m["case"] == case and m["rank"] == rank:
            shape = m.get("shape")
    return mermaid(tensors, shape, f"MoonEP stages of case {case}, rank {rank}")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("root", help="a dump directory written with the launcher's --dump (its reference/ or candidate/ folder)")
    p.add_argument("--case", required=True)
    p.add_argument("--rank", type=int, default=0)
    p.add_argument("--out", default="", help="file for the chart (default: standard output)")
    args = p.parse_args(argv)
    text = chart_from_dump(args.root, args.case, args.rank)
    if args.out:
        pathlib.Path(args.out).write_text(text)
    else:
        print(text, end="")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
