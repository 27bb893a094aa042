"""Aggregates the per-launch stage traces written by a profiling session
(``<dir>/rank<R>/launch<N>/trace.json``) into one report for the whole job:

* ``trace_index.json``   every launch with its op, bytes, span and bandwidth
* ``analysis.md``        slowest rank / launch per op, per-stage totals, bottleneck hints
* ``perfetto_trace.json`` Chrome / Perfetto trace, one track per (rank, block), one slice per stage
* ``report.html``        the same tables for a browser

Same role as the reference's aggregator (tools/collectives/tilexr_collective_profile_report.py:
25-1158).  All ranks of one node share the GPU nanosecond timer, so no clock-offset
compensation is applied; ``--align`` shifts every rank so that its first event starts at zero.

    python -m tilexr_b200.tools.profile_report prof_dir [--out report_dir] [--align]
"""
from __future__ import annotations

import argparse
import html
import json
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, List


def load_traces(root: Path) -> List[dict]:
    traces = []
    for path in sorted(root.glob("rank*/launch*/trace.json")):
        try:
            t = json.loads(path.read_text())
        except (OSError, json.JSONDecodeError) as exc:
            traces.append({"path": str(path), "error": str(exc)})
            continue
        t["path"] = str(path)
        traces.append(t)
    return traces


def launch_span_us(trace: dict) -> float:
    ticks = trace.get("ticksPerUs", 1000) or 1000
    recs = [r for r in trace.get("records", []) if r["stage"] == 0 and r["count"] > 0]
    if not recs:
        return 0.0
    return (max(r["lastEnd"] for r in recs) - min(r["firstStart"] for r in recs)) / ticks


def stage_totals(trace: dict) -> Dict[str, dict]:
    ticks = trace.get("ticksPerUs", 1000) or 1000
    names = {s["id"]: s["name"] for s in trace.get("stages", [])}
    out: Dict[str, dict] = {}
    for r in trace.get("records", []):
        if r["count"] == 0:
            continue
        d = out.setdefault(names.get(r["stage"], str(r["stage"])), {"sum_us": 0.0, "max_block_us": 0.0, "max_block": -1, "bytes": 0})
        us = r["sum"] / ticks
        d["sum_us"] += us
        d["bytes"] += r.get("bytes", 0)
        if us > d["max_block_us"]:
            d["max_block_us"], d["max_block"] = us, r["core"]
    return out


def build_index(traces: List[dict]) -> List[dict]:
    index = []
    for t in traces:
        if "error" in t:
            index.append({"path": t["path"], "error": t["error"]})
            continue
        span = launch_span_us(t)
        index.append({
            "path": t["path"], "op": t["op"], "rank": t["rank"], "rankSize": t["rankSize"], "launchId": t["launchId"],
            "messageBytes": t["messageBytes"], "blocks": t["blocks"], "span_us": span,
            "algbw_GBps": (t["messageBytes"] / span / 1000.0) if span > 0 else 0.0,
            "incomplete": t.get("incomplete", False), "stages": stage_totals(t),
        })
    return index


def analyse(index: List[dict]) -> str:
    lines = ["# Collective profile", ""]
    good = [e for e in index if "error" not in e]
    bad = [e for e in index if "error" in e]
    by_op = defaultdict(list)
    for e in good:
        by_op[e["op"]].append(e)
    for op, entries in sorted(by_op.items()):
        slow = max(entries, key=lambda e: e["span_us"])
        fast = min(entries, key=lambda e: e["span_us"])
        lines += [f"## {op}", "",
                  f"- launches: {len(entries)} over {len({e['rank'] for e in entries})} ranks",
                  f"- slowest: rank {slow['rank']} launch {slow['launchId']}: {slow['span_us']:.1f} us ({slow['algbw_GBps']:.1f} GB/s)",
                  f"- fastest: rank {fast['rank']} launch {fast['launchId']}: {fast['span_us']:.1f} us"]
        totals = defaultdict(float)
        for e in entries:
            for name, d in e["stages"].items():
                if name not in ("kernel_total", "chunk_total"):
                    totals[name] += d["max_block_us"]
        if totals:
            worst = max(totals, key=totals.get)
            hint = {
                "flag_poll_wait": "blocks mostly wait for tiles from peers: look at the slowest producer rank, or add producer blocks",
                "local_input_to_ipc": "pushing tiles over NVLink dominates: transfer bound",
                "peer_ipc_to_output": "copying landed tiles to the output dominates: register the output buffer (zero-copy path)",
                "post_sync": "launches wait for peers to finish earlier launches (window reuse guard)",
            }.get(worst, "")
            lines.append(f"- dominant stage (sum of per-launch slowest blocks): `{worst}` {totals[worst]:.1f} us. {hint}")
        if any(e["incomplete"] for e in entries):
            lines.append("- some launches were written as incomplete reports")
        lines.append("")
    for e in bad:
        lines.append(f"- unreadable trace {e['path']}: {e['error']}")
    return "\n".join(lines) + "\n"


def perfetto(traces: List[dict], align: bool) -> dict:
    events = []
    for t in traces:
        if "error" in t:
            continue
        ticks = t.get("ticksPerUs", 1000) or 1000
        names = {s["id"]: s["name"] for s in t.get("stages", [])}
        recs = [r for r in t.get("records", []) if r["count"] > 0]
        base = min((r["firstStart"] for r in recs), default=0) if align else 0
        for r in recs:
            events.append({
                "name": names.get(r["stage"], str(r["stage"])), "cat": t["op"], "ph": "X",
                "ts": (r["firstStart"] - base) / ticks, "dur": max((r["lastEnd"] - r["firstStart"]) / ticks, 0.001),
                "pid": t["rank"], "tid": r["core"],
                "args": {"launch": t["launchId"], "count": r["count"], "busy_us": r["sum"] / ticks, "bytes": r.get("bytes", 0)},
            })
        events.append({"name": "process_name", "ph": "M", "pid": t["rank"], "args": {"name": f"rank {t['rank']}"}})
    return {"traceEvents": events, "displayTimeUnit": "ns"}


def render_html(index: List[dict], analysis: str) -> str:
    rows = []
    for e in index:
        if "error" in e:
            continue
        rows.append(f"<tr><td>{html.escape(e['op'])}</td><td>{e['rank']}</td><td>{e['launchId']}</td><td>{e['messageBytes']}</td>"
                    f"<td>{e['blocks']}</td><td>{e['span_us']:.1f}</td><td>{e['algbw_GBps']:.1f}</td></tr>")
    return ("<html><head><meta charset='utf-8'><title>TileXR profile</title><style>td,th{padding:2px 8px;border:1px solid #999}"
            "table{border-collapse:collapse}</style></head><body><h2>Launches</h2><table><tr><th>op</th><th>rank</th><th>launch</th>"
            "<th>bytes</th><th>blocks</th><th>span us</th><th>GB/s</th></tr>" + "".join(rows) + "</table><h2>Analysis</h2><pre>" +
            html.escape(analysis) + "</pre></body></html>\n")


def write_report(root: Path, out: Path, align: bool = False) -> dict:
    traces = load_traces(root)
    index = build_index(traces)
    analysis = analyse(index)
    out.mkdir(parents=True, exist_ok=True)
    (out / "trace_index.json").write_text(json.dumps(index, indent=1))
    (out / "analysis.md").write_text(analysis)
    (out / "perfetto_trace.json").write_text(json.dumps(perfetto(traces, align)))
    (out / "report.html").write_text(render_html(index, analysis))
    return {"launches": len(index), "out": str(out)}


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("root")
    p.add_argument("--out", default="")
    p.add_argument("--align", action="store_true")
    a = p.parse_args(argv)
    root = Path(a.root)
    res = write_report(root, Path(a.out) if a.out else root / "report", a.align)
    print(json.dumps(res))
    return 0 if res["launches"] else 1


if __name__ == "__main__":
    sys.exit(main())
