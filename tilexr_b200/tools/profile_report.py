"""Aggregates the per-launch stage traces written by a profiling session
(``<dir>/rank<R>/launch<N>/trace.json``) into one report for the whole job:

* ``trace_index.json``   every launch with its op, bytes, span and bandwidth
* ``analysis.md``        slowest rank / launch per op, per-stage totals, bottleneck hints
* ``perfetto_trace.json`` Chrome / Perfetto trace, one track per (rank, block), one slice per stage
* ``report.html``        the same tables for a browser
* ``diagnostics.json``   what is wrong with the input: unreadable or inconsistent traces, launches that some rank did not
                         record, launches missing from the sampling pattern (``--measured-iters`` / ``--sample-every``)
* ``ai_prompt.md``       the findings as a self-contained question for an assistant (``--ai-prompt``)

Same role as the reference's aggregator (tools/collectives/tilexr_collective_profile_report.py:
25-1158).  All ranks of one node share the GPU nanosecond timer; ``--align`` shifts every rank so that its first event
starts at zero.  Traces from several hosts (two-level jobs, ``--ranks-per-host L``: host = rank // L) carry each host's own
timer: the offset of a host against host 0 is estimated from the launches that both recorded (a collective ends on all its
ranks within a few microseconds, so the median difference of the hosts' end times over the launches is the timers'
difference), written to ``clock_offsets.json`` and taken out of the Perfetto trace.

    python -m tilexr_b200.tools.profile_report prof_dir [--out report_dir] [--align] [--measured-iters N --sample-every M] [--ai-prompt]
                                               [--ranks-per-host L]
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


REQUIRED_KEYS = ("op", "rank", "rankSize", "launchId", "messageBytes", "blocks", "records")


def sanitize(trace: dict) -> List[str]:
    """What is inconsistent in one trace (empty: nothing).  A trace with problems is still indexed when it has the keys."""
    problems = []
    missing = [k for k in REQUIRED_KEYS if k not in trace]
    if missing:
        return [f"missing keys: {', '.join(missing)}"]
    if not isinstance(trace.get("ticksPerUs", 1000), (int, float)) or trace.get("ticksPerUs", 1000) <= 0:
        problems.append("ticksPerUs is not a positive number")
    if not 0 <= trace["rank"] < max(1, trace["rankSize"]):
        problems.append(f"rank {trace['rank']} outside a communicator of {trace['rankSize']}")
    known = {s["id"] for s in trace.get("stages", [])}
    for r in trace["records"]:
        if r.get("count", 0) <= 0:
            continue
        if r["lastEnd"] < r["firstStart"]:
            problems.append(f"stage {r['stage']} of block {r['core']} ends before it starts")
        if r["sum"] > (r["lastEnd"] - r["firstStart"]) * max(1, r["count"]) + 1:
            problems.append(f"stage {r['stage']} of block {r['core']} was busy longer than its span allows")
        if known and r["stage"] not in known:
            problems.append(f"stage id {r['stage']} is not in the stage table")
    if not any(r.get("stage") == 0 and r.get("count", 0) > 0 for r in trace["records"]):
        problems.append("no kernel_total record: the launch's span is unknown")
    return problems


def expected_launch_ids(measured_iters: int, sample_every: int) -> List[int]:
    """Launch ids a session that samples every `sample_every`-th of `measured_iters` launches must have recorded."""
    if measured_iters <= 0 or sample_every <= 0:
        return []
    return list(range(0, measured_iters, sample_every))


def group_launches(index: List[dict]) -> List[dict]:
    """The launches that belong together across ranks (same op, message size and launch id): the span from the first
    rank's start to the last rank's end (all ranks of a node read one nanosecond timer), the skew between the ranks'
    starts and ends, the slowest rank and the ranks that did not record the launch."""
    groups: Dict[tuple, List[dict]] = defaultdict(list)
    for e in index:
        if "error" not in e:
            groups[(e["op"], e["messageBytes"], e["launchId"])].append(e)
    out = []
    for (op, nbytes, launch), entries in sorted(groups.items()):
        world = max(e["rankSize"] for e in entries)
        have = sorted(e["rank"] for e in entries)
        timed = [e for e in entries if e["span_us"] > 0]
        row = {"op": op, "messageBytes": nbytes, "launchId": launch, "ranks": have, "missing_ranks": [r for r in range(world) if r not in have]}
        if timed:
            start = min(e["start_us"] for e in timed)
            end = max(e["start_us"] + e["span_us"] for e in timed)
            slow = max(timed, key=lambda e: e["span_us"])
            row.update(group_span_us=end - start, start_skew_us=max(e["start_us"] for e in timed) - start,
                       end_skew_us=end - min(e["start_us"] + e["span_us"] for e in timed), slowest_rank=slow["rank"],
                       slowest_rank_span_us=slow["span_us"], group_algbw_GBps=nbytes / (end - start) / 1000.0 if end > start else 0.0)
        out.append(row)
    return out


def diagnose(traces: List[dict], index: List[dict], groups: List[dict], measured_iters: int = 0, sample_every: int = 0) -> List[dict]:
    found = []
    for t in traces:
        if "error" in t:
            found.append({"kind": "unreadable", "path": t["path"], "detail": t["error"]})
            continue
        for problem in sanitize(t):
            found.append({"kind": "inconsistent", "path": t["path"], "detail": problem})
    for g in groups:
        if g["missing_ranks"]:
            found.append({"kind": "missing_rank", "op": g["op"], "launchId": g["launchId"], "detail": f"ranks {g['missing_ranks']} did not record it"})
    want = expected_launch_ids(measured_iters, sample_every)
    if want:
        by_op: Dict[tuple, set] = defaultdict(set)
        for g in groups:
            by_op[(g["op"], g["messageBytes"])].add(g["launchId"])
        for (op, nbytes), have in sorted(by_op.items()):
            base = min(have)
            lost = [base + i for i in want if base + i not in have]
            if lost:
                found.append({"kind": "missing_launch", "op": op, "messageBytes": nbytes, "detail": f"launches {lost} of the sampling pattern were not recorded"})
    return found


def ai_prompt(index: List[dict], groups: List[dict], diagnostics: List[dict], analysis: str) -> str:
    """The report as one self-contained question: what was measured, the tables, what looks wrong, what to answer."""
    lines = ["# Question", "",
             "The tables below come from in-kernel stage timers of tile-flag collectives on NVLink-connected GPUs (one row per launch and rank,",
             "times in microseconds on a timer all ranks share).  Say which stage or rank limits each operation, whether the skew between ranks",
             "or the work inside the kernels explains it, and what to change first.", "", "## Launch groups", "",
             "| op | bytes | launch | group span us | start skew us | end skew us | slowest rank | GB/s |", "|---|---|---|---|---|---|---|---|"]
    for g in groups:
        if "group_span_us" in g:
            lines.append(f"| {g['op']} | {g['messageBytes']} | {g['launchId']} | {g['group_span_us']:.1f} | {g['start_skew_us']:.1f} | {g['end_skew_us']:.1f} | "
                         f"{g['slowest_rank']} | {g['group_algbw_GBps']:.1f} |")
    lines += ["", "## Findings of the aggregator", "", analysis.strip(), "", "## Problems with the input", ""]
    lines += [f"- {d['kind']}: {d['detail']}" for d in diagnostics] or ["- none"]
    return "\n".join(lines) + "\n"


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
    for d in out.values():
        # bytes over the busy time of all blocks: what the stage moves per unit of block time
        d["GBps_per_block_time"] = d["bytes"] / d["sum_us"] / 1000.0 if d["sum_us"] > 0 and d["bytes"] > 0 else 0.0
    return out


def build_index(traces: List[dict]) -> List[dict]:
    index = []
    for t in traces:
        if "error" in t:
            index.append({"path": t["path"], "error": t["error"]})
            continue
        if any(k not in t for k in REQUIRED_KEYS):
            index.append({"path": t["path"], "error": "missing keys: " + ", ".join(k for k in REQUIRED_KEYS if k not in t)})
            continue
        span = launch_span_us(t)
        ticks = t.get("ticksPerUs", 1000) or 1000
        starts = [r["firstStart"] for r in t["records"] if r.get("stage") == 0 and r.get("count", 0) > 0]
        index.append({
            "start_us": (min(starts) / ticks) if starts else 0.0,
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


def estimate_clock_offsets(traces: List[dict], ranks_per_host: int) -> Dict[int, dict]:
    """{host: {"offset_us", "launches", "spread_us"}}: how far each host's timer is ahead of host 0's, the number of launches
    the estimate rests on, and the spread (largest minus smallest difference) that says how far to trust it."""
    if ranks_per_host <= 0:
        return {}
    ends: Dict[tuple, Dict[int, float]] = defaultdict(dict)              # (op, launch) -> host -> latest end in us
    for t in traces:
        if "error" in t or any(k not in t for k in REQUIRED_KEYS):
            continue
        ticks = t.get("ticksPerUs", 1000) or 1000
        recs = [r for r in t["records"] if r.get("count", 0) > 0]
        if not recs:
            continue
        host = int(t["rank"]) // ranks_per_host
        end = max(r["lastEnd"] for r in recs) / ticks
        key = (t["op"], t["launchId"])
        ends[key][host] = max(ends[key].get(host, end), end)
    diffs: Dict[int, List[float]] = defaultdict(list)
    for per_host in ends.values():
        if 0 not in per_host:
            continue
        for host, end in per_host.items():
            diffs[host].append(end - per_host[0])
    out = {}
    for host, d in sorted(diffs.items()):
        d.sort()
        out[host] = {"offset_us": 0.0 if host == 0 else d[len(d) // 2], "launches": len(d), "spread_us": d[-1] - d[0]}
    return out


def perfetto(traces: List[dict], align: bool, ranks_per_host: int = 0, offsets: Dict[int, dict] = None) -> dict:
    events = []
    for t in traces:
        if "error" in t or any(k not in t for k in REQUIRED_KEYS):
            continue
        ticks = t.get("ticksPerUs", 1000) or 1000
        names = {s["id"]: s["name"] for s in t.get("stages", [])}
        recs = [r for r in t.get("records", []) if r["count"] > 0]
        base = min((r["firstStart"] for r in recs), default=0) if align else 0
        if not align and ranks_per_host > 0 and offsets:
            base = offsets.get(int(t["rank"]) // ranks_per_host, {}).get("offset_us", 0.0) * ticks      # this host's timer runs ahead by that much
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


def render_groups(groups: List[dict], diagnostics: List[dict]) -> str:
    lines = ["## Launches across ranks", "", "| op | bytes | launch | ranks | group span us | start skew us | end skew us | slowest rank (us) | GB/s |",
             "|---|---|---|---|---|---|---|---|---|"]
    for g in groups:
        if "group_span_us" not in g:
            continue
        lines.append(f"| {g['op']} | {g['messageBytes']} | {g['launchId']} | {len(g['ranks'])} | {g['group_span_us']:.1f} | {g['start_skew_us']:.1f} | "
                     f"{g['end_skew_us']:.1f} | {g['slowest_rank']} ({g['slowest_rank_span_us']:.1f}) | {g['group_algbw_GBps']:.1f} |")
    lines += ["", "## Problems with the input", ""]
    lines += [f"- {d['kind']}: {d.get('path', d.get('op', ''))} {d['detail']}" for d in diagnostics] or ["- none"]
    return "\n".join(lines) + "\n"


def write_report(root: Path, out: Path, align: bool = False, measured_iters: int = 0, sample_every: int = 0, emit_ai_prompt: bool = False,
                 ranks_per_host: int = 0) -> dict:
    traces = load_traces(root)
    offsets = estimate_clock_offsets(traces, ranks_per_host)
    index = build_index(traces)
    groups = group_launches(index)
    diagnostics = diagnose(traces, index, groups, measured_iters, sample_every)
    analysis = analyse(index) + "\n" + render_groups(groups, diagnostics)
    out.mkdir(parents=True, exist_ok=True)
    (out / "trace_index.json").write_text(json.dumps(index, indent=1))
    (out / "launch_groups.json").write_text(json.dumps(groups, indent=1))
    (out / "diagnostics.json").write_text(json.dumps(diagnostics, indent=1))
    (out / "analysis.md").write_text(analysis)
    (out / "perfetto_trace.json").write_text(json.dumps(perfetto(traces, align, ranks_per_host, offsets)))
    if ranks_per_host > 0:
        (out / "clock_offsets.json").write_text(json.dumps({str(h): v for h, v in offsets.items()}, indent=1))
    (out / "report.html").write_text(render_html(index, analysis))
    if emit_ai_prompt:
        (out / "ai_prompt.md").write_text(ai_prompt(index, groups, diagnostics, analysis))
    return {"launches": len(index), "groups": len(groups), "problems": len(diagnostics), "out": str(out), "hosts": len(offsets)}


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("root")
    p.add_argument("--out", default="")
    p.add_argument("--align", action="store_true")
    p.add_argument("--measured-iters", type=int, default=0, help="launches of the measured loop (with --sample-every: which launch ids must exist)")
    p.add_argument("--sample-every", type=int, default=0)
    p.add_argument("--ai-prompt", action="store_true", help="also write ai_prompt.md")
    p.add_argument("--ranks-per-host", type=int, default=0, help="traces come from several hosts of this many ranks: estimate and remove the hosts' timer offsets")
    a = p.parse_args(argv)
    root = Path(a.root)
    res = write_report(root, Path(a.out) if a.out else root / "report", a.align, a.measured_iters, a.sample_every, a.ai_prompt, a.ranks_per_host)
    print(json.dumps(res))
    return 0 if res["launches"] else 1


if __name__ == "__main__":
    sys.exit(main())
