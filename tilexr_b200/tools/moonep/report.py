"""Text and JSON reports of harness runs (reference: tools/moonep/report.py)."""
from __future__ import annotations

import json
from typing import Dict, Iterable, List


def correctness_markdown(results: Iterable[Dict[str, object]]) -> str:
    lines = ["| case | rank | verdict | failing stages |", "|---|---|---|---|"]
    for r in results:
        failing = [f"{s['stage']}: {s['detail']}" for s in r["stages"] if not s["ok"]]
        lines.append(f"| {r['case']} | {r['rank']} | {'pass' if r['ok_all_ranks'] else 'FAIL'} | {'; '.join(failing) or '-'} |")
    return "\n".join(lines)


def benchmark_markdown(rows: List[Dict[str, object]]) -> str:
    lines = ["| case | stage | us (max over ranks) | GB/s per rank |", "|---|---|---|---|"]
    for r in rows:
        for stage, us in r["stage_us"].items():
            gbps = r.get("stage_gbps", {}).get(stage)
            lines.append(f"| {r['case']} | {stage} | {us:.1f} | {'' if gbps is None else f'{gbps:.1f}'} |")
    return "\n".join(lines)


def write_json(path: str, payload) -> None:
    with open(path, "w") as f:
        json.dump(payload, f, indent=1, sort_keys=True)
