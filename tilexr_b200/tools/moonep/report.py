"""Reports of harness runs (reference: tools/moonep/report.py).

Three layers:

* sample statistics -- ``percentile``, ``metric_summary`` (P50 / P99 / mean / min / max with the samples at or
  below ``INVALID_SAMPLE_US`` counted apart: an event pair that reads 0-1 us did not bracket a kernel);
* rank aggregation -- a stage's time in an iteration is the slowest rank's, so ``aggregate_rank_samples`` takes the
  per-iteration maximum over ranks before the statistics, and keeps each rank's own P50 to show the spread;
  ``aggregate_rank_artifacts`` does the same from the ``rank<N>.jsonl`` files that ranks of several nodes leave in
  one directory;
* renderings -- markdown tables for correctness and stage performance, one CSV row per (case, stage).
"""
from __future__ import annotations

import csv
import json
import math
import pathlib
from typing import Dict, Iterable, List, Mapping, Optional, Sequence

INVALID_SAMPLE_US = 1.0


# ---- statistics ------------------------------------------------------------------------------------------------

def percentile(values: Iterable[float], quantile: float) -> float:
    """Linear interpolation between closest ranks (the definition numpy calls 'linear'); NaN for no samples."""
    v = sorted(float(x) for x in values)
    if not v:
        return math.nan
    if not 0.0 <= quantile <= 1.0:
        raise ValueError("quantile must lie in [0, 1]")
    pos = quantile * (len(v) - 1)
    lo = int(math.floor(pos))
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def metric_summary(values: Sequence[float], invalid_at_or_below: float = INVALID_SAMPLE_US) -> Dict[str, float]:
    valid = [float(x) for x in values if float(x) > invalid_at_or_below and math.isfinite(float(x))]
    out = {"samples": len(values), "invalid": len(values) - len(valid)}
    if not valid:
        out.update({"mean": math.nan, "min": math.nan, "max": math.nan, "p50": math.nan, "p99": math.nan})
        return out
    out.update({"mean": sum(valid) / len(valid), "min": min(valid), "max": max(valid), "p50": percentile(valid, 0.5),
                "p99": percentile(valid, 0.99)})
    return out


def aggregate_rank_samples(per_rank: Sequence[Sequence[float]]) -> Dict[str, object]:
    """``per_rank[r][i]`` = device time of iteration i on rank r.  Ranks that recorded fewer iterations bound the
    number of iterations compared."""
    if not per_rank:
        return {"cross_rank_max": metric_summary([]), "rank_p50": []}
    n = min(len(s) for s in per_rank)
    slowest = [max(float(s[i]) for s in per_rank) for i in range(n)]
    return {"cross_rank_max": metric_summary(slowest), "rank_p50": [metric_summary(s)["p50"] for s in per_rank],
            "iterations": n, "ranks": len(per_rank)}


def bandwidth_gbps(bytes_moved: float, micros: float) -> float:
    if not micros or not math.isfinite(micros) or micros <= 0:
        return math.nan
    return bytes_moved / micros / 1e3


# ---- files -----------------------------------------------------------------------------------------------------

def write_json(path, payload) -> None:
    pathlib.Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        json.dump(payload, f, indent=1, sort_keys=True)


def write_jsonl(path, rows: Iterable[Mapping[str, object]]) -> None:
    pathlib.Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r, sort_keys=True) + "\n")


def read_jsonl(path) -> List[Dict[str, object]]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def rank_sample_rows(case: str, rank: int, samples: Mapping[str, Sequence[float]], bytes_by_stage: Mapping[str, float]):
    """One JSONL row per (stage, iteration) as a rank writes them for a later cross-node aggregation."""
    for stage, vals in samples.items():
        for i, us in enumerate(vals):
            yield {"case": case, "rank": rank, "stage": stage, "iteration": i, "us": float(us),
                   "bytes": float(bytes_by_stage.get(stage, 0.0))}


def aggregate_rank_artifacts(directory) -> List[Dict[str, object]]:
    """Reads every ``rank*.jsonl`` under ``directory`` and returns one summary per (case, stage): statistics of the
    per-iteration slowest rank, the per-rank medians, and the bandwidth of the largest per-rank byte count at P50."""
    rows: List[Dict[str, object]] = []
    for p in sorted(pathlib.Path(directory).glob("rank*.jsonl")):
        rows += read_jsonl(p)
    table: Dict[tuple, Dict[int, Dict[int, float]]] = {}
    stage_bytes: Dict[tuple, float] = {}
    for r in rows:
        key = (r["case"], r["stage"])
        table.setdefault(key, {}).setdefault(int(r["rank"]), {})[int(r["iteration"])] = float(r["us"])
        stage_bytes[key] = max(stage_bytes.get(key, 0.0), float(r.get("bytes", 0.0)))
    out = []
    for (case, stage), by_rank in sorted(table.items()):
        per_rank = [[v for _, v in sorted(it.items())] for _, it in sorted(by_rank.items())]
        agg = aggregate_rank_samples(per_rank)
        agg.update({"case": case, "stage": stage, "bytes_per_rank": stage_bytes[(case, stage)],
                    "gbps_at_p50": bandwidth_gbps(stage_bytes[(case, stage)], agg["cross_rank_max"]["p50"])})
        out.append(agg)
    return out


# ---- renderings ------------------------------------------------------------------------------------------------

def correctness_markdown(results: Iterable[Dict[str, object]]) -> str:
    lines = ["| case | rank | verdict | failing stages |", "|---|---|---|---|"]
    for r in results:
        failing = [f"{s['stage']}: {s['detail']}" for s in r["stages"] if not s["ok"]]
        lines.append(f"| {r['case']} | {r['rank']} | {'pass' if r['ok_all_ranks'] else 'FAIL'} | {'; '.join(failing) or '-'} |")
    return "\n".join(lines)


def _fmt(v: Optional[float], digits: int = 1) -> str:
    return "" if v is None or (isinstance(v, float) and not math.isfinite(v)) else f"{v:.{digits}f}"


def benchmark_markdown(rows: List[Dict[str, object]]) -> str:
    """One line per (case, stage): P50 / P99 / max of the per-iteration slowest rank, bytes by the stage's formula and
    the bandwidth at P50.  Rows of the older form (``stage_us`` medians only) are rendered with empty statistics."""
    lines = ["| case | stage | P50 us | P99 us | max us | invalid | MB per rank | GB/s at P50 |", "|---|---|---|---|---|---|---|---|"]
    for r in rows:
        stats = r.get("stage_stats")
        for stage, us in r["stage_us"].items():
            s = stats[stage]["cross_rank_max"] if stats else {"p50": us, "p99": None, "max": None, "invalid": 0}
            nbytes = r.get("stage_bytes", {}).get(stage)
            gbps = r.get("stage_gbps", {}).get(stage)
            lines.append(f"| {r['case']} | {stage} | {_fmt(s['p50'])} | {_fmt(s['p99'])} | {_fmt(s['max'])} | {s['invalid']} | "
                         f"{_fmt(None if nbytes is None else nbytes / 1e6)} | {_fmt(gbps)} |")
    return "\n".join(lines)


def write_stage_csv(path, rows: List[Dict[str, object]]) -> None:
    pathlib.Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["case", "ranks", "stage", "p50_us", "p99_us", "mean_us", "min_us", "max_us", "samples", "invalid", "bytes_per_rank",
                    "gbps_at_p50"])
        for r in rows:
            for stage, st in r.get("stage_stats", {}).items():
                s = st["cross_rank_max"]
                w.writerow([r["case"], r.get("ranks", ""), stage, s["p50"], s["p99"], s["mean"], s["min"], s["max"], s["samples"],
                            s["invalid"], r.get("stage_bytes", {}).get(stage, ""), r.get("stage_gbps", {}).get(stage, "")])
