"""In-kernel stage profiler session as a context manager.

The collectives, EP dispatch and EP combine kernels record per-block begin/end times of their stages into a
device buffer while a session is active; the native library turns them into `rank<r>/launch<i>/{trace.json,
summary.csv, analysis.md}` under the output directory (reference: src/collectives/host/perf_trace_session.cpp
and perf_trace_report.cpp, public API src/include/tilexr_collectives_perf.h).
"""
from __future__ import annotations

import contextlib
import csv
import pathlib
from typing import Dict, Iterator, List


@contextlib.contextmanager
def stage_profile(output_dir: str, sample_every_n: int = 1) -> Iterator[None]:
    """Profiles every `sample_every_n`-th launch issued inside the block and writes the reports at exit."""
    import torch

    from .. import _C

    session = _C.perf_session_create(str(output_dir), sample_every_n, False, "")
    session.activate()
    try:
        yield
        torch.cuda.synchronize()
    finally:
        session.deactivate()
        session.write_report()
        session.destroy()


def read_summaries(output_dir: str) -> List[Dict[str, object]]:
    """Rows of every launch's summary.csv below `output_dir`, with `rank` and `launch` columns added."""
    rows: List[Dict[str, object]] = []
    for path in sorted(pathlib.Path(output_dir).glob("rank*/launch*/summary.csv")):
        with open(path, newline="") as f:
            for row in csv.DictReader(f):
                row["rank"] = path.parent.parent.name
                row["launch"] = path.parent.name
                rows.append(row)
    return rows


def format_summaries(output_dir: str) -> str:
    rows = read_summaries(output_dir)
    if not rows:
        return "(no profiled launches)"
    cols = [c for c in rows[0].keys() if c not in ("rank", "launch")]
    out = []
    last = None
    for r in rows:
        key = (r["rank"], r["launch"])
        if key != last:
            out.append(f"-- {r['rank']} {r['launch']}")
            out.append("   " + "  ".join(f"{c:>18}" for c in cols))
            last = key
        out.append("   " + "  ".join(f"{str(r[c]):>18}" for c in cols))
    return "\n".join(out)
