"""Decoder of the per-block profile records of the second-generation MoonEP combine (reference:
tools/moonep/combine_v2_trace.py; record layout: csrc/include/tilexr_moonep_trace.h,
``TileXRMoonEpCombineProfileRecord``, 256 bytes).

    python -m tilexr_b200.tools.moonep.combine_v2_trace records.bin --chrome combine.json --summary

``decode_profile_records`` returns one dict per block that ran; ``stage_table`` gives, per stage between two time
points, the slowest and the mean block; ``chrome_trace`` draws the stages of every block on a track of its own.
"""
from __future__ import annotations

import argparse
import json
import struct
from typing import Dict, List

MARKER = 0x50475854
RECORD_FORMAT = "<IHH6IQ8Q12QIIiIqQQ2Q"
RECORD_BYTES = struct.calcsize(RECORD_FORMAT)
TIME_POINTS = ("begin", "index_cleared", "index_built", "send_end", "reduce_end", "end")
STAGES = (("clear index", 0, 1), ("build index", 1, 2), ("send groups", 2, 3), ("reduce tokens", 3, 4), ("finish", 4, 5))
METRICS = ("rows_indexed", "groups_sent", "rows_folded", "bytes_sent", "remote_groups", "tokens_reduced", "slot_waits", "slot_wait_ns",
           "probes")
assert RECORD_BYTES == 256


def decode_profile_records(raw: bytes) -> List[Dict[str, object]]:
    out = []
    for off in range(0, len(raw) - RECORD_BYTES + 1, RECORD_BYTES):
        f = struct.unpack_from(RECORD_FORMAT, raw, off)
        marker, version, record_bytes, rank, block, block_dim, grid_dim, n_time, n_metric, epoch = f[:10]
        if marker != MARKER or record_bytes != RECORD_BYTES:
            continue                                  # a block that never ran (the workspace starts zeroed)
        times = f[10:18]
        metrics = f[18:30]
        status, step, peer, _, slot, expected, observed = f[30:37]
        rec = {"rank": rank, "block": block, "block_dim": block_dim, "grid_dim": grid_dim, "epoch": epoch, "version": version,
               "time_ns": {name: times[i] for i, name in enumerate(TIME_POINTS[:n_time])},
               "metrics": {name: metrics[i] for i, name in enumerate(METRICS[:n_metric])}}
        if status != 0:
            rec["failure"] = {"status": status, "after": TIME_POINTS[step] if step < len(TIME_POINTS) else step, "peer": peer, "slot": slot,
                              "expected": expected, "observed": observed}
        out.append(rec)
    return out


def stage_table(records: List[Dict[str, object]]) -> List[Dict[str, object]]:
    rows = []
    for name, a, b in STAGES:
        spans = []
        for r in records:
            t = r["time_ns"]
            ta, tb = t.get(TIME_POINTS[a], 0), t.get(TIME_POINTS[b], 0)
            if ta and tb and tb >= ta:
                spans.append((tb - ta) / 1e3)
        if spans:
            rows.append({"stage": name, "blocks": len(spans), "max_us": max(spans), "mean_us": sum(spans) / len(spans)})
    return rows


def totals(records: List[Dict[str, object]]) -> Dict[str, int]:
    out = {m: 0 for m in METRICS}
    for r in records:
        for m, v in r["metrics"].items():
            out[m] += v
    return out


def chrome_trace(records: List[Dict[str, object]]) -> Dict[str, object]:
    starts = [r["time_ns"]["begin"] for r in records if r["time_ns"].get("begin")]
    t0 = min(starts) if starts else 0
    events = []
    for r in records:
        t = r["time_ns"]
        for name, a, b in STAGES:
            ta, tb = t.get(TIME_POINTS[a], 0), t.get(TIME_POINTS[b], 0)
            if ta and tb and tb >= ta:
                events.append({"name": name, "ph": "X", "pid": r["rank"], "tid": r["block"], "ts": (ta - t0) / 1e3, "dur": (tb - ta) / 1e3,
                               "args": r["metrics"] if name == "send groups" else {}})
        if "failure" in r:
            events.append({"name": "wait gave up", "ph": "i", "pid": r["rank"], "tid": r["block"], "ts": (t.get("end", t0) - t0) / 1e3, "s": "t",
                           "args": r["failure"]})
    return {"traceEvents": events, "displayTimeUnit": "ns"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("records", help="file with the raw bytes of the profile region of the combine workspace")
    ap.add_argument("--chrome", default="")
    ap.add_argument("--summary", action="store_true")
    args = ap.parse_args(argv)
    with open(args.records, "rb") as f:
        recs = decode_profile_records(f.read())
    if args.chrome:
        with open(args.chrome, "w") as f:
            json.dump(chrome_trace(recs), f)
    if args.summary or not args.chrome:
        print(f"{len(recs)} block records")
        for r in stage_table(recs):
            print(f"  {r['stage']:<14} max {r['max_us']:9.2f} us  mean {r['mean_us']:9.2f} us  ({r['blocks']} blocks)")
        print("  totals:", json.dumps(totals(recs)))
        for r in recs:
            if "failure" in r:
                print(f"  block {r['block']}: {r['failure']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
