"""Decoder of the MoonEP dispatch event trace (reference: tools/moonep/dispatch_trace.py).

The kernel writes the layout of ``csrc/include/tilexr_moonep_trace.h``: a 256-byte header, one record per (iteration,
block) and ``eventCapacity`` 48-byte events per record; times are nanoseconds of the GPU's global timer.

    python -m tilexr_b200.tools.moonep.dispatch_trace trace.bin --chrome trace.json      # open in Perfetto / chrome://tracing
    python -m tilexr_b200.tools.moonep.dispatch_trace trace.bin --summary

``decode_trace`` returns ``{"header": {...}, "blocks": [{..., "events": [...]}]}``; ``phase_summary`` folds it into one
row per phase (count, total / mean / max microseconds, bytes, rows); ``chrome_trace`` renders one track per block.
"""
from __future__ import annotations

import argparse
import json
import struct
from collections import defaultdict
from typing import Dict, List

MARKER = 0x544D5854
VERSION = 1
HEADER_BYTES = 256
HEADER_FORMAT = "<IHH8I4Q"          # marker, version, headerBytes, 8 x u32, ticksPerUs, traceBytes, blockRecordOffset, eventOffset
BLOCK_FORMAT = "<3Q6I3Q"            # beginNs, endNs, epoch, iteration, block, rank, eventCount, droppedCount, status, reserved[3]
EVENT_FORMAT = "<4QIiII"            # beginNs, endNs, bytes, sequence, phase, peer, rows, reserved
BLOCK_BYTES = struct.calcsize(BLOCK_FORMAT)
EVENT_BYTES = struct.calcsize(EVENT_FORMAT)
PHASES = ("plan-check", "zero-fill", "route-send", "flag-raise", "flag-wait", "output-copy")


def trace_layout(iterations: int, blocks: int, event_capacity: int) -> Dict[str, int]:
    if not 0 < iterations <= 100 or blocks <= 0 or not 0 < event_capacity <= 4096:
        raise ValueError("iterations in [1, 100], blocks > 0, event_capacity in [1, 4096]")
    records = iterations * blocks
    block_off = HEADER_BYTES
    event_off = block_off + records * BLOCK_BYTES
    return {"block_record_offset": block_off, "event_offset": event_off, "trace_bytes": event_off + records * event_capacity * EVENT_BYTES}


def decode_trace(raw: bytes) -> Dict[str, object]:
    if len(raw) < HEADER_BYTES:
        raise ValueError("the buffer is shorter than a trace header")
    (marker, version, header_bytes, rank, rank_size, iterations, blocks, capacity, phases, block_bytes, event_bytes, ticks, total, block_off,
     event_off) = struct.unpack_from(HEADER_FORMAT, raw, 0)
    if marker != MARKER:
        raise ValueError(f"not a MoonEP trace (marker {marker:#x}); did a traced launch run?")
    if version != VERSION or header_bytes != HEADER_BYTES or block_bytes != BLOCK_BYTES or event_bytes != EVENT_BYTES:
        raise ValueError("the trace was written by another version of the layout")
    if total > len(raw):
        raise ValueError(f"the trace says {total} bytes, the buffer has {len(raw)}")
    header = {"rank": rank, "rank_size": rank_size, "iterations": iterations, "blocks": blocks, "event_capacity": capacity,
              "phases": phases, "ticks_per_us": ticks, "trace_bytes": total}
    out: List[Dict[str, object]] = []
    for index in range(iterations * blocks):
        begin, end, epoch, iteration, block, r, count, dropped, status, *_ = struct.unpack_from(BLOCK_FORMAT, raw, block_off + index * BLOCK_BYTES)
        if begin == 0 and end == 0:
            continue                                  # this iteration has not run (yet)
        events = []
        base = event_off + index * capacity * EVENT_BYTES
        for e in range(min(count, capacity)):
            b, en, nbytes, seq, phase, peer, rows, _ = struct.unpack_from(EVENT_FORMAT, raw, base + e * EVENT_BYTES)
            events.append({"begin_ns": b, "end_ns": en, "bytes": nbytes, "sequence": seq, "phase": phase,
                           "phase_name": PHASES[phase] if phase < len(PHASES) else f"phase-{phase}", "peer": peer, "rows": rows})
        out.append({"begin_ns": begin, "end_ns": end, "epoch": epoch, "iteration": iteration, "block": block, "rank": r,
                    "event_count": count, "dropped": dropped, "status": status, "events": events})
    return {"header": header, "blocks": out}


def phase_summary(trace: Dict[str, object]) -> List[Dict[str, object]]:
    acc = defaultdict(lambda: {"count": 0, "total_us": 0.0, "max_us": 0.0, "bytes": 0, "rows": 0})
    ticks = float(trace["header"]["ticks_per_us"]) or 1000.0
    for blk in trace["blocks"]:
        for e in blk["events"]:
            a = acc[e["phase_name"]]
            us = (e["end_ns"] - e["begin_ns"]) / ticks
            a["count"] += 1
            a["total_us"] += us
            a["max_us"] = max(a["max_us"], us)
            a["bytes"] += e["bytes"]
            a["rows"] += e["rows"]
    rows = []
    for name in list(PHASES) + sorted(set(acc) - set(PHASES)):
        if name in acc:
            a = acc[name]
            rows.append({"phase": name, **a, "mean_us": a["total_us"] / max(a["count"], 1)})
    return rows


def chrome_trace(trace: Dict[str, object]) -> Dict[str, object]:
    """Trace Event Format: pid = rank, tid = block, one complete event per phase, times relative to the first block's start."""
    ticks = float(trace["header"]["ticks_per_us"]) or 1000.0
    t0 = min((b["begin_ns"] for b in trace["blocks"]), default=0)
    events = []
    for blk in trace["blocks"]:
        events.append({"name": f"dispatch iteration {blk['iteration']}", "ph": "X", "pid": blk["rank"], "tid": blk["block"],
                       "ts": (blk["begin_ns"] - t0) / ticks, "dur": max(blk["end_ns"] - blk["begin_ns"], 0) / ticks,
                       "args": {"epoch": blk["epoch"], "status": blk["status"], "dropped": blk["dropped"]}})
        for e in blk["events"]:
            events.append({"name": e["phase_name"], "ph": "X", "pid": blk["rank"], "tid": blk["block"], "ts": (e["begin_ns"] - t0) / ticks,
                           "dur": max(e["end_ns"] - e["begin_ns"], 0) / ticks, "args": {"peer": e["peer"], "bytes": e["bytes"], "rows": e["rows"]}})
    return {"traceEvents": events, "displayTimeUnit": "ns"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("trace", help="file with the raw bytes of the trace buffer")
    ap.add_argument("--chrome", default="", help="write a Chrome / Perfetto trace here")
    ap.add_argument("--summary", action="store_true")
    args = ap.parse_args(argv)
    with open(args.trace, "rb") as f:
        trace = decode_trace(f.read())
    if args.chrome:
        with open(args.chrome, "w") as f:
            json.dump(chrome_trace(trace), f)
    if args.summary or not args.chrome:
        print(f"rank {trace['header']['rank']} of {trace['header']['rank_size']}: {len(trace['blocks'])} block records")
        for r in phase_summary(trace):
            print(f"  {r['phase']:<12} n={r['count']:<6} total {r['total_us']:10.1f} us  mean {r['mean_us']:8.2f}  max {r['max_us']:8.2f}  "
                  f"{r['bytes'] / 1e6:10.2f} MB  {r['rows']} rows")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
