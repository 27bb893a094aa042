"""Stage tracing and latency capture of a MoonEP buffer inside a real model run, switched on from the environment (the
reference's torch facade has the same switches: integrations/moonep_torch/tilexr_moonep/torch_api.py:669-790).

    TILEXR_MOONEP_TRACE_STAGES=1             print every stage call (rank, stage, sequence number)
    TILEXR_MOONEP_PERF_CAPTURE_DIR=DIR       time every stage call with events on the stream and, when the buffer is closed,
                                             write DIR/rank<r>_performance.json
    TILEXR_MOONEP_PERF_CAPTURE_ID=NAME       required with the directory: names the capture inside the file
    TILEXR_MOONEP_PERF_CAPTURE_OPERATORS=N   stop after N operators (default 55: one training step of five layers)
    TILEXR_MOONEP_PERF_CAPTURE_SKIP_OPERATORS=M   leave the first M stage calls out (warm-up steps)

The per-rank files fold into one document with `merge_capture_files`, which `tools/moonep/model_flow.py compare` reads
beside a harness run or the reference's published replay.
"""
from __future__ import annotations

import json
import math
import os
import pathlib
import sys
import time
import uuid
from typing import List, Optional

KERNELS = {"planning": "TileXRMoonEpPlannerKernel", "dispatch_forward": "TileXRMoonEpDispatchKernel", "dispatch_backward": "TileXRMoonEpDispatchKernel",
           "prefetch_weight": "TileXRMoonEpPrefetchKernel", "combine_forward": "TileXRMoonEpCombineKernel", "combine_backward": "TileXRMoonEpCombineKernel",
           "reduce_grad": "TileXRMoonEpReduceGradKernel"}


def _flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in ("1", "true", "yes", "on")


class _HostEvent:
    def __init__(self):
        self.t = 0.0

    def record(self):
        self.t = time.perf_counter()

    def elapsed_time(self, other: "_HostEvent") -> float:
        return (other.t - self.t) * 1e3


class StageCapture:
    """One per buffer.  `begin(stage)` / `end(token)` bracket a stage call; `write(rank)` stores what was captured."""

    def __init__(self, rank: int, environ=None, cuda: Optional[bool] = None):
        env = os.environ if environ is None else environ
        self.rank = rank
        self.trace = env.get("TILEXR_MOONEP_TRACE_STAGES", "0").strip().lower() in ("1", "true", "yes", "on")
        self.dir = env.get("TILEXR_MOONEP_PERF_CAPTURE_DIR", "")
        self.capture_id = env.get("TILEXR_MOONEP_PERF_CAPTURE_ID", "")
        self.seen = 0
        self.records: List[dict] = []
        self.skip = self.limit = 0
        if self.dir:
            try:
                self.skip = int(env.get("TILEXR_MOONEP_PERF_CAPTURE_SKIP_OPERATORS", "0"))
                self.limit = int(env.get("TILEXR_MOONEP_PERF_CAPTURE_OPERATORS", "55"))
            except ValueError as exc:
                raise ValueError("the capture's operator counts must be integers") from exc
            if self.skip < 0 or self.limit <= 0 or not self.capture_id:
                raise ValueError("a latency capture needs TILEXR_MOONEP_PERF_CAPTURE_ID, a positive operator count and a non-negative skip")
        if cuda is None:
            import torch

            cuda = torch.cuda.is_available()
        self.cuda = cuda

    @property
    def active(self) -> bool:
        return self.trace or bool(self.dir)

    def _event(self):
        if self.cuda:
            import torch

            return torch.cuda.Event(enable_timing=True)
        return _HostEvent()

    def begin(self, stage: str):
        index = self.seen
        self.seen += 1
        if self.trace:
            print(f"[TileXR MoonEP rank {self.rank}] {stage} (call {index})", file=sys.stderr, flush=True)
        if not self.dir or index < self.skip or len(self.records) >= self.limit:
            return None
        start = self._event()
        start.record()
        return index, stage, start

    def end(self, token) -> None:
        if token is None:
            return
        index, stage, start = token
        stop = self._event()
        stop.record()
        self.records.append({"source_operator": index, "stage": stage, "start": start, "stop": stop})

    def write(self) -> Optional[str]:
        """Writes rank<r>_performance.json (atomically) and returns its path; None when no capture was asked for.  The caller
        has synchronised the device.  A capture that saw fewer operators than asked for is written with `complete: false`."""
        if not self.dir:
            return None
        operators = []
        for sequence, rec in enumerate(self.records):
            us = float(rec["start"].elapsed_time(rec["stop"])) * 1000.0
            if not math.isfinite(us) or us < 0.0:
                raise RuntimeError(f"operator {sequence} of the capture has no valid latency")
            operators.append({"sequence": sequence, "source_operator": rec["source_operator"], "stage": rec["stage"], "phase": "model",
                              "layer": -1, "kernel_version": KERNELS.get(rec["stage"], rec["stage"]), "kernel_launches_per_call": 1, "latency_us": us})
        payload = {"schema_version": 1, "capture_id": self.capture_id, "rank": self.rank, "complete": len(operators) == self.limit,
                   "timing_source": "cuda events on the buffer's stream" if self.cuda else "host clock", "operators": operators}
        d = pathlib.Path(self.dir)
        d.mkdir(parents=True, exist_ok=True)
        target = d / f"rank{self.rank}_performance.json"
        temporary = d / f"{target.name}.tmp.{os.getpid()}.{uuid.uuid4().hex}"
        with open(temporary, "w", encoding="utf-8", newline="\n") as f:
            json.dump(payload, f, indent=2, sort_keys=True, allow_nan=False)
            f.write("\n")
            f.flush()
            os.fsync(f.fileno())
        os.replace(temporary, target)
        return str(target)


def merge_capture_files(directory: str) -> dict:
    """The rank files of one capture as one document (`ranks.<r>.operators[]`), the form the model-flow tools compare."""
    ranks = {}
    capture_id = None
    for p in sorted(pathlib.Path(directory).glob("rank*_performance.json")):
        d = json.loads(p.read_text())
        if capture_id is not None and d["capture_id"] != capture_id:
            raise ValueError(f"{p}: capture {d['capture_id']!r} among files of capture {capture_id!r}")
        capture_id = d["capture_id"]
        ranks[str(d["rank"])] = {"operators": d["operators"], "complete": d.get("complete", True)}
    if not ranks:
        raise ValueError(f"no rank*_performance.json under {directory}")
    return {"schema": "tilexr-moonep-capture-v1", "case": capture_id, "world_size": len(ranks), "iterations": 1,
            "operator_order": [o["stage"] for o in next(iter(ranks.values()))["operators"]], "ranks": ranks}
