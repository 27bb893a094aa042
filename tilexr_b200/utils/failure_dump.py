"""Dump-on-failure: what a rank knows about a stage that gave up, written to one JSON file per rank.

A kernel whose wait ran out records the wait in the communicator's DFX block (operator, epoch, the peer and flag slot
it waited for, expected and observed flag words, the block) and raises an abort word on every peer.  ``dump`` puts that
record beside the things needed to read it later: device status, link description, the knobs of the environment, the
launch counter, and, when given, extra context of the caller (the shapes of the step, a plan's status words).

    from tilexr_b200.utils import failure_dump
    failure_dump.check(comm, "moe layer 17")        # after a synchronisation; raises after dumping

With ``TILEXR_DUMP_DIR`` set, :func:`check` and the MoonEP buffer's ``check_pending_status`` write
``<dir>/tilexr_failure_rank<r>_<n>.json``; without it nothing is written.  (Reference: the DFX dump of
src/comm/tilexr_comm.cpp `PrintDFX2Log` and the failure records of the MoonEP harness, tools/moonep/report.py.)
"""
from __future__ import annotations

import json
import os
import time
from typing import Optional

DFX_FIELDS = ("epoch", "operator", "count", "run_status", "fail_code", "fail_peer", "fail_slot", "fail_expected", "fail_observed",
              "fail_block", "launches")
RUN_STATUS = {0xBEEF: "running", 0xD0E: "finished", 0xDEAD: "failed"}
_counter = 0


def describe(comm, context: Optional[dict] = None) -> dict:
    dfx = list(comm.dfx())
    record = {name: int(dfx[i]) for i, name in enumerate(DFX_FIELDS) if i < len(dfx)}
    record["run_status_name"] = RUN_STATUS.get(record.get("run_status", 0), "unknown")
    record["fail_expected_epoch"] = record.get("fail_expected", 0) >> 32
    record["fail_observed_epoch"] = record.get("fail_observed", 0) >> 32
    out = {"time": time.time(), "rank": comm.rank, "world_size": comm.world_size, "device_status": int(comm.device_status()),
           "dfx": record, "extra_flag": int(comm.extra_flag), "knobs": {k: v for k, v in os.environ.items() if k.startswith(("TILEXR_", "LCCL_"))}}
    info = getattr(comm, "physical_info", None)
    if info is not None:
        out["physical_info"] = {k: (list(v) if isinstance(v, tuple) else v) for k, v in info().items()}
    if context:
        out["context"] = context
    return out


def dump(comm, directory: Optional[str] = None, context: Optional[dict] = None) -> Optional[str]:
    """Writes the record and returns its path; without a directory (argument or ``TILEXR_DUMP_DIR``) returns None."""
    global _counter
    directory = directory or os.environ.get("TILEXR_DUMP_DIR", "")
    if not directory:
        return None
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, f"tilexr_failure_rank{comm.rank}_{_counter}.json")
    _counter += 1
    with open(path, "w") as f:
        json.dump(describe(comm, context), f, indent=1, default=str)
    return path


def check(comm, what: str = "", context: Optional[dict] = None) -> None:
    """Call after the stream has been synchronised: raises (after dumping, if a directory is configured) when a kernel of
    this communicator gave up."""
    status = int(comm.device_status())
    if status == 0:
        return
    path = dump(comm, None, dict(context or {}, what=what))
    comm.print_dfx()
    raise RuntimeError(f"{what or 'a TileXR kernel'} failed on rank {comm.rank}: device status {status}" + (f"; record in {path}" if path else ""))
