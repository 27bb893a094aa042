"""Python front end of the protocol checker (csrc/checker): run modelled protocols on the CPU,
inject single-step faults, analyse event traces -- the checker's own, or what the production flag
primitives and host kernels did in a real multi-process run (`record_host_trace`).

    python -m tilexr_b200.tools.checker --op ep_dispatch --ranks 4 --experts 8 --out report/
    python -m tilexr_b200.tools.checker --trace rank0.jsonl,rank1.jsonl
"""
from __future__ import annotations

import argparse
import contextlib
import sys

from .. import _C

INJECTIONS = ("read_before_copy", "stale_magic", "missing_flag", "peer_user_read", "pipe_wait", "deadlock", "skip_reuse_guard",
              "corrupt_output")


def run_case(**spec) -> dict:
    """Keys: op, rank_size, server_count, count, tile_elems, bs, h, top_k, moe_expert_num, scheduler, magic, launches,
    inject_<name>, out_dir.  Returns passed / findings / summary / json / events_jsonl."""
    return _C.checker_run(spec)


def check_trace(jsonl: str) -> list:
    """Ordering analysis of an event trace (one JSON event per line)."""
    return list(_C.checker_check_trace(jsonl))


@contextlib.contextmanager
def record_host_trace(comm, path: str):
    """Record what this rank's host kernels (`_C.host_*` on a `host_memory=True` communicator) and the flag
    primitives below them do while the block runs, as checker events in `path`.  Event ids are global over the
    ranks, so `check_trace_files` of all ranks' files judges the run as a whole."""
    _C.host_trace_start(comm, path)
    try:
        yield
    finally:
        _C.host_trace_stop(comm)


def check_trace_files(paths) -> list:
    """Ordering analysis of one run recorded by several ranks (one file each)."""
    return check_trace("".join(open(p).read() for p in paths))


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--op", default="allgather")
    p.add_argument("--ranks", type=int, default=2)
    p.add_argument("--servers", type=int, default=1)
    p.add_argument("--count", type=int, default=1024)
    p.add_argument("--tile", type=int, default=256)
    p.add_argument("--bs", type=int, default=8)
    p.add_argument("--h", type=int, default=16)
    p.add_argument("--topk", type=int, default=2)
    p.add_argument("--experts", type=int, default=4)
    p.add_argument("--launches", type=int, default=1)
    p.add_argument("--scheduler", default="round_robin")
    p.add_argument("--out", default="")
    p.add_argument("--trace", default="", help="event file(s) to analyse, comma separated (one per rank of a recorded run)")
    for name in INJECTIONS:
        p.add_argument("--inject-" + name.replace("_", "-"), action="store_true")
    a = p.parse_args(argv)
    if a.trace:
        findings = check_trace_files(a.trace.split(","))
        for f in findings:
            print(*f)
        return 1 if findings else 0
    spec = dict(op=a.op, rank_size=a.ranks, server_count=a.servers, count=a.count, tile_elems=a.tile, bs=a.bs, h=a.h, top_k=a.topk,
                moe_expert_num=a.experts, launches=a.launches, scheduler=a.scheduler)
    for name in INJECTIONS:
        spec["inject_" + name] = getattr(a, "inject_" + name)
    if a.out:
        spec["out_dir"] = a.out
    rep = run_case(**spec)
    print(rep["summary"], end="")
    return 0 if rep["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
