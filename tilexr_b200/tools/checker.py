"""Python front end of the protocol checker (csrc/checker): run modelled protocols on the CPU,
inject single-step faults, analyse event traces.

    python -m tilexr_b200.tools.checker --op ep_dispatch --ranks 4 --experts 8 --out report/
"""
from __future__ import annotations

import argparse
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
    p.add_argument("--trace", default="")
    for name in INJECTIONS:
        p.add_argument("--inject-" + name.replace("_", "-"), action="store_true")
    a = p.parse_args(argv)
    if a.trace:
        findings = check_trace(open(a.trace).read())
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
