"""Python front end of the protocol checker (csrc/checker): run modelled protocols on the CPU,
inject single-step faults, analyse event traces -- the checker's own, or what the production flag
primitives and host kernels did in a real multi-process run (`record_host_trace`).

    python -m tilexr_b200.tools.checker --op ep_dispatch --ranks 4 --experts 8 --out report/
    python -m tilexr_b200.tools.checker --trace rank0.jsonl,rank1.jsonl
    python -m tilexr_b200.tools.checker --verify-installed-traces [--trace-names host_ep_dispatch_combine] [--keep DIR]
"""
from __future__ import annotations

import argparse
import contextlib
import json
import pathlib
import sys

from .. import _C

INJECTIONS = ("read_before_copy", "stale_magic", "missing_flag", "peer_user_read", "pipe_wait", "deadlock", "skip_reuse_guard",
              "corrupt_output", "skip_entry_meeting", "shared_slice")


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


# ---- installed traces ---------------------------------------------------------------------------------------------------
# A manifest under checker_traces/ names a recipe (host kernels run between real processes over host-memory windows), the
# number of ranks, and the events the recording must contain on every rank.  Verifying it records the run, judges the trace
# and checks that coverage: a recorder that silently stopped reporting some kind of event would otherwise let every later
# run "pass" (the reference pins coverage the same way: tools/checker/installed_traces/*_trace_manifest.json with
# required_event_coverage, checked by its --verify-installed-traces).

TRACE_DIR = pathlib.Path(__file__).resolve().parent / "checker_traces"


def _recipe_all_gather(txr, comm, rank, world):
    import torch

    x = torch.arange(3 * 4096, dtype=torch.float32) + rank
    out = torch.empty(world * x.numel())
    for _ in range(3):                       # three launches: both data halves and the reuse guard
        txr._C.host_all_gather(comm, x, out, 16384)


def _recipe_all_reduce(txr, comm, rank, world):
    import torch

    txr._C.host_all_reduce(comm, torch.full((1024,), float(rank + 1)))
    txr._C.host_all_reduce(comm, torch.full((1024,), float(rank + 2)))


def _recipe_ep(txr, comm, rank, world):
    import torch

    from ..utils import oracle

    g = torch.Generator().manual_seed(77 + rank)
    bs, h, E, K = 16, 64, 2 * world, 2
    x = torch.randn(bs, h, generator=g)
    ids, w = oracle.routing_topk_ref(torch.randn(bs, E, generator=g), K, score_func=0, renormalize=True)
    expand, assist, nums, counts, total = txr._C.host_ep_dispatch(comm, x, ids, E, bs * world * K)
    txr._C.host_ep_combine(comm, expand[:total].contiguous(), assist, total, ids, w, E)


def _recipe_exchange(txr, comm, rank, world):
    import torch

    x = torch.arange(world * 5000, dtype=torch.float32) + 10000 * rank
    for root in range(world):
        txr._C.host_all_to_all(comm, x, 4096)
        txr._C.host_reduce_scatter(comm, x)
        b = torch.full((5000,), float(rank))
        txr._C.host_broadcast(comm, b, root, 4096)


def _recipe_moonep(txr, comm, rank, world):
    import dataclasses

    from .moonep.case_factory import make_inputs
    from .moonep.contracts import MoonEPCase
    from .moonep.host_backend import HostMemoryBackend

    case = MoonEPCase(name="trace", ranks=world, tokens=16, hidden=32, top_k=2, experts=4 * world, prefetch_slots=2, token_padding=2, ffn=4, seed=3)
    backend = HostMemoryBackend(comm, tile_bytes=4096)
    for launch in range(2):                  # two plans over the same windows: both data halves, the reuse guard, rows left from the plan before
        c = dataclasses.replace(case, seed=case.seed + launch)
        backend.run(c, make_inputs(c, rank))


RECIPES = {"host_all_gather": _recipe_all_gather, "host_all_reduce": _recipe_all_reduce, "host_ep_dispatch_combine": _recipe_ep,
           "host_all_to_all_reduce_scatter_broadcast": _recipe_exchange, "host_moonep_stages": _recipe_moonep}


def _trace_worker(rank: int, world: int, port: int, recipe: str, out_dir: str, errors) -> None:
    import os
    import traceback

    try:
        import torch.distributed as dist

        import tilexr_b200 as txr

        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        comm = txr.init_from_torch_distributed(host_memory=True, buffer_mb=16)
        with record_host_trace(comm, os.path.join(out_dir, f"rank{rank}.jsonl")):
            RECIPES[recipe](txr, comm, rank, world)
        comm.destroy()
        dist.destroy_process_group()
    except Exception:
        errors.put((rank, traceback.format_exc()))


def record_installed_trace(recipe: str, ranks: int, out_dir: str) -> list:
    """Runs `recipe` between `ranks` processes and returns the per-rank event files."""
    import socket

    import torch.multiprocessing as mp

    if recipe not in RECIPES:
        raise ValueError(f"unknown recipe {recipe}; known: {', '.join(sorted(RECIPES))}")
    pathlib.Path(out_dir).mkdir(parents=True, exist_ok=True)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    procs = [ctx.Process(target=_trace_worker, args=(r, ranks, port, recipe, out_dir, errors)) for r in range(ranks)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    if not errors.empty():
        rank, text = errors.get()
        raise RuntimeError(f"recording {recipe}: rank {rank} failed\n{text}")
    if any(p.exitcode != 0 for p in procs):
        raise RuntimeError(f"recording {recipe}: a rank did not finish (exit codes {[p.exitcode for p in procs]})")
    return [str(pathlib.Path(out_dir) / f"rank{r}.jsonl") for r in range(ranks)]


def event_coverage(paths) -> dict:
    """{rank: {(kind, source): count}} of recorded event files."""
    cover: dict = {}
    for p in paths:
        for line in open(p):
            if not line.strip():
                continue
            e = json.loads(line)
            per = cover.setdefault(int(e["rank"]), {})
            key = (e["kind"], e.get("source", ""))
            per[key] = per.get(key, 0) + 1
    return cover


def missing_coverage(manifest: dict, paths) -> list:
    """Entries of the manifest's required_event_coverage that some rank's recording does not meet."""
    cover = event_coverage(paths)
    missing = []
    for rank in range(int(manifest["ranks"])):
        per = cover.get(rank, {})
        for need in manifest["required_event_coverage"]:
            have = sum(n for (kind, source), n in per.items() if kind == need["kind"] and need.get("source", "") in source)
            if have < int(need.get("min_per_rank", 1)):
                missing.append({"rank": rank, "kind": need["kind"], "source": need.get("source", ""), "have": have, "need": int(need.get("min_per_rank", 1))})
    return missing


def load_manifests(names: str = "") -> list:
    wanted = [n.strip() for n in names.split(",") if n.strip()]
    found = [json.loads(p.read_text()) for p in sorted(TRACE_DIR.glob("*_trace_manifest.json"))]
    unknown = [n for n in wanted if n not in {m["name"] for m in found}]
    if unknown:
        raise ValueError(f"no installed trace named {', '.join(unknown)}")
    return [m for m in found if not wanted or m["name"] in wanted]


def verify_installed_traces(names: str = "", keep_dir: str = "") -> list:
    """Records every installed trace (or the named ones), judges it and checks its event coverage.  No GPU is involved."""
    import tempfile

    rows = []
    for m in load_manifests(names):
        with tempfile.TemporaryDirectory() as tmp:
            out_dir = str(pathlib.Path(keep_dir) / m["name"]) if keep_dir else tmp
            paths = record_installed_trace(m["recipe"], int(m["ranks"]), out_dir)
            findings = check_trace_files(paths)
            missing = missing_coverage(m, paths)
            events = sum(sum(per.values()) for per in event_coverage(paths).values())
        rows.append({"name": m["name"], "recipe": m["recipe"], "ranks": m["ranks"], "events": events, "findings": findings,
                     "missing_coverage": missing, "ok": not findings and not missing})
    return rows


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
    p.add_argument("--zero-copy", action="store_true", help="allgather: tiles go straight into the peers' registered outputs, behind an entry meeting")
    p.add_argument("--out", default="")
    p.add_argument("--trace", default="", help="event file(s) to analyse, comma separated (one per rank of a recorded run)")
    p.add_argument("--verify-installed-traces", action="store_true",
                   help="record every installed trace between real processes on the CPU, judge it and check its event coverage")
    p.add_argument("--trace-names", default="", help="with --verify-installed-traces: comma-separated manifest names (default: all)")
    p.add_argument("--keep", default="", help="with --verify-installed-traces: keep the recorded event files under this directory")
    for name in INJECTIONS:
        p.add_argument("--inject-" + name.replace("_", "-"), action="store_true")
    a = p.parse_args(argv)
    if a.verify_installed_traces:
        rows = verify_installed_traces(a.trace_names, a.keep)
        for r in rows:
            print(f"{r['name']}: {'ok' if r['ok'] else 'FAILED'} ({r['ranks']} ranks, {r['events']} events, {len(r['findings'])} findings, "
                  f"{len(r['missing_coverage'])} coverage gaps)")
            for f in r["findings"]:
                print("  finding:", *f)
            for m in r["missing_coverage"]:
                print("  coverage:", json.dumps(m))
        return 0 if rows and all(r["ok"] for r in rows) else 1
    if a.trace:
        findings = check_trace_files(a.trace.split(","))
        for f in findings:
            print(*f)
        return 1 if findings else 0
    spec = dict(op=a.op, rank_size=a.ranks, server_count=a.servers, count=a.count, tile_elems=a.tile, bs=a.bs, h=a.h, top_k=a.topk,
                moe_expert_num=a.experts, launches=a.launches, scheduler=a.scheduler, zero_copy=a.zero_copy)
    for name in INJECTIONS:
        spec["inject_" + name] = getattr(a, "inject_" + name)
    if a.out:
        spec["out_dir"] = a.out
    rep = run_case(**spec)
    print(rep["summary"], end="")
    return 0 if rep["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
