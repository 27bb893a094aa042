"""Dispatch on its own, in a tight loop: what a training run does thousands of times per minute with the same buffers
(reference: tools/moonep/dispatch_hot_loop.py).

Three things are looked at, for hidden rows alone (`hidden`), or rows with their route weights (`pair`):

* **repeated exact**: the same plan dispatched N times into the same receive tensor; after every launch the received rows
  must equal, bit for bit, what the plan says they are.  Rows are cleared by nothing but the kernel itself, so a launch
  that relied on an earlier launch's data would still pass once; that is what the next check is for.
* **alternating plans**: two plans of different routings take turns.  A row that plan A fills and plan B leaves empty must
  be zero after B's launch, a row both fill must hold B's source; stale rows, a reused flag of the previous epoch or a
  missed zero-fill show up as a mismatch with the index of the first bad row and the rank it should have come from.
* **latency**: the launches' device times, P50 / P99 / longest, with the bytes the plan moves.

The receive tensors are symmetric memory that the peers write directly.  The dispatch kernel lets a peer write them only
after this rank has entered the same launch, so what a launch delivered stays valid until this rank's own next dispatch:
the checks read the tensors on the host while faster ranks may already have launched again.  (A first version of the
kernel had no such meeting, and on two GPUs this tool caught a rank's route weights overwritten by its peer's next launch
while the host was still comparing the rows.)

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m tilexr_b200.tools.moonep.dispatch_hot_loop \\
        --cases perf --case-ids flow_r8_s4096_k8_h7168 --iters 200 --check-every 10
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .contracts import MoonEPCase

MODES = ("hidden", "pair")


def expected_rows(case: MoonEPCase, dsts: Sequence[torch.Tensor], hidden: Sequence[torch.Tensor], weights: Optional[Sequence[torch.Tensor]],
                  rank: int):
    """What rank `rank` must hold after a dispatch: `dsts[s]` / `hidden[s]` / `weights[s]` are source s's plan destinations
    (int, `r * NvS + row`, negative = no row), rows and route weights.  Returns (rows [NvS, H], weights [NvS] or None,
    source rank per row [NvS], -1 where nobody writes)."""
    nvs, K = case.nvs, case.top_k
    rows = torch.zeros(nvs, case.hidden, dtype=hidden[0].dtype)
    wrow = None if weights is None else torch.zeros(nvs, dtype=torch.float32)
    source = torch.full((nvs,), -1, dtype=torch.int32)
    for src, raw in enumerate(dsts):
        raw = raw.to(torch.int64).reshape(-1)
        keep = (raw >= 0) & (raw // nvs == rank)
        route = torch.nonzero(keep).reshape(-1)
        slot = raw[keep] % nvs
        rows[slot] = hidden[src][route // K]
        if wrow is not None:
            wrow[slot] = weights[src].reshape(-1)[route].float()
        source[slot] = src
    return rows, wrow, source


def first_mismatch(got: torch.Tensor, want: torch.Tensor, source: torch.Tensor) -> Optional[Dict[str, object]]:
    """None when equal; else where the first differing row is, which rank it should have come from (-1: it should be empty)
    and how many rows differ."""
    if torch.equal(got, want):
        return None
    bad = (got != want).reshape(got.shape[0], -1).any(dim=1)
    row = int(torch.nonzero(bad)[0])
    g, w = got[row].reshape(-1), want[row].reshape(-1)
    col = int(torch.nonzero(g != w)[0])
    return {"rows_differ": int(bad.sum()), "first_row": row, "first_column": col, "expected_source_rank": int(source[row]),
            "got": float(g[col]), "want": float(w[col]), "got_row_is_zero": bool((g == 0).all())}


def percentiles(samples: Sequence[float]) -> Dict[str, float]:
    s = sorted(samples)
    if not s:
        return {"p50": 0.0, "p99": 0.0, "max": 0.0, "count": 0}
    at = lambda q: s[min(len(s) - 1, int(q * (len(s) - 1) + 0.5))]
    return {"p50": at(0.5), "p99": at(0.99), "max": s[-1], "count": len(s)}


def _gather_cpu(t: torch.Tensor, world: int) -> List[torch.Tensor]:
    if world == 1:
        return [t.cpu()]
    out: List[Optional[torch.Tensor]] = [None] * world
    dist.all_gather_object(out, t.cpu())
    return out


def run_case(comm, case: MoonEPCase, mode: str = "pair", iters: int = 100, warmup: int = 5, check_every: int = 10) -> Dict[str, object]:
    """The three checks of the module docstring on this rank; every rank returns its own record (`ok` is rank-local)."""
    from ...integrations.moonep import TileXRMoonEPBuffer
    from .case_factory import make_inputs, routing

    if mode not in MODES:
        raise ValueError(f"mode must be one of {MODES}")
    world, rank = comm.world_size, comm.rank
    buf = TileXRMoonEPBuffer(comm, case.tokens, case.hidden, case.top_k, case.experts, token_padding=case.token_padding,
                             B=case.prefetch_slots, dtype=case.torch_dtype())
    dev = buf.hidden_nvsh.device
    sets = []
    for variant in range(2):                                  # plan A: the case's routing; plan B: the next seed's
        c = dataclasses.replace(case, seed=case.seed + 101 * variant)
        inp = make_inputs(c, rank, dev)
        topk = routing(c, rank).to(dev)
        plan = buf.planning(topk)
        torch.cuda.synchronize()
        buf.check_pending_status(plan)
        w = inp.route_weights_sk if mode == "pair" else None
        want, want_w, source = expected_rows(case, _gather_cpu(plan.dst, world), _gather_cpu(inp.hidden_sh, world),
                                             None if w is None else _gather_cpu(w, world), rank)
        sets.append({"plan": plan, "hidden": inp.hidden_sh, "weights": w, "want": want, "want_w": want_w, "source": source})

    def launch(s):
        return buf.dispatch(s["hidden"], s["weights"], s["plan"])

    def check(s, rows, wn, what: str, i: int):
        # No meeting of the ranks here: a peer that is already in its next launch must not touch these tensors before this
        # rank launches again (the kernel's entry meeting), and the comparison of the rows takes long enough to show it.
        torch.cuda.synchronize()
        bad = first_mismatch(rows.cpu(), s["want"], s["source"])
        if bad is None and s["want_w"] is not None:
            bad = first_mismatch(wn.cpu().reshape(-1, 1), s["want_w"].reshape(-1, 1), s["source"])
            if bad is not None:
                bad["tensor"] = "route weights"
        if bad is not None:
            bad.update(check=what, iteration=i)
            failures.append(bad)

    failures: List[Dict[str, object]] = []
    for _ in range(warmup):
        launch(sets[0])
    # repeated exact
    for i in range(iters):
        rows, wn = launch(sets[0])
        if check_every > 0 and (i % check_every == 0 or i == iters - 1):
            check(sets[0], rows, wn, "repeated exact", i)
    # alternating plans
    for i in range(iters):
        s = sets[i & 1]
        rows, wn = launch(s)
        if check_every > 0 and (i % check_every <= 1 or i >= iters - 2):
            check(s, rows, wn, "alternating plans", i)
    # latency of back-to-back launches
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in events:
        a.record()
        launch(sets[0])
        b.record()
    torch.cuda.synchronize()
    lat = percentiles([a.elapsed_time(b) * 1e3 for a, b in events])
    status = comm.device_status()
    elem = torch.empty((), dtype=case.torch_dtype()).element_size()
    sent = int((sets[0]["plan"].dst.cpu() >= 0).sum())
    nbytes = sent * (case.hidden * elem + (4 if mode == "pair" else 0))
    buf.close()
    return {"case": case.name, "mode": mode, "rank": rank, "iterations": iters, "ok": not failures and status == 0, "device_status": status,
            "failures": failures[:8], "latency_us": lat, "bytes": nbytes, "gbps_at_p50": 0.0 if lat["p50"] <= 0 else nbytes / lat["p50"] / 1e3}


def run_case_host(comm, case: MoonEPCase, mode: str = "pair", iters: int = 20, check_every: int = 1) -> Dict[str, object]:
    """The repeated-exact and alternating-plans checks on a host-memory communicator (gloo ranks, no GPU): the rows travel
    through the same windows, flags and launch epochs, a launch every time into fresh outputs that the kernel fills or
    zeroes.  Latencies are wall clock around the launch."""
    import time

    from ... import _C
    from .case_factory import make_inputs, routing
    from .host_backend import HostMemoryBackend
    from .planner_reference import dst_local_from_plans, reference_plan

    if mode not in MODES:
        raise ValueError(f"mode must be one of {MODES}")
    rank, K = comm.rank, case.top_k
    gather = HostMemoryBackend(comm)._all_gather
    sets = []
    for variant in range(2):
        c = dataclasses.replace(case, seed=case.seed + 101 * variant)
        inp = make_inputs(c, rank)
        topk = gather(routing(c, rank).to(torch.int32))
        dst = reference_plan(case, topk, rank)["dst"].to(torch.int32).contiguous()
        dsts = gather(dst)
        hidden = inp.hidden_sh.float().contiguous()
        w = inp.route_weights_sk.float().contiguous().reshape(-1) if mode == "pair" else None
        want, want_w, source = expected_rows(dataclasses.replace(case, dtype="float32"), dsts, gather(hidden), None if w is None else gather(w), rank)
        sets.append({"dst": dst, "dst_local": dst_local_from_plans(case, dsts, rank).to(torch.int32), "hidden": hidden, "weights": w, "want": want,
                     "want_w": want_w, "source": source})
    failures: List[Dict[str, object]] = []
    times: List[float] = []

    def launch(s):
        t0 = time.perf_counter()
        out = _C.host_moon_dispatch(comm, s["hidden"], s["weights"], s["dst"], s["dst_local"], K)
        times.append((time.perf_counter() - t0) * 1e6)
        return out

    def check(s, rows, wn, what: str, i: int):
        bad = first_mismatch(rows, s["want"], s["source"])
        if bad is None and s["want_w"] is not None:
            bad = first_mismatch(wn.reshape(-1, 1), s["want_w"].reshape(-1, 1), s["source"])
            if bad is not None:
                bad["tensor"] = "route weights"
        if bad is not None:
            bad.update(check=what, iteration=i)
            failures.append(bad)

    for i in range(iters):
        rows, wn = launch(sets[0])
        if check_every > 0 and (i % check_every == 0 or i == iters - 1):
            check(sets[0], rows, wn, "repeated exact", i)
    for i in range(iters):
        s = sets[i & 1]
        rows, wn = launch(s)
        if check_every > 0 and (i % check_every <= 1 or i >= iters - 2):
            check(s, rows, wn, "alternating plans", i)
    status = comm.device_status()
    sent = int((sets[0]["dst"] >= 0).sum())
    nbytes = sent * (case.hidden * 4 + (4 if mode == "pair" else 0))
    lat = percentiles(times)
    return {"case": case.name, "mode": mode, "rank": rank, "iterations": iters, "ok": not failures and status == 0, "device_status": status,
            "failures": failures[:8], "latency_us": lat, "bytes": nbytes, "gbps_at_p50": 0.0 if lat["p50"] <= 0 else nbytes / lat["p50"] / 1e3}


def main(argv=None) -> int:
    from .case_factory import add_case_arguments, apply_overrides, load_cases, overrides_from_args, select_cases

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--cases", default="smoke")
    add_case_arguments(ap)
    ap.add_argument("--mode", choices=MODES, default="pair")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--check-every", type=int, default=10, help="0: no result checks, latency only")
    ap.add_argument("--json", default="")
    ap.add_argument("--backend", choices=["device", "host"], default="device", help="host: gloo ranks on a host-memory communicator, no GPU")
    args = ap.parse_args(argv)
    import tilexr_b200 as txr

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    host = args.backend == "host"
    if not host:
        torch.cuda.set_device(local)
    cases = [apply_overrides(c, overrides_from_args(args)) for c in select_cases(load_cases(args.cases), args.case_ids) if c.ranks == world]
    need = max([c.nvs * c.hidden * (4 if host else 2) + c.nvs * 4 for c in cases] + [32 << 20])
    buffer_mb = int(2 * need / (1 << 20)) + 64
    if host:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29700 + os.getpid() % 200))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        comm = txr.init_from_torch_distributed(host_memory=True, buffer_mb=buffer_mb)
    elif world > 1:
        dist.init_process_group("nccl")
        comm = txr.init_from_torch_distributed(buffer_mb=buffer_mb)
    else:
        comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{29700 + os.getpid() % 200}", buffer_mb=buffer_mb, device=local)
    results = []
    for c in cases:
        r = run_case_host(comm, c, args.mode, args.iters, args.check_every) if host else run_case(comm, c, args.mode, args.iters, args.warmup, args.check_every)
        if world > 1:
            every: List[Optional[dict]] = [None] * world
            dist.all_gather_object(every, r)
        else:
            every = [r]
        results.append({"case": c.name, "mode": args.mode, "ok": all(x["ok"] for x in every), "ranks": every,
                        "p50_us_slowest_rank": max(x["latency_us"]["p50"] for x in every), "p99_us_slowest_rank": max(x["latency_us"]["p99"] for x in every)})
        if rank == 0:
            x = results[-1]
            print(f"{x['case']} [{x['mode']}]: {'ok' if x['ok'] else 'FAILED'}, P50 {x['p50_us_slowest_rank']:.1f} us, P99 {x['p99_us_slowest_rank']:.1f} us "
                  f"(slowest rank), {every[0]['gbps_at_p50']:.1f} GB/s on rank 0")
            for e in every:
                for f in e["failures"]:
                    print(f"  rank {e['rank']}: {json.dumps(f)}")
    if args.json and rank == 0:
        with open(args.json, "w") as f:
            json.dump(results, f, indent=1)
    comm.destroy()
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0 if all(r["ok"] for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
