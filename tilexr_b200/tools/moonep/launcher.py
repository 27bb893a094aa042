"""Command line of the MoonEP harness (reference: tools/moonep/launcher.py, scripts/run_moonep.sh).

Run under torchrun, one process per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m tilexr_b200.tools.moonep.launcher \\
        --mode correctness --cases smoke
    ... --mode benchmark --cases correctness --json out.json
    ... --mode replay --capture DIR

Cases whose rank count differs from the world size are skipped.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["correctness", "benchmark", "replay"], default="correctness")
    ap.add_argument("--cases", default="smoke", help="name of a case file under cases/ or a path")
    ap.add_argument("--capture", default="", help="replay: directory written by RouteRecorder")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)

    import tilexr_b200 as txr
    from . import report
    from .benchmark import benchmark_case
    from .case_factory import load_cases
    from .correctness import CorrectnessRunner
    from .model_replay import replay
    from .rendezvous import completion_barrier
    from .tilexr_backend import TileXRBackend
    from .torch_reference_backend import TorchReferenceBackend

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl")
        comm = txr.init_from_torch_distributed(buffer_mb=256)
    else:
        comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{29700 + os.getpid() % 200}", buffer_mb=256, device=local)
    results = []
    failed = False
    if args.mode == "replay":
        results = replay(args.capture, comm, iters=max(1, args.iters))
        if rank == 0:
            print(json.dumps(results["total_us"]))
    else:
        cases = [c for c in load_cases(args.cases) if c.ranks == world]
        if not cases and rank == 0:
            print(f"no case of {args.cases} is written for {world} ranks", file=sys.stderr)
        if args.mode == "correctness":
            runner = CorrectnessRunner(TorchReferenceBackend(), TileXRBackend(comm), device="cpu")
            for c in cases:
                r = runner.run_case(c)
                results.append(r)
                failed |= not r["ok_all_ranks"]
            if rank == 0:
                print(report.correctness_markdown(results))
        else:
            for c in cases:
                results.append(benchmark_case(comm, c, iters=args.iters, warmup=args.warmup))
            if rank == 0:
                print(report.benchmark_markdown(results))
    if args.json and rank == 0:
        report.write_json(args.json, results)
    if world > 1:
        key = os.environ.get("TILEXR_MOONEP_BARRIER_KEY", "tilexr-moonep").encode()
        port = int(os.environ.get("MASTER_PORT", "29500")) + 17
        completion_barrier(rank, world, os.environ.get("MASTER_ADDR", "127.0.0.1"), port, key, f"done-{args.mode}")
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
