"""Command line of the MoonEP harness (reference: tools/moonep/launcher.py, scripts/run_moonep.sh).

Run under torchrun, one process per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m tilexr_b200.tools.moonep.launcher \\
        --mode correctness --cases smoke [--dump DIR]
    ... --mode benchmark --cases perf --json out.json --csv out.csv --samples DIR
    ... --mode prefetch --cases perf          (PrefetchWeight on its own, synthetic borrow table)
    ... --mode reduce-grad --cases perf       (ReduceGrad on its own)
    ... --mode replay --capture DIR
    ... --mode model-flow --cases perf --layers 5 --iters 5 --json performance.json   (the operator sequence of a training step)
    python -m tilexr_b200.tools.moonep.launcher --mode aggregate --samples DIR   (no GPU: folds rank*.jsonl of several nodes)

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
    ap.add_argument("--mode", choices=["correctness", "benchmark", "prefetch", "reduce-grad", "replay", "model-flow", "aggregate"], default="correctness")
    ap.add_argument("--cases", default="smoke", help="name of a case file under cases/ or a path")
    from .case_factory import add_case_arguments, apply_overrides, overrides_from_args, select_cases

    add_case_arguments(ap)
    ap.add_argument("--capture", default="", help="replay: directory written by RouteRecorder")
    ap.add_argument("--layers", type=int, default=5, help="model-flow: MoE layers of the step")
    ap.add_argument("--no-recompute", action="store_true", help="model-flow: backward without recomputing the forward operators")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default="")
    ap.add_argument("--csv", default="", help="benchmark modes: one row per (case, stage) with P50 / P99")
    ap.add_argument("--samples", default="", help="benchmark: directory for per-rank sample files; aggregate: where to read them")
    ap.add_argument("--stage-barrier", action="store_true",
                    help="benchmark: synchronise the device and the ranks in front of every stage, so that a stage's time excludes the skew of the one before")
    ap.add_argument("--nccl-baseline", action="store_true",
                    help="benchmark: also time dispatch and combine as a torch + NCCL program (index_select, all_to_all_single with the plan's splits, index_add_)")
    ap.add_argument("--dump", default="", help="correctness: directory for both sides' stage tensors (compare offline with tools.moonep.tensor_dump)")
    ap.add_argument("--trace", action="store_true", help="benchmark: also record the dispatch kernel's event trace once per case and print its phases")
    ap.add_argument("--backend", choices=["device", "host"], default="device",
                    help="correctness: 'host' runs the stages on a host-memory communicator (gloo ranks, no GPU): the same windows, flags and "
                         "launch epochs with memcpy for the copies")
    ap.add_argument("--buffer-mb", type=int, default=0, help="communicator window size (default: sized for the largest case)")
    args = ap.parse_args(argv)

    if args.mode == "aggregate":
        from . import report as _report

        rows = _report.aggregate_rank_artifacts(args.samples)
        for r in rows:
            s = r["cross_rank_max"]
            print(f"{r['case']} {r['stage']}: P50 {s['p50']:.1f} us, P99 {s['p99']:.1f} us, {r['gbps_at_p50']:.1f} GB/s ({s['invalid']} invalid)")
        if args.json:
            _report.write_json(args.json, rows)
        return 0

    import tilexr_b200 as txr
    from . import report
    from .benchmark import benchmark_case
    from .prefetch_weight_benchmark import prefetch_weight_benchmark
    from .reduce_grad_benchmark import reduce_grad_benchmark
    from .case_factory import load_cases
    from .correctness import CorrectnessRunner
    from .model_replay import replay
    from .rendezvous import completion_barrier
    from .tilexr_backend import TileXRBackend
    from .torch_reference_backend import TorchReferenceBackend

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    host = args.backend == "host"
    if host and args.mode not in ("correctness", "replay", "model-flow"):
        ap.error("--backend host runs the correctness, replay and model-flow modes only")
    if not host:
        torch.cuda.set_device(local)
    buffer_mb = args.buffer_mb
    if buffer_mb <= 0:
        # two halves, each holding the K rows per token that a combine receives, of the largest case that will run
        buffer_mb = 256
        if args.mode != "replay":
            for c in select_cases(load_cases(args.cases), args.case_ids):
                if c.ranks == world:
                    c = apply_overrides(c, overrides_from_args(args))
                    need = c.nvs * c.hidden * (4 if host else 2) + c.nvs * 4
                    buffer_mb = max(buffer_mb, int(2 * need / (1 << 20)) + 64)
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
    failed = False
    if args.mode == "replay":
        if host:
            from .model_replay import replay_host

            results = replay_host(args.capture, comm, iters=max(1, args.iters))
            failed |= not results["verified"]
        else:
            results = replay(args.capture, comm, iters=max(1, args.iters))
        if rank == 0:
            print(json.dumps(results["total_us"]))
    else:
        cases = [apply_overrides(c, overrides_from_args(args)) for c in select_cases(load_cases(args.cases), args.case_ids) if c.ranks == world]
        if not cases and rank == 0:
            print(f"no case of {args.cases} is written for {world} ranks", file=sys.stderr)
        if args.mode == "model-flow":
            from . import model_flow

            for c in cases:
                if host:
                    doc = model_flow.run_case_host(comm, c, layers=args.layers, iters=max(1, args.iters), warmup=max(0, args.warmup), recompute=not args.no_recompute)
                else:
                    doc = model_flow.run_case(comm, c, layers=args.layers, iters=max(1, args.iters), warmup=max(1, args.warmup), recompute=not args.no_recompute)
                if world > 1:
                    docs = [None] * world
                    dist.all_gather_object(docs, doc)
                    doc = model_flow.merge_rank_documents(docs)
                results.append(doc)
                if rank == 0:
                    print(model_flow.markdown(doc))
        elif args.mode == "correctness":
            if host:
                from .host_backend import HostMemoryBackend

                candidate = HostMemoryBackend(comm)
            else:
                candidate = TileXRBackend(comm)
            runner = CorrectnessRunner(TorchReferenceBackend(), candidate, device="cpu", dump_dir=args.dump)
            for c in cases:
                r = runner.run_case(c)
                results.append(r)
                failed |= not r["ok_all_ranks"]
            if rank == 0:
                print(report.correctness_markdown(results))
        else:
            run = {"benchmark": lambda c: benchmark_case(comm, c, iters=args.iters, warmup=args.warmup, sample_dir=args.samples, trace=args.trace, nccl_baseline=args.nccl_baseline,
                                                      stage_barrier=args.stage_barrier),
                   "prefetch": lambda c: prefetch_weight_benchmark(comm, c, iters=args.iters, warmup=args.warmup),
                   "reduce-grad": lambda c: reduce_grad_benchmark(comm, c, iters=args.iters, warmup=args.warmup)}[args.mode]
            for c in cases:
                if args.mode != "benchmark" and c.ffn <= 0:
                    continue
                r = run(c)
                results.append(r)
                failed |= r.get("verified") is False
            if rank == 0:
                print(report.benchmark_markdown(results))
                for r in results:
                    if "nccl_baseline_us" in r:
                        b = r["nccl_baseline_us"]
                        print(f"{r['case']} torch + NCCL: dispatch {b['dispatch']:.1f} us, combine {b['combine']:.1f} us "
                              f"(this library: {r['stage_us']['dispatch']:.1f} / {r['stage_us']['combine']:.1f})")
                    for ph in r.get("dispatch_phases", []):
                        print(f"{r['case']} dispatch phase {ph['phase']}: {ph['count']} events, mean {ph['mean_us']:.1f} us, "
                              f"longest {ph['max_us']:.1f} us, {ph['bytes'] / 1e6:.1f} MB, {ph['rows']} rows")
                if args.csv:
                    report.write_stage_csv(args.csv, results)
    if args.json and rank == 0:
        report.write_json(args.json, results)
    if world > 1:
        key = os.environ.get("TILEXR_MOONEP_BARRIER_KEY", "tilexr-moonep").encode()
        port = int(os.environ.get("MASTER_PORT", "29500")) + 17
        completion_barrier(rank, world, os.environ.get("MASTER_ADDR", "127.0.0.1"), port, key, f"done-{args.mode}")
    comm.destroy()
    if dist.is_initialized():
        dist.destroy_process_group()
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
