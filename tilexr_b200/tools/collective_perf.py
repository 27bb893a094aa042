"""nccl-tests style sweep of the collective kernels (and of NCCL, for the baseline column).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29555 \
        -m tilexr_b200.tools.collective_perf --op all_gather --min-bytes 4096 --max-bytes 1073741824 \
        --step-factor 4 --iters 20 --warmup-iters 5 --check 1 --baseline nccl --csv out.csv

Timing follows the reference's perf tool (tests/collectives/tilexr-tests/tilexr_collective_perf.cpp:
964-1048): warm-up launches, then one start/stop CUDA event pair per measured launch; the time
of a size is the max over ranks of each rank's average.  ``algbw = output bytes per rank / time``
and ``busbw = algbw * (R-1)/R`` for every op, which is the reference's convention; for all-reduce
the nccl-tests convention ``2 (R-1)/R`` is printed as well.  ``--symmetric 1`` places the output
in registered memory so that peers write it directly.
"""
from __future__ import annotations

import argparse
import csv
import os
import sys

import torch
import torch.distributed as dist

OPS = ("all_gather", "all_to_all", "all_reduce", "reduce_scatter", "broadcast")
EXTRA_OPS = ("all_to_all_transpose",)      # not part of --op all
TRANSPOSE_BURST = 512                      # elements of one row that go to one peer


def parse(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--op", default="all_gather", choices=OPS + EXTRA_OPS + ("all",))
    p.add_argument("--min-bytes", type=int, default=4096)
    p.add_argument("--max-bytes", type=int, default=64 << 20)
    p.add_argument("--step-factor", type=int, default=4)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup-iters", type=int, default=5)
    p.add_argument("--datatype", default="bfloat16")
    p.add_argument("--check", type=int, default=1)
    p.add_argument("--baseline", default="none", choices=["none", "nccl"])
    p.add_argument("--symmetric", type=int, default=0)
    p.add_argument("--buffer-mb", type=int, default=1024)
    p.add_argument("--csv", default="")
    p.add_argument("--min-algbw", type=float, default=0.0)
    p.add_argument("--max-latency-us", type=float, default=0.0)
    p.add_argument("--comm-mode", default="device", choices=["device", "host"],
                   help="host: the same sweep on a host-memory communicator under gloo (fp32, wall-clock times): the plumbing without a GPU")
    return p.parse_args(argv)


def message_elems(op: str, nbytes: int, world: int, esize: int):
    """Elements of (input, output) for a per-rank message of nbytes."""
    n = max(nbytes // esize, 1)
    if op == "all_gather":
        return n, n * world
    if op == "all_to_all":
        n = max(n // world, 1) * world
        return n, n
    if op == "all_to_all_transpose":
        width = world * TRANSPOSE_BURST
        n = max(n // width, 1) * width
        return n, n
    if op == "reduce_scatter":
        n = max(n // world, 1)
        return n * world, n
    return n, n


def run_ours(txr, comm, op, x, out, keep=False):
    if op == "all_gather":
        txr.all_gather(comm, x, out=out)
    elif op == "all_to_all":
        txr.all_to_all(comm, x, out=out)
    elif op == "all_to_all_transpose":
        # the sending kernel gathers the column blocks; the result is a fresh tensor, as for the NCCL arm's transpose
        res = txr.collectives.all_to_all_transpose(comm, x.view(-1, comm.world_size * TRANSPOSE_BURST))
        if keep:
            out.copy_(res.reshape(-1))
    elif op == "all_reduce":
        txr.all_reduce(comm, x, out=out)
    elif op == "reduce_scatter":
        txr.reduce_scatter(comm, x, out=out)
    else:
        txr.broadcast(comm, out, root=0)


def run_nccl(op, x, out):
    if op == "all_gather":
        dist.all_gather_into_tensor(out, x)
    elif op == "all_to_all":
        dist.all_to_all_single(out, x)
    elif op == "all_to_all_transpose":
        world = dist.get_world_size()
        dist.all_to_all_single(out, x.view(-1, world, TRANSPOSE_BURST).transpose(0, 1).contiguous())
    elif op == "all_reduce":
        out.copy_(x)
        dist.all_reduce(out)
    elif op == "reduce_scatter":
        dist.reduce_scatter_tensor(out, x)
    else:
        dist.broadcast(out, src=0)


def time_launches(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0)
    avg = sum(times) / len(times)
    t = torch.tensor([avg, min(times), max(times)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def pattern(src: int, n: int) -> torch.Tensor:
    """Rank `src`'s input: small integers in fp32, so that every sum is exact and a misplaced element shows its origin."""
    i = torch.arange(n, dtype=torch.int64)
    return ((i * 7 + src * 13) % 251 - 125).to(torch.float32)


def expected_host(op: str, world: int, rank: int, n_in: int) -> torch.Tensor:
    """What `rank` must hold after `op` when every rank s sends pattern(s, n_in) (root 0 for the broadcast)."""
    ins = [pattern(s, n_in) for s in range(world)]
    if op == "all_gather":
        return torch.cat(ins)
    if op == "all_to_all":
        c = n_in // world
        return torch.cat([ins[s][rank * c:(rank + 1) * c] for s in range(world)])
    total = torch.stack(ins).sum(0)
    if op == "all_reduce":
        return total
    if op == "reduce_scatter":
        c = n_in // world
        return total[rank * c:(rank + 1) * c]
    return ins[0]


def main_host(args) -> int:
    """The sweep on host-memory windows: the host kernels on the production flag primitives between gloo ranks, checked against
    the pattern; times are wall clock around each launch (max over ranks of the average), which says how the plumbing behaves,
    not how a GPU would."""
    import time

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import tilexr_b200 as txr

    comm = txr.init_from_torch_distributed(host_memory=True, buffer_mb=min(args.buffer_mb, 256))
    C = txr._C
    tile = 16384
    ops = [o for o in (OPS if args.op == "all" else (args.op,))]
    if any(o in EXTRA_OPS for o in ops):
        raise SystemExit("--comm-mode host has the five plain collectives")
    rows, failures = [], 0
    if rank == 0:
        print(f"# ranks {world}  host memory, fp32  iters {args.iters}")
        print(f"# {'op':<15}{'bytes':>12}{'avg us':>10}{'min us':>10}{'max us':>10}{'algbw GB/s':>12}{'busbw GB/s':>12}{'errors':>8}")
    # the window holds one slice per source and at most 1024 tiles per pair
    limit = min(((comm.data_half_bytes // max(world, 1)) & ~255), 1024 * tile)
    for op in ops:
        size = args.min_bytes
        while size <= args.max_bytes:
            n_in, n_out = message_elems(op, size, world, 4)
            per_pair = (n_in if op in ("all_gather", "all_reduce", "broadcast") else n_in // world) * 4      # bytes one source leaves in one window
            if per_pair > limit:
                break
            x = pattern(rank, n_in)

            def launch():
                if op == "all_gather":
                    out = torch.empty(n_out)
                    C.host_all_gather(comm, x, out, tile)
                    return out
                if op == "all_to_all":
                    return C.host_all_to_all(comm, x, tile)
                if op == "all_reduce":
                    return C.host_all_reduce(comm, x)
                if op == "reduce_scatter":
                    return C.host_reduce_scatter(comm, x)
                b = x.clone() if rank == 0 else torch.zeros(n_in)
                C.host_broadcast(comm, b, 0, tile)
                return b

            errors = 0
            if args.check:
                errors = int((launch() != expected_host(op, world, rank, n_in)).sum())
            for _ in range(args.warmup_iters):
                launch()
            dist.barrier()
            times = []
            for _ in range(args.iters):
                t0 = time.perf_counter()
                launch()
                times.append((time.perf_counter() - t0) * 1e6)
            t = torch.tensor([sum(times) / len(times), min(times), max(times), float(errors)], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            avg, mn, mx, errors = float(t[0]), float(t[1]), float(t[2]), int(t[3])
            out_bytes = n_out * 4
            algbw = out_bytes / avg / 1000.0
            busbw = algbw * (world - 1) / world
            failures += errors
            rows.append([op, world, size, out_bytes, avg, mn, mx, algbw, busbw, float("nan"), float("nan"), float("nan"), errors])
            if rank == 0:
                print(f"  {op:<15}{size:>12}{avg:>10.1f}{mn:>10.1f}{mx:>10.1f}{algbw:>12.2f}{busbw:>12.2f}{errors:>8}", flush=True)
            size *= args.step_factor
    if rank == 0 and args.csv:
        write_csv(args.csv, rows)
    comm.destroy()
    dist.destroy_process_group()
    return 1 if failures else 0


def write_csv(path: str, rows) -> None:
    with open(path, "w", newline="") as f:
        wr = csv.writer(f)
        wr.writerow(["op", "ranks", "bytes_per_rank", "output_bytes", "avg_us", "min_us", "max_us", "algbw_GBps",
                     "busbw_GBps", "nccl_avg_us", "nccl_busbw_GBps", "speedup_vs_nccl", "errors"])
        wr.writerows(rows)


def main(argv=None):
    args = parse(argv)
    if args.comm_mode == "host":
        return main_host(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    import tilexr_b200 as txr

    comm = txr.init_from_torch_distributed(buffer_mb=args.buffer_mb)
    dtype = getattr(torch, args.datatype)
    esize = torch.empty((), dtype=dtype).element_size()
    ops = OPS if args.op == "all" else (args.op,)
    rows = []
    failures = 0
    if rank == 0:
        print(f"# ranks {world}  dtype {args.datatype}  iters {args.iters}  symmetric {args.symmetric}")
        print(f"# {'op':<15}{'bytes':>12}{'avg us':>10}{'min us':>10}{'max us':>10}{'algbw GB/s':>12}{'busbw GB/s':>12}"
              f"{'nccl us':>10}{'nccl bus':>10}{'speedup':>9}{'errors':>8}")
    for op in ops:
        size = args.min_bytes
        while size <= args.max_bytes:
            n_in, n_out = message_elems(op, size, world, esize)
            g = torch.Generator(device="cuda").manual_seed(1000 + rank)
            if dtype.is_floating_point:
                x = (torch.rand(n_in, device="cuda", generator=g) * 2 - 1).to(dtype)
            else:
                x = torch.randint(-100, 100, (n_in,), device="cuda", generator=g).to(dtype)
            out = comm.symm_empty([n_out], dtype) if args.symmetric else torch.empty(n_out, dtype=dtype, device="cuda")
            if op == "broadcast":
                out.copy_(x)
            errors = 0
            if args.check:
                ref = torch.empty_like(out)
                if op == "broadcast":
                    ref.copy_(x)
                run_ours(txr, comm, op, x, out, keep=True)
                if dtype.is_floating_point and op in ("all_reduce", "reduce_scatter"):
                    # reference summed in fp32 and rounded once (NCCL may accumulate 16-bit types in their own
                    # precision hop by hop, which alone exceeds a 2 % tolerance now and then at 8 ranks)
                    ref32 = torch.empty(out.shape, dtype=torch.float32, device=out.device)
                    run_nccl(op, x.float(), ref32)
                    torch.cuda.synchronize()
                    errors = int((~torch.isclose(out.float(), ref32.to(dtype).float(), rtol=2e-2, atol=2e-2)).sum().item())
                else:
                    run_nccl(op, x, ref)
                    torch.cuda.synchronize()
                    errors = int((out != ref).sum().item())
                if comm.device_status() != 0:
                    errors += 1
            avg, mn, mx = time_launches(lambda: run_ours(txr, comm, op, x, out), args.iters, args.warmup_iters)
            out_bytes = n_out * esize
            algbw = out_bytes / avg / 1000.0
            busbw = algbw * (world - 1) / world
            nccl_avg = nccl_bus = speed = float("nan")
            if args.baseline == "nccl":
                nccl_avg, _, _ = time_launches(lambda: run_nccl(op, x, out), args.iters, args.warmup_iters)
                nccl_bus = out_bytes / nccl_avg / 1000.0 * (world - 1) / world
                speed = nccl_avg / avg
            failures += errors
            if args.min_algbw and algbw < args.min_algbw:
                failures += 1
            if args.max_latency_us and avg > args.max_latency_us:
                failures += 1
            rows.append([op, world, size, out_bytes, avg, mn, mx, algbw, busbw, nccl_avg, nccl_bus, speed, errors])
            if rank == 0:
                print(f"  {op:<15}{size:>12}{avg:>10.1f}{mn:>10.1f}{mx:>10.1f}{algbw:>12.2f}{busbw:>12.2f}"
                      f"{nccl_avg:>10.1f}{nccl_bus:>10.2f}{speed:>9.2f}{errors:>8}", flush=True)
            if args.symmetric:
                comm.symm_free(out)
            del x, out
            size *= args.step_factor
    if rank == 0 and args.csv:
        write_csv(args.csv, rows)
    comm.destroy()
    dist.destroy_process_group()
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
