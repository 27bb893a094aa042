"""Collectives through the NVSwitch multicast object against NCCL and against this package's
peer-to-peer kernels: numerics first (against an fp32 sum of all ranks' inputs), then device times.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29561 \
        -m tilexr_b200.tools.nvls_perf --sizes-kb 64,1024,16384,262144 --json out.json

Every time is the maximum over ranks of a CUDA-event measurement on the launching stream.  When the GPUs
cannot be bound to a multicast object the tool prints ``{"nvls": "unavailable", ...}`` and exits 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def timed(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1000.0 / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def check(ws, comm, rank, world, dtype, n):
    """Numerics of the four operations on `n` elements per rank; returns a list of failures."""
    from tilexr_b200.ops import nvls  # noqa: F401

    bad = []
    gens = [torch.Generator().manual_seed(500 + r) for r in range(world)]
    xs = [torch.randn(n, generator=g).to(dtype) for g in gens]
    ref = torch.zeros(n, dtype=torch.float32)
    for x in xs:
        ref += x.float()
    mine = xs[rank].cuda()
    tol = 1e-5 if dtype == torch.float32 else (2e-2 if dtype == torch.bfloat16 else 4e-3)
    scale = ref.abs().max().item() + 1e-6

    buf = ws.view(dtype, n)
    buf.copy_(mine)
    ws.all_reduce_(buf)
    torch.cuda.synchronize()
    got = buf.cpu().float()
    if (got - ref).abs().max().item() > tol * scale:
        bad.append(f"all_reduce {dtype}: max err {(got - ref).abs().max().item():.4g}")
    # every rank holds the same bits
    gathered = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(gathered, buf.clone())
    if not all(torch.equal(gathered[0], g) for g in gathered):
        bad.append(f"all_reduce {dtype}: ranks differ")

    buf.copy_(mine)
    rs = ws.reduce_scatter(buf)
    torch.cuda.synchronize()
    per = n // world
    if (rs.cpu().float() - ref[rank * per:(rank + 1) * per]).abs().max().item() > tol * scale:
        bad.append(f"reduce_scatter {dtype}")
    dist.barrier()

    shard = mine[:per].contiguous()
    ws.all_gather_(shard, buf)
    torch.cuda.synchronize()
    want = torch.cat([x[:per] for x in xs])
    if not torch.equal(buf.cpu(), want):
        bad.append(f"all_gather {dtype}")
    dist.barrier()

    root = world - 1
    ws.broadcast_(buf, root, src=mine if rank == root else None)
    torch.cuda.synchronize()
    if not torch.equal(buf.cpu(), xs[root]):
        bad.append(f"broadcast {dtype}")
    dist.barrier()

    y = ws.all_reduce(mine.reshape(4, -1))
    torch.cuda.synchronize()
    if y.shape != (4, n // 4) or (y.cpu().float().reshape(-1) - ref).abs().max().item() > tol * scale:
        bad.append(f"all_reduce (copying form) {dtype}")
    if dtype != torch.float32:
        bad += check_norm(ws, rank, world, dtype)
    if comm.device_status() != 0:
        bad.append(f"device status {comm.device_status()}")
    return bad


def norm_reference(xs, res, gamma, eps, dtype):
    """fp32 oracle of the fused op; the sum of x is rounded to the storage type first, as it leaves the switch."""
    total = torch.zeros_like(xs[0], dtype=torch.float32)
    for x in xs:
        total += x.float()
    new_res = (total.to(dtype).float() + res.float()).to(dtype)
    v = new_res.float()
    y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    return y.to(dtype), new_res


def check_norm(ws, rank, world, dtype, rows=37, h=1024):
    bad = []
    gens = [torch.Generator().manual_seed(900 + r) for r in range(world)]
    xs = [torch.randn(rows, h, generator=g).to(dtype) for g in gens]
    g0 = torch.Generator().manual_seed(77)
    res = torch.randn(rows, h, generator=g0).to(dtype)
    gamma = (1 + 0.1 * torch.randn(h, generator=g0)).to(dtype)
    n = rows * h
    size = n * 2
    x = ws.view(dtype, n, 0).view(rows, h)
    r = ws.view(dtype, n, (size + 255) // 256 * 256).view(rows, h)
    y = ws.view(dtype, n, 2 * ((size + 255) // 256 * 256)).view(rows, h)
    want_y, want_res = norm_reference(xs, res, gamma, 1e-6, dtype)
    tol = 3e-2 if dtype == torch.bfloat16 else 4e-3
    for out in (y, x):                       # separate output, then in place
        x.copy_(xs[rank])
        r.copy_(res)
        torch.cuda.synchronize()
        dist.barrier()                       # nobody multicasts into a buffer that a peer is still filling
        ws.all_reduce_rmsnorm_(x, gamma.cuda(), residual=r, eps=1e-6, y=out)
        torch.cuda.synchronize()
        ey = (out.cpu().float() - want_y.float()).abs().max().item()
        er = (r.cpu().float() - want_res.float()).abs().max().item()
        if ey > tol * (want_y.float().abs().max().item() + 1) or er > tol * (want_res.float().abs().max().item() + 1):
            bad.append(f"all_reduce_rmsnorm {dtype}: y err {ey:.4g}, residual err {er:.4g}")
        dist.barrier()
    x.copy_(xs[rank])
    torch.cuda.synchronize()
    dist.barrier()
    ws.all_reduce_rmsnorm_(x, gamma.cuda(), eps=1e-6, y=y)     # without a residual
    torch.cuda.synchronize()
    want_y2, _ = norm_reference(xs, torch.zeros_like(res), gamma, 1e-6, dtype)
    if (y.cpu().float() - want_y2.float()).abs().max().item() > tol * (want_y2.float().abs().max().item() + 1):
        bad.append(f"all_reduce_rmsnorm without residual {dtype}")
    dist.barrier()
    return bad


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--sizes-kb", default="64,1024,16384,262144")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--json", default="")
    p.add_argument("--check-only", action="store_true")
    p.add_argument("--norm-batches", default="", help="also time all-reduce + residual + RMSNorm for these batch sizes (hidden 8192)")
    p.add_argument("--hidden", type=int, default=8192)
    args = p.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29561")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    import tilexr_b200 as txr
    from tilexr_b200.ops import nvls

    sizes = [int(v) << 10 for v in args.sizes_kb.split(",")]
    comm = txr.init_from_torch_distributed(buffer_mb=1024)
    norm_batches = [int(v) for v in args.norm_batches.split(",") if v]
    norm_bytes = max([3 * (b * args.hidden * 2 + 256) for b in norm_batches] + [0])
    try:
        ws = nvls.Workspace(comm, max(sizes + [1 << 20, norm_bytes]))
    except (nvls.NvlsUnavailable, RuntimeError) as e:  # the allocator raises RuntimeError without multicast support
        if rank == 0:
            print(json.dumps({"nvls": "unavailable", "why": str(e).splitlines()[0][:200], "world": world}))
        dist.destroy_process_group()
        return 0

    failures = []
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        failures += check(ws, comm, rank, world, dtype, 8 * world * 1024 + 8 * world)
    flag = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(flag)
    if flag.item() != 0:
        print(f"rank {rank}: NVLS numerics FAILED: {failures}", file=sys.stderr)
        dist.destroy_process_group()
        return 1
    out = {"nvls": "ok", "world": world, "numerics": "pass", "rows": []}
    if not args.check_only:
        for nbytes in sizes:
            n = nbytes // 2
            x = torch.randn(n, device="cuda").to(torch.bfloat16)
            buf = ws.view(torch.bfloat16, n)
            buf.copy_(x)
            y = torch.empty_like(x)
            shard = x[: n // world].contiguous()
            rs_out = torch.empty_like(shard)
            ag_out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
            row = {"bytes": nbytes}
            row["nvls_all_reduce_us"] = timed(lambda: ws.all_reduce_(buf), args.iters, 5)
            row["p2p_all_reduce_us"] = timed(lambda: txr.all_reduce(comm, x, out=y), args.iters, 5)
            row["nccl_all_reduce_us"] = timed(lambda: dist.all_reduce(x), args.iters, 5)
            x.normal_()
            buf.copy_(x)
            row["nvls_reduce_scatter_us"] = timed(lambda: ws.reduce_scatter(buf, rs_out), args.iters, 5)
            row["p2p_reduce_scatter_us"] = timed(lambda: txr.reduce_scatter(comm, x, out=rs_out), args.iters, 5)
            row["nccl_reduce_scatter_us"] = timed(lambda: dist.reduce_scatter_tensor(rs_out, x), args.iters, 5)
            row["nvls_all_gather_us"] = timed(lambda: ws.all_gather_(shard, buf), args.iters, 5)
            row["p2p_all_gather_us"] = timed(lambda: txr.all_gather(comm, shard, out=ag_out.view(world, -1)), args.iters, 5)
            row["nccl_all_gather_us"] = timed(lambda: dist.all_gather_into_tensor(ag_out, shard), args.iters, 5)
            row["nvls_broadcast_us"] = timed(lambda: ws.broadcast_(buf, 0), args.iters, 5)
            row["p2p_broadcast_us"] = timed(lambda: txr.broadcast(comm, x, root=0), args.iters, 5)
            row["nccl_broadcast_us"] = timed(lambda: dist.broadcast(x, 0), args.iters, 5)
            x.normal_()
            out["rows"].append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
        out["norm_rows"] = []
        H = args.hidden
        gamma = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        for b in norm_batches:
            n = b * H
            stride = (n * 2 + 255) // 256 * 256
            x = ws.view(torch.bfloat16, n, 0).view(b, H)
            r = ws.view(torch.bfloat16, n, stride).view(b, H)
            y = ws.view(torch.bfloat16, n, 2 * stride).view(b, H)
            x.normal_()
            r.zero_()
            lx = torch.randn(b, H, device="cuda").to(torch.bfloat16)
            lr = torch.zeros_like(lx)
            ly = torch.empty_like(lx)
            torch.cuda.synchronize()
            dist.barrier()

            def nccl_path():
                dist.all_reduce(lx)
                lr.add_(lx)
                v = lr.float()
                ly.copy_(v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float())

            row = {"batch": b, "bytes": n * 2}
            row["nvls_fused_us"] = timed(lambda: ws.all_reduce_rmsnorm_(x, gamma, residual=r, eps=1e-6, y=y), args.iters, 5)
            row["p2p_fused_us"] = timed(lambda: txr.collectives.all_reduce_rmsnorm(comm, lx, gamma, 1e-6, residual=lr, out=ly), args.iters, 5)
            row["nccl_torch_us"] = timed(nccl_path, args.iters, 5)
            out["norm_rows"].append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
        torch.cuda.synchronize()
        if comm.device_status() != 0:
            print(f"rank {rank}: device status {comm.device_status()}", file=sys.stderr)
            dist.destroy_process_group()
            return 1
    if rank == 0:
        print(json.dumps(out if args.check_only else {k: v for k, v in out.items() if k not in ("rows", "norm_rows")}))
        if args.json:
            with open(args.json, "w") as f:
                json.dump(out, f, indent=1)
    dist.barrier()
    del ws
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
