"""Tensor-parallel MLP benchmark: all-gather -> GEMM on the up/gate projection and
GEMM -> reduce-scatter on the down projection (Llama-3-70B: hidden 8192, FFN 28672), against
NCCL + cuBLAS doing the same in two steps.  Also times the plain tcgen05 GEMM against cuBLAS.

    python -m tilexr_b200.tools.tp_mlp_perf                      # 1 GPU: GEMM vs cuBLAS
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29556 \
        -m tilexr_b200.tools.tp_mlp_perf --tokens 8192
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def timed(fn, iters=10, warmup=3, world=1):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / iters
    if world > 1:
        t = torch.tensor([us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item())
    return us


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--tokens", type=int, default=8192)
    p.add_argument("--hidden", type=int, default=8192)
    p.add_argument("--ffn", type=int, default=28672)
    p.add_argument("--iters", type=int, default=10)
    args = p.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    import tilexr_b200 as txr

    out = {"ranks": world, "tokens": args.tokens, "hidden": args.hidden, "ffn": args.ffn}
    g = torch.Generator(device="cuda").manual_seed(rank)
    T, H, F = args.tokens, args.hidden, args.ffn
    if world == 1:
        shapes = [(T, 2 * F // 8, H), (T, H, F // 8), (4096, 4096, 4096), (8192, 8192, 8192)]
        res = []
        for (m, n, k) in shapes:
            a = (torch.randn(m, k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
            b = (torch.randn(n, k, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
            ours = timed(lambda: txr.gemm.matmul(a, b), args.iters)
            cublas = timed(lambda: torch.matmul(a, b.t()), args.iters)
            err = (txr.gemm.matmul(a, b).float() - torch.matmul(a, b.t()).float()).abs().max().item()
            fl = 2.0 * m * n * k
            res.append({"m": m, "n": n, "k": k, "tilexr_us": ours, "cublas_us": cublas, "tilexr_tflops": fl / ours / 1e6,
                        "cublas_tflops": fl / cublas / 1e6, "max_abs_diff_vs_cublas": err})
        out["gemm"] = res
        print(json.dumps(out))
        return 0

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29556")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    comm = txr.init_from_torch_distributed(buffer_mb=256)
    rows = T // world
    fl_loc = F // world
    x = (torch.randn(rows, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w13 = (torch.randn(2 * fl_loc, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(H, fl_loc, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    act = (torch.randn(T, fl_loc, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    stage_a = comm.symm_empty([T, H], torch.bfloat16)
    stage_c = comm.symm_empty([T, H], torch.bfloat16)
    gathered = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    red = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")

    def nccl_ag_gemm():
        dist.all_gather_into_tensor(gathered, x)
        return torch.matmul(gathered, w13.t())

    def nccl_gemm_rs():
        full = torch.matmul(act, w2.t())
        dist.reduce_scatter_tensor(red, full)
        return red

    ours_ag = txr.gemm.all_gather_matmul(comm, x, w13, stage_a)
    ref_ag = nccl_ag_gemm()
    ours_rs = txr.gemm.matmul_reduce_scatter(comm, act, w2, stage_c)
    ref_rs = nccl_gemm_rs().clone()
    torch.cuda.synchronize()
    out["ag_gemm_max_diff"] = (ours_ag.float() - ref_ag.float()).abs().max().item()
    out["gemm_rs_max_diff"] = (ours_rs.float() - ref_rs.float()).abs().max().item()
    out["status"] = comm.device_status()
    out["ag_gemm_us"] = timed(lambda: txr.gemm.all_gather_matmul(comm, x, w13, stage_a), args.iters, 3, world)
    out["nccl_ag_gemm_us"] = timed(nccl_ag_gemm, args.iters, 3, world)
    out["gemm_only_us"] = timed(lambda: torch.matmul(gathered, w13.t()), args.iters, 3, world)
    out["gemm_rs_us"] = timed(lambda: txr.gemm.matmul_reduce_scatter(comm, act, w2, stage_c), args.iters, 3, world)
    out["nccl_gemm_rs_us"] = timed(nccl_gemm_rs, args.iters, 3, world)
    fl_ag = 2.0 * T * 2 * fl_loc * H
    fl_rs = 2.0 * T * H * fl_loc
    out["ag_gemm_tflops"] = fl_ag / out["ag_gemm_us"] / 1e6
    out["gemm_rs_tflops"] = fl_rs / out["gemm_rs_us"] / 1e6
    out["ag_bytes_per_rank"] = (world - 1) * rows * H * 2
    out["rs_bytes_per_rank"] = (world - 1) * rows * H * 2
    if rank == 0:
        print(json.dumps(out))
    comm.destroy()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
