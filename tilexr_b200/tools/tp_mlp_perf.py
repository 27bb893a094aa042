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
    p.add_argument("--fp8-block", type=int, default=1,
                   help="also time the block-scaled fp8 variants (1 x 128 activation scales, 128 x 128 weight scales) of both fusions "
                        "against the same GEMM behind an NCCL all-gather of rows and scales / in front of an NCCL reduce-scatter")
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
    out["tilexr_gemm_only_us"] = timed(lambda: txr.gemm.matmul(gathered, w13), args.iters, 3, world)
    out["gemm_rs_us"] = timed(lambda: txr.gemm.matmul_reduce_scatter(comm, act, w2, stage_c), args.iters, 3, world)
    out["rs_tilexr_gemm_only_us"] = timed(lambda: txr.gemm.matmul(act, w2), args.iters, 3, world)
    out["rs_cublas_gemm_only_us"] = timed(lambda: torch.matmul(act, w2.t()), args.iters, 3, world)
    out["nccl_gemm_rs_us"] = timed(nccl_gemm_rs, args.iters, 3, world)
    fl_ag = 2.0 * T * 2 * fl_loc * H
    fl_rs = 2.0 * T * H * fl_loc
    out["ag_gemm_tflops"] = fl_ag / out["ag_gemm_us"] / 1e6
    out["gemm_rs_tflops"] = fl_rs / out["gemm_rs_us"] / 1e6
    out["ag_bytes_per_rank"] = (world - 1) * rows * H * 2
    out["rs_bytes_per_rank"] = (world - 1) * rows * H * 2
    if args.fp8_block and rows % 256 == 0 and H % 512 == 0 and fl_loc % 128 == 0:
        qx, sx = txr.quant.fp8_quant_1x128(x)
        qact, sact = txr.quant.fp8_quant_1x128(act)
        qw13, sw13 = txr.gemm.quantize_weight_128x128(w13.float())
        qw2, sw2 = txr.gemm.quantize_weight_128x128(w2.float())
        stage_q = comm.symm_empty([T, H], torch.float8_e4m3fn)
        stage_s = comm.symm_empty([T, H // 128], torch.float32)
        gathered_q = torch.empty(T, H, dtype=torch.float8_e4m3fn, device="cuda")
        gathered_s = torch.empty(T, H // 128, dtype=torch.float32, device="cuda")

        def nccl_ag_block():
            dist.all_gather_into_tensor(gathered_q.view(torch.uint8), qx.view(torch.uint8))
            dist.all_gather_into_tensor(gathered_s, sx)
            return txr.gemm.matmul_fp8_block(gathered_q, gathered_s, qw13, sw13)

        def nccl_block_rs():
            full = txr.gemm.matmul_fp8_block(qact, sact, qw2, sw2)
            dist.reduce_scatter_tensor(red, full)
            return red

        fused_ag = txr.gemm.all_gather_matmul_fp8_block(comm, qx, sx, stage_q, stage_s, qw13, sw13)
        two_step_ag = nccl_ag_block()
        fused_rs = txr.gemm.matmul_reduce_scatter_fp8_block(comm, qact, sact, qw2, sw2, stage_c)
        two_step_rs = nccl_block_rs().clone()
        torch.cuda.synchronize()
        out["fp8_block"] = {
            "ag_gemm_identical_to_two_step": bool(torch.equal(fused_ag, two_step_ag)),
            "gemm_rs_max_diff_vs_two_step": (fused_rs.float() - two_step_rs.float()).abs().max().item(),
            "status": comm.device_status(),
            "ag_gemm_us": timed(lambda: txr.gemm.all_gather_matmul_fp8_block(comm, qx, sx, stage_q, stage_s, qw13, sw13), args.iters, 3, world),
            "nccl_ag_then_gemm_us": timed(nccl_ag_block, args.iters, 3, world),
            "gemm_only_us": timed(lambda: txr.gemm.matmul_fp8_block(gathered_q, gathered_s, qw13, sw13), args.iters, 3, world),
            "gemm_rs_us": timed(lambda: txr.gemm.matmul_reduce_scatter_fp8_block(comm, qact, sact, qw2, sw2, stage_c), args.iters, 3, world),
            "gemm_then_nccl_rs_us": timed(nccl_block_rs, args.iters, 3, world),
            "rs_gemm_only_us": timed(lambda: txr.gemm.matmul_fp8_block(qact, sact, qw2, sw2), args.iters, 3, world),
        }
        out["fp8_block"]["ag_gemm_tflops"] = fl_ag / out["fp8_block"]["ag_gemm_us"] / 1e6
        out["fp8_block"]["gemm_rs_tflops"] = fl_rs / out["fp8_block"]["gemm_rs_us"] / 1e6
    if rank == 0:
        print(json.dumps(out))
    comm.destroy()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
