"""Decode-time all-reduce + residual add + RMSNorm: the fused kernel (one-shot / two-shot) against
NCCL all_reduce followed by torch ops, bf16 [batch, hidden], batch 1..256 and beyond.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29557 \
        -m tilexr_b200.tools.ar_norm_perf --hidden 8192 --batches 1,4,16,64,256,1024,4096
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


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--hidden", type=int, default=8192)
    p.add_argument("--batches", default="1,4,16,64,256,1024,4096,16384")
    p.add_argument("--iters", type=int, default=30)
    args = p.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29557")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    import tilexr_b200 as txr
    from tilexr_b200.ops import collectives as coll

    comm = txr.init_from_torch_distributed(buffer_mb=1024)
    H = args.hidden
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    gamma = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    dist.broadcast(gamma, 0)
    rows = []
    for b in [int(v) for v in args.batches.split(",")]:
        x = torch.randn(b, H, device="cuda", generator=g).to(torch.bfloat16)
        res0 = torch.randn(b, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)).to(torch.bfloat16)
        res = res0.clone()
        ref_res = res0.clone()

        def nccl():
            y = x.clone()
            dist.all_reduce(y)
            s = y + ref_res
            return torch.nn.functional.rms_norm(s.float(), (H,), gamma.float(), 1e-6).to(torch.bfloat16), s

        entry = {"batch": b, "bytes": b * H * 2}
        y_ref, s_ref = nccl()
        for name, algo in (("one_shot", coll.AR_ONE_SHOT), ("two_shot", coll.AR_TWO_SHOT)):
            if algo == coll.AR_ONE_SHOT and b * H * 2 > (8 << 20):
                continue
            res.copy_(res0)
            y = coll.all_reduce_rmsnorm(comm, x, gamma, 1e-6, residual=res, algo=algo)
            torch.cuda.synchronize()
            entry[name + "_max_diff"] = (y.float() - y_ref.float()).abs().max().item()
            entry[name + "_us"] = timed(lambda: coll.all_reduce_rmsnorm(comm, x, gamma, 1e-6, residual=res, algo=algo), args.iters, 5)
        entry["auto_choice"] = txr._C.all_reduce_rmsnorm_choose(b * H * 2, world)
        entry["nccl_us"] = timed(nccl, args.iters, 5)
        entry["status"] = comm.device_status()
        rows.append(entry)
        if rank == 0:
            print(json.dumps(entry), flush=True)
    comm.destroy()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
