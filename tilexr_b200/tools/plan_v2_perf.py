"""Device time of the MoonEP planners on an emulated world (R ranks on one GPU, one cooperative launch per call):
the topology-aware V2 planner against the V3 balance planner, and the V2 plan's quality figures.

    python -m tilexr_b200.tools.plan_v2_perf --ranks 8 --tokens 512 --topk 8 --experts 256 --slots 32 --skew 0.3
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch


def routing(R, S, K, E, seed, skew):
    g = np.random.default_rng(seed)
    p = np.full(E, (1.0 - skew) / E)
    p[: E // R] += skew / (E // R)          # the experts of rank 0 are hot
    p = p / p.sum()
    topk = np.stack([np.stack([g.choice(E, size=K, replace=False, p=p) for _ in range(S)]) for _ in range(R)]).astype(np.int32)
    tpe = np.stack([np.bincount(topk[r].reshape(-1), minlength=E) for r in range(R)]).astype(np.int32)
    return topk, tpe


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / iters


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--ranks", type=int, default=8)
    p.add_argument("--tokens", type=int, default=512)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--experts", type=int, default=256)
    p.add_argument("--slots", type=int, default=32)
    p.add_argument("--padding", type=int, default=16)
    p.add_argument("--skew", type=float, default=0.3)
    args = p.parse_args()
    import tilexr_b200 as txr
    from tilexr_b200 import _C

    R, S, K, E, B = args.ranks, args.tokens, args.topk, args.experts, args.slots
    topk, tpe = routing(R, S, K, E, 1, args.skew)
    nvs = 2 * S * K + (E + B) * args.padding
    world = txr.init_emulated_world(R, device=0, buffer_mb=64)
    dev_topk = [torch.from_numpy(topk[r]).cuda() for r in range(R)]
    dev_tpe = torch.from_numpy(tpe).cuda()
    gids = torch.arange(R, dtype=torch.int32).cuda()
    plans = world.run(lambda c, r: _C.moonep_plan_v2(c, dev_topk[r], dev_tpe, gids, B, nvs, args.padding, 0))
    world.check()
    status = plans[0]["status"].cpu().tolist()
    v2_us = timed(lambda: world.run(lambda c, r: _C.moonep_plan_v2(c, dev_topk[r], dev_tpe, gids, B, nvs, args.padding, 0)))
    torch.cuda.synchronize()
    phases = [v / 1e3 for v in world[0].dfx()[16:21]]      # rank 0's last launch: mail, validate + set-up, balance, routes, consensus (us)
    v3_us = timed(lambda: world.run(lambda c, r: _C.moonep_planning(c, dev_topk[r], E, B, args.padding)))
    world.check()
    loads_before = tpe.sum(0).reshape(R, E // R).sum(1)
    dup = int(sum((pl["dst"] < 0).sum().item() for pl in plans))
    print(json.dumps({"ranks": R, "tokens_per_rank": S, "top_k": K, "experts": E, "slots": B, "skew": args.skew,
                      "plan_v2_us": v2_us, "plan_v3_us": v3_us, "status": status,
                      "plan_v2_phases_us": dict(zip(("mail", "validate_setup", "balance", "routes", "consensus"), phases)),
                      "plan_v2_kernel_us": sum(phases),      # rank 0's block, first to last phase; plan_v2_us also holds the host's work for R ranks
                      "load_before_max_over_cap": float(loads_before.max()) / (S * K),
                      "deficit_after": status[3], "intra_rounds": status[1], "inter_rounds": status[2], "expert_moves": status[6],
                      "max_remote_experts": status[4], "duplicate_routes": dup, "routes": R * S * K,
                      "note": "R ranks share one GPU: every rank's planner block runs on the same device"}))
    world.destroy()


if __name__ == "__main__":
    main()
