"""Smoke run of the vLLM-facing collectives: every operation once through ``TileXRVllmCollectivesAdapter`` with values that
make a wrong rank, order or count visible, checked on every rank (the reference's integrations/vllm_ascend/smoke_collectives.py).

    VLLM_TILEXR_COLLECTIVES=1 python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m tilexr_b200.tools.vllm_collectives_smoke --count 4096 --dtype bfloat16

Values: rank r contributes ``r + 1 + (i % 7)`` at element i, so sums, concatenations and exchanges have closed forms.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "int32": torch.int32}


def make_values(rank: int, count: int, dtype, device="cpu") -> torch.Tensor:
    return ((torch.arange(count, device=device) % 7) + rank + 1).to(dtype)


def expected_all_reduce(world: int, count: int, dtype) -> torch.Tensor:
    base = (torch.arange(count) % 7).to(torch.float64)
    return (base * world + world * (world + 1) / 2).to(dtype)


def expected_all_gather(world: int, count: int, dtype) -> torch.Tensor:
    return torch.cat([make_values(r, count, dtype) for r in range(world)])


def expected_reduce_scatter(world: int, rank: int, count: int, dtype) -> torch.Tensor:
    """Input of ``count * world`` elements per rank; rank r keeps chunk r of the sum."""
    full = expected_all_reduce(world, count * world, dtype)
    return full[rank * count:(rank + 1) * count]


def expected_all_to_all(world: int, rank: int, count: int, dtype) -> torch.Tensor:
    """Input of ``count * world`` elements per rank; chunk p goes to rank p, so rank r ends with chunk r of every rank."""
    return torch.cat([make_values(src, count * world, dtype)[rank * count:(rank + 1) * count] for src in range(world)])


def expected_broadcast(root: int, count: int, dtype) -> torch.Tensor:
    return make_values(root, count, dtype)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--count", type=int, default=4096)
    p.add_argument("--dtype", default="bfloat16", choices=sorted(DTYPES))
    p.add_argument("--root", type=int, default=0)
    args = p.parse_args()
    import torch.distributed as dist

    import tilexr_b200 as txr
    from tilexr_b200.integrations import vllm_collectives as vc

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if not dist.is_initialized():
        dist.init_process_group("nccl")
    comm = txr.init_from_torch_distributed(buffer_mb=64)
    adapter = vc.TileXRVllmCollectivesAdapter(comm)
    dtype, n, dev = DTYPES[args.dtype], args.count, "cuda"
    results = {}

    def check(name, got, want):
        if got is None:
            results[name] = f"fallback ({adapter.last_error!r})" if adapter.last_error is not None else "fallback"
            return
        torch.cuda.synchronize()
        results[name] = "ok" if torch.equal(got.cpu(), want) else "MISMATCH"

    check("all_reduce", adapter.all_reduce(make_values(rank, n, dtype, dev)), expected_all_reduce(world, n, dtype))
    check("all_gather", adapter.all_gather(make_values(rank, n, dtype, dev), 0), expected_all_gather(world, n, dtype))
    check("reduce_scatter", adapter.reduce_scatter(make_values(rank, n * world, dtype, dev), 0), expected_reduce_scatter(world, rank, n, dtype))
    check("all_to_all", adapter.all_to_all(make_values(rank, n * world, dtype, dev), 0, 0), expected_all_to_all(world, rank, n, dtype))
    check("broadcast", adapter.broadcast(make_values(rank, n, dtype, dev), args.root % world), expected_broadcast(args.root % world, n, dtype))
    status = comm.device_status()
    bad = [k for k, v in results.items() if v != "ok"] if vc.enabled() else [k for k, v in results.items() if v == "MISMATCH"]
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "results": results, "device_status": status})
    if rank == 0:
        print(json.dumps({"world": world, "count": n, "dtype": args.dtype, "gate": vc.enabled(), "ranks": gathered}))
    comm.destroy()
    dist.destroy_process_group()
    if bad or status != 0:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
