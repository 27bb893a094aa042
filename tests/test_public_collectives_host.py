"""The public tensor-level collectives (`txr.all_reduce`, ...) and the vLLM-facing forms with their `dim` semantics, on CPU
tensors between three gloo ranks over a host-memory communicator, against torch.distributed."""
import os
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import free_port


def _worker(rank, world, port, q):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import tilexr_b200 as txr
        from tilexr_b200.integrations import vllm_collectives as vc

        comm = txr.init_from_torch_distributed(host_memory=True, buffer_mb=16)
        g = torch.Generator().manual_seed(40 + rank)
        x = torch.randn(world * 4, 6, generator=g)
        every = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(every, x)
        total = every[0].clone()
        for e in every[1:]:
            total = total + e                                          # rank order, like the kernels
        # the plain ops
        assert torch.equal(txr.all_reduce(comm, x), total)
        assert torch.equal(txr.all_gather(comm, x), torch.stack(every))
        assert torch.equal(txr.reduce_scatter(comm, x), total[rank * 4:(rank + 1) * 4])
        a2a = torch.empty_like(x)
        dist.all_to_all_single(a2a, x)
        assert torch.equal(txr.all_to_all(comm, x), a2a)
        out = torch.empty_like(x)
        assert txr.all_reduce(comm, x, out=out) is out and torch.equal(out, total)
        b = x.clone()
        txr.broadcast(comm, b, root=1)
        assert torch.equal(b, every[1])
        ids = torch.arange(8, dtype=torch.int64) + 100 * rank            # bytes travel whatever the type
        assert torch.equal(txr.all_gather(comm, ids)[2], torch.arange(8) + 200)
        with pytest.raises(ValueError):
            txr.all_reduce(comm, x.to(torch.bfloat16))
        with pytest.raises(ValueError):
            txr.all_reduce(comm, x, op=txr.collectives.ReduceOp.MAX)
        # the vLLM-facing forms: pieces concatenated or scattered along `dim`
        y = torch.randn(2, world * 2, 5, generator=g)
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        ysum = ys[0].clone()
        for e in ys[1:]:
            ysum = ysum + e
        assert torch.equal(vc.all_reduce(comm, y), ysum)
        for dim in (0, 1, -1):
            assert torch.equal(vc.all_gather(comm, y, dim), torch.cat(ys, dim=dim))
        assert torch.equal(vc.reduce_scatter(comm, y, 1), ysum.chunk(world, dim=1)[rank])
        want = torch.cat([e.chunk(world, dim=1)[rank] for e in ys], dim=1)
        assert torch.equal(vc.all_to_all(comm, y, 1, 1), want)
        t = y.transpose(0, 2)                                          # not contiguous: broadcast goes through a staging copy
        ref = ys[0].transpose(0, 2)
        assert torch.equal(vc.broadcast(comm, t.clone(memory_format=torch.preserve_format), 0), ref)
        with pytest.raises(ValueError):
            vc.reduce_scatter(comm, torch.zeros(2, world * 2 + 1), 1)
        comm.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def test_public_ops_on_cpu_tensors_between_three_processes():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, status in results:
        assert status == "ok", f"rank {rank}: {status}"
