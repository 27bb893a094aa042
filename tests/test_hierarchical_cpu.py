"""Two-level collectives between real processes on the CPU: 4 (and 6) gloo ranks cut into nodes of 2 (and 3), host-memory
communicators of this library inside a node, gloo between nodes, every collective compared with torch.distributed on the
whole world."""
import os
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import free_port


def _worker(rank, world, local, port, q):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from tilexr_b200.parallel.hierarchical import HierarchicalComm

        h = HierarchicalComm.from_torch_distributed(local_world_size=local, buffer_mb=16, host_memory=True)
        assert (h.rank, h.world_size, h.local_size, h.nodes) == (rank, world, local, world // local)
        g = torch.Generator().manual_seed(100 + rank)
        n = 24 * world
        for it in range(2):                                          # a second round reuses windows and groups
            x = torch.randn(n, generator=g)
            want = x.clone()
            dist.all_reduce(want)
            assert torch.allclose(h.all_reduce(x), want, rtol=1e-5, atol=1e-5)
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            assert torch.equal(h.all_gather(x), torch.stack(parts))
            m = x.view(world, -1)
            total = torch.stack(parts).sum(0).view(world, -1)
            assert torch.allclose(h.reduce_scatter(m).reshape(-1), total[rank], rtol=1e-5, atol=1e-5)
            a2a = torch.empty_like(x)
            dist.all_to_all_single(a2a, x)
            assert torch.equal(h.all_to_all(x.view(world, -1)).reshape(-1), a2a)
            for root in (0, world - 1, (it + 1) % world):
                b = torch.randn(10, generator=g)
                ref = b.clone()
                dist.broadcast(ref, src=root)
                assert torch.equal(h.broadcast(b, root), ref)
        h.barrier()
        h.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("world,local", [(4, 2), (6, 3), (2, 2)])
def test_two_level_collectives_match_the_flat_ones(world, local):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, local, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, status in sorted(results):
        assert status == "ok", f"rank {rank}:\n{status}"
