"""Two-level expert parallelism between real processes on the CPU: gloo ranks cut into nodes, the hop between nodes on gloo,
the dispatch / combine inside a node on host-memory communicators of this library, compared with a dense mixture of experts
computed from every rank's inputs."""
import os
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import free_port


def _expert(e, rows):
    """A cheap expert that differs per expert and is not linear in the row."""
    return rows * (1.0 + 0.25 * e) + torch.tanh(rows) * (e % 3)


def _worker(rank, world, local, port, q):
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from tilexr_b200.parallel.hierarchical import HierarchicalComm
        from tilexr_b200.parallel.hierarchical_ep import HierarchicalEP, HostEpOps

        h = HierarchicalComm.from_torch_distributed(local_world_size=local, buffer_mb=16, host_memory=True)
        per_rank = 2
        E = per_rank * world
        ep = HierarchicalEP(h, E, HostEpOps())
        assert ep.per_node == per_rank * local
        with pytest.raises(ValueError):
            HierarchicalEP(h, E + 1, HostEpOps())
        g = torch.Generator().manual_seed(500 + rank)
        for it, (bs, K, H) in enumerate([(12, 3, 16), (7, 2, 16), (5, 4, 8)]):
            x = torch.randn(bs, H, generator=g)
            ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(bs)]).to(torch.int32)
            w = torch.rand(bs, K, generator=g)
            if it == 1:
                ids[0, 0] = -1                                          # an inactive route
                ids[:, 1] = (rank * per_rank) % E                       # every token also goes to an expert of this rank
            if it == 2:
                ids[:] = torch.arange(K, dtype=torch.int32)             # all routes of all ranks on node 0: the other nodes receive nothing
            d = ep.dispatch(x, ids)
            assert int(d.expert_token_nums.sum()) == d.recv_total
            # what arrived: every rank's routes to this rank's experts, sorted by local expert
            all_ids = [torch.empty_like(ids) for _ in range(world)]
            dist.all_gather(all_ids, ids)
            for le in range(per_rank):
                want = sum(int((a == rank * per_rank + le).sum()) for a in all_ids)
                assert int(d.expert_token_nums[le]) == want
            out = torch.zeros_like(d.expand_x)
            row = 0
            for le in range(per_rank):
                n = int(d.expert_token_nums[le])
                out[row:row + n] = _expert(rank * per_rank + le, d.expand_x[row:row + n])
                row += n
            y = ep.combine(out, d, w)
            ref = torch.zeros(bs, H)
            for k in range(K):
                for t in range(bs):
                    e = int(ids[t, k])
                    if e >= 0:
                        ref[t] += w[t, k] * _expert(e, x[t])
            assert torch.allclose(y, ref, rtol=1e-5, atol=1e-5), (it, (y - ref).abs().max())
            unweighted = ep.combine(out, d)
            ref1 = torch.zeros(bs, H)
            for k in range(K):
                for t in range(bs):
                    if int(ids[t, k]) >= 0:
                        ref1[t] += _expert(int(ids[t, k]), x[t])
            assert torch.allclose(unweighted, ref1, rtol=1e-5, atol=1e-5)
        h.barrier()
        h.destroy()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("world,local", [(4, 2), (6, 3), (2, 2)])
def test_two_level_dispatch_and_combine_match_a_dense_mixture(world, local):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, local, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, status in results:
        assert status == "ok", f"rank {rank}: {status}"


def test_device_adapter_calls_the_ep_ops_with_their_own_signature(monkeypatch):
    """`DeviceEpOps` cannot run without a GPU; its calls are bound against the real signatures of `ops.ep.dispatch` / `combine`
    and it must read fields that `DispatchResult` has."""
    import dataclasses
    import inspect

    from tilexr_b200.ops import ep
    from tilexr_b200.parallel.hierarchical_ep import DeviceEpOps

    real_dispatch, real_combine = inspect.signature(ep.dispatch), inspect.signature(ep.combine)
    seen = {}

    def fake_dispatch(*args, **kwargs):
        bound = real_dispatch.bind(*args, **kwargs)
        seen["dispatch"] = bound.arguments
        x, ids = bound.arguments["x"], bound.arguments["expert_ids"]
        rows = bound.arguments["max_recv_rows"]
        empty = torch.zeros(0)
        fields = {f.name: empty for f in dataclasses.fields(ep.DispatchResult)}
        fields.update(expand_x=torch.zeros(rows, x.shape[1]), expert_token_nums=torch.tensor([2, 1]), recv_total=torch.tensor([3], dtype=torch.int32),
                      topk_ids=ids, bs=x.shape[0], top_k=bound.arguments["top_k"], num_experts=bound.arguments["num_experts"], dedup=False,
                      shared_expert_num=0, shared_expert_rank_num=0, tp_world_size=1)
        return ep.DispatchResult(**fields)

    def fake_combine(*args, **kwargs):
        bound = real_combine.bind(*args, **kwargs)
        seen["combine"] = bound.arguments
        return torch.ones(bound.arguments["d"].bs, bound.arguments["expert_out"].shape[1])

    monkeypatch.setattr(ep, "dispatch", fake_dispatch)
    monkeypatch.setattr(ep, "combine", fake_combine)
    ops = DeviceEpOps()
    rows, ids = torch.randn(5, 8), torch.tensor([[0], [1], [3], [-1], [2]], dtype=torch.int32)
    h = ops.dispatch("comm", rows, ids, 4, 10)
    assert h.recv_total == 3 and h.expand_x.shape == (10, 8) and int(h.expert_token_nums.sum()) == 3
    d = seen["dispatch"]
    assert d["comm"] == "comm" and d["top_k"] == 1 and d["num_experts"] == 4 and d["max_recv_rows"] == 10 and d["dedup"] is False
    y = ops.combine("comm", torch.zeros(10, 8), h)
    assert y.shape == (5, 8)
    c = seen["combine"]
    assert c["d"] is h.state and c["expert_scales"].shape == (5, 1) and c["expert_scales"].dtype == torch.float32
