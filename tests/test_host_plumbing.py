"""CPU / gloo world_size=2 plumbing: tile-flag all-gather and expert-parallel dispatch + combine
between two real processes over host-memory windows.

Shapes follow the no-GPU configuration of the benchmark plan: 128 tokens x hidden 1024 fp32 per
rank, 8 experts (4 per rank), softmax top-2 with renormalised weights; all-gather of 4 MiB per
rank in 64 KiB tiles, each tile guarded by its own magic-tagged flag.
"""
import os
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import free_port


def _worker(rank, world, port, scenario, result_queue):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import tilexr_b200 as txr
        from tilexr_b200.utils import oracle

        comm = txr.init_from_torch_distributed(host_memory=True, buffer_mb=64)
        assert comm.rank == rank and comm.world_size == world
        g = torch.Generator().manual_seed(1234 + rank)
        if scenario == "allgather":
            x = torch.randn(1 << 20, generator=g)            # 4 MiB fp32
            out = torch.empty(world * x.numel())
            for _ in range(3):                                # epochs 1..3 exercise both halves and the reuse guard
                txr._C.host_all_gather(comm, x, out, 64 * 1024)
            gathered = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(gathered, x)
            assert torch.equal(out, torch.cat(gathered))
            red = txr._C.host_all_reduce(comm, x[:4096].contiguous())
            ref = x[:4096].clone()
            dist.all_reduce(ref)
            assert torch.allclose(red, ref, atol=1e-6)
        elif scenario == "ep":
            bs, h, E, K = 128, 1024, 8, 2
            x = torch.randn(bs, h, generator=g)
            logits = torch.randn(bs, E, generator=g)
            ids, w = oracle.routing_topk_ref(logits, K, score_func=0, renormalize=True)
            xs = [torch.empty_like(x) for _ in range(world)]
            idl = [torch.empty_like(ids) for _ in range(world)]
            wl = [torch.empty_like(w) for _ in range(world)]
            dist.all_gather(xs, x)
            dist.all_gather(idl, ids)
            dist.all_gather(wl, w)
            ref = oracle.ep_dispatch_ref(xs, idl, E)
            for it in range(2):
                expand, assist, nums, counts, total = txr._C.host_ep_dispatch(comm, x, ids, E, bs * world * K)
                mine = ref[rank]
                assert total == len(mine["rows"])
                assert torch.equal(expand[:total], mine["expand_x"])
                assert torch.equal(assist[:total], mine["assist"])
                assert torch.equal(nums, mine["token_nums"])
                assert torch.equal(counts, mine["send_counts"])
                expert_out = expand[:total] * 2.0 + 1.0        # a stand-in expert
                y = txr._C.host_ep_combine(comm, expert_out.contiguous(), assist, total, ids, w, E)
                yref = torch.zeros_like(x)
                for t in range(bs):
                    for k in range(K):
                        yref[t] += w[t, k] * (x[t] * 2.0 + 1.0)
                assert torch.allclose(y, yref, rtol=1e-5, atol=1e-5), (y - yref).abs().max()
        elif scenario == "lost_flag":
            # rank 1 never raises its flags: rank 0 must give up within the budget and say why
            x = torch.ones(4096)
            out = torch.empty(world * 4096)
            comm.set_wait_timeout_ms(300)
            if rank == 1:
                txr._C.host_inject_skip_flags(True)
                txr._C.host_all_gather(comm, x, out, 4096)
                assert comm.device_status() == 0
            else:
                with pytest.raises(RuntimeError):
                    txr._C.host_all_gather(comm, x, out, 4096)
                assert comm.device_status() == 1             # TILEXR_DEV_WAIT_TIMEOUT
                d = comm.dfx()
                assert d[3] == 0xDEAD and d[5] == 1           # failed, waiting for peer 1
        dist.barrier()
        comm.destroy()
        dist.destroy_process_group()
        result_queue.put((rank, "ok"))
    except Exception:
        result_queue.put((rank, traceback.format_exc()))


def _run(scenario, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, status in results:
        assert status == "ok", f"rank {rank}:\n{status}"


def test_tile_flag_all_gather_two_ranks():
    _run("allgather")


def test_ep_dispatch_combine_two_ranks():
    _run("ep")


def test_lost_flag_is_detected_on_the_host():
    _run("lost_flag")
