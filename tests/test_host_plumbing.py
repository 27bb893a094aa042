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
        assert comm.physical_info()["link"] == "host_memory" and not comm.physical_info()["nvls_bound"]
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
        elif scenario == "collectives":
            # all-to-all, reduce-scatter and broadcast over the same tiles and flags, several launches each (both halves,
            # the reuse guard), against torch.distributed on the same data
            for it in range(3):
                n = 3 * 4096 + 7                                      # not a whole number of tiles
                x = torch.randn(world * n, generator=g)
                got = txr._C.host_all_to_all(comm, x, 4096)
                want = torch.empty_like(x)
                dist.all_to_all_single(want, x)
                assert torch.equal(got, want)
                red = txr._C.host_reduce_scatter(comm, x)
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x)
                acc = parts[0][rank * n:(rank + 1) * n].clone()
                for p in parts[1:]:
                    acc = acc + p[rank * n:(rank + 1) * n]           # rank order, like the kernel
                assert torch.equal(red, acc)
                root = it % world
                b = torch.randn(n, generator=g)
                ref = b.clone()
                dist.broadcast(ref, src=root)
                txr._C.host_broadcast(comm, b, root, 4096)
                assert torch.equal(b, ref)
            with pytest.raises(RuntimeError):
                txr._C.host_broadcast(comm, torch.zeros(8), world, 4096)      # a root outside the communicator
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
        elif scenario in ("traced", "traced_lost_flag"):
            # the production flag primitives and host kernels, recorded while they run between two processes, judged
            # by the protocol checker
            from tilexr_b200.tools import checker
            trace_dir = os.environ["TILEXR_TEST_TRACE_DIR"]
            path = os.path.join(trace_dir, f"rank{rank}.jsonl")
            if scenario == "traced":
                bs, h, E, K = 16, 64, 4, 2
                x = torch.randn(bs, h, generator=g)
                ids, w = oracle.routing_topk_ref(torch.randn(bs, E, generator=g), K, score_func=0, renormalize=True)
                big = torch.randn(3 * 4096, generator=g)
                out = torch.empty(world * big.numel())
                with checker.record_host_trace(comm, path):
                    for _ in range(3):                        # both data halves and the reuse guard
                        txr._C.host_all_gather(comm, big, out, 16384)
                    txr._C.host_all_reduce(comm, big[:1024].contiguous())
                    expand, assist, nums, counts, total = txr._C.host_ep_dispatch(comm, x, ids, E, bs * world * K)
                    txr._C.host_ep_combine(comm, expand[:total].contiguous(), assist, total, ids, w, E)
            else:
                comm.set_wait_timeout_ms(300)
                x = torch.ones(4096)
                out = torch.empty(world * 4096)
                with checker.record_host_trace(comm, path):
                    if rank == 1:
                        txr._C.host_inject_skip_flags(True)
                        txr._C.host_all_gather(comm, x, out, 4096)
                    else:
                        with pytest.raises(RuntimeError):
                            txr._C.host_all_gather(comm, x, out, 4096)
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
                # the dump-on-failure record says the same, in a file
                import json
                import tempfile

                from tilexr_b200.utils import failure_dump
                with tempfile.TemporaryDirectory() as tmp:
                    os.environ["TILEXR_DUMP_DIR"] = tmp
                    try:
                        with pytest.raises(RuntimeError, match="device status 1"):
                            failure_dump.check(comm, "lost-flag all-gather", {"bytes": 4096 * 4})
                    finally:
                        os.environ.pop("TILEXR_DUMP_DIR")
                    rec = json.load(open(os.path.join(tmp, os.listdir(tmp)[0])))
                    assert rec["dfx"]["run_status_name"] == "failed" and rec["dfx"]["fail_peer"] == 1 and rec["device_status"] == 1
                    assert rec["context"]["what"] == "lost-flag all-gather" and rec["physical_info"]["link"] == "host_memory"
        dist.barrier()
        comm.destroy()
        dist.destroy_process_group()
        result_queue.put((rank, "ok"))
    except Exception:
        result_queue.put((rank, traceback.format_exc()))


def _traced(scenario, tmp_path, world=2):
    os.environ["TILEXR_TEST_TRACE_DIR"] = str(tmp_path)
    try:
        _run(scenario, world)
    finally:
        os.environ.pop("TILEXR_TEST_TRACE_DIR", None)
    return [str(tmp_path / f"rank{r}.jsonl") for r in range(world)]


def test_production_protocol_trace_passes_the_checker(tmp_path):
    from tilexr_b200.tools import checker
    paths = _traced("traced", tmp_path)
    text = "".join(open(p).read() for p in paths)
    kinds = [line.split('"kind": "')[1].split('"')[0] for line in text.splitlines()]
    assert kinds.count("FlagStore") > 20 and kinds.count("FlagWait") > 20 and kinds.count("Copy") > 10 and kinds.count("Read") > 10
    assert checker.check_trace_files(paths) == []
    # the same run with rank 1's flag stores taken out of the record: the checker must miss them ...
    lines = text.splitlines(keepends=True)
    dropped = [l for l in lines if not ('"kind": "FlagStore"' in l and '"rank": 1,' in l)]
    names = {f[0] for f in checker.check_trace("".join(dropped))}
    assert "FLAG_NO_PRODUCER" in names
    # ... and with rank 0's waits taken out, its reads of rank 1's data are no longer ordered after the copies
    unwaited = [l for l in lines if not ('"kind": "FlagWait"' in l and '"rank": 0,' in l)]
    names = {f[0] for f in checker.check_trace("".join(unwaited))}
    assert "READ_BEFORE_COPY" in names


def test_production_run_with_a_lost_flag_is_reported_by_the_checker(tmp_path):
    from tilexr_b200.tools import checker
    paths = _traced("traced_lost_flag", tmp_path)
    findings = checker.check_trace_files(paths)
    assert any(f[0] == "FLAG_NO_PRODUCER" and f[1] == 0 for f in findings), findings


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


@pytest.mark.parametrize("world", [2, 3])
def test_all_to_all_reduce_scatter_broadcast(world):
    _run("collectives", world)


def test_lost_flag_is_detected_on_the_host():
    _run("lost_flag")
