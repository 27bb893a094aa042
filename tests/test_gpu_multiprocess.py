"""One process per GPU over NVLink peer mappings (CUDA IPC), bootstrapped by the library's own
TCP exchange.  Needs at least two GPUs; on a one-GPU box the emulated-world tests cover the
same kernels."""
import os
import traceback

import pytest
import torch
import torch.multiprocessing as mp

from conftest import free_port

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    try:
        os.environ["TILEXR_WAIT_TIMEOUT_MS"] = "5000"
        torch.cuda.set_device(rank)
        import tilexr_b200 as txr
        from tilexr_b200.ops import ep
        from tilexr_b200.utils import oracle

        comm = txr.init_process(rank, world, comm_id=f"127.0.0.1:{port}", buffer_mb=128, device=rank)
        info = comm.physical_info()
        assert info["link"] == "nvlink" and info["p2p_native_atomics"] and info["compute_capability"] == (10, 0) and info["sm_count"] == 148
        assert info["nvls_bound"] == comm.nvls_available()
        gens = [torch.Generator().manual_seed(100 + r) for r in range(world)]
        xs = [torch.randn(1 << 18, generator=g).to(torch.bfloat16) for g in gens]
        mine = xs[rank].cuda()
        for _ in range(3):
            ag = txr.all_gather(comm, mine)
            ar = txr.all_reduce(comm, mine)
            a2a = txr.all_to_all(comm, mine)
            rs = txr.reduce_scatter(comm, mine)
        sym = comm.symm_empty([world, 1 << 18], torch.bfloat16)
        txr.all_gather(comm, mine, out=sym)
        b = mine.clone()
        txr.broadcast(comm, b, root=world - 1)
        torch.cuda.synchronize()
        assert comm.device_status() == 0
        assert torch.equal(ag.cpu().reshape(-1), oracle.all_gather_ref(xs))
        assert torch.equal(sym.cpu().reshape(-1), oracle.all_gather_ref(xs))
        full = oracle.all_reduce_ref(xs)
        n = (1 << 18) // world
        if comm.nvls_available():
            # sums of this size are formed inside the switch: fp32 accumulation in an order of its own, one
            # rounding; every rank holds the same bits
            assert torch.allclose(ar.cpu().float(), full.float(), rtol=2 ** -7, atol=1e-6)
            assert torch.allclose(rs.cpu().float(), full[rank * n:(rank + 1) * n].float(), rtol=2 ** -7, atol=1e-6)
            gathered = txr.all_gather(comm, ar)
            torch.cuda.synchronize()
            assert all(torch.equal(gathered[r], ar) for r in range(world))
        else:
            assert torch.equal(ar.cpu(), full)
            assert torch.equal(rs.cpu(), full[rank * n:(rank + 1) * n])
        assert torch.equal(a2a.cpu(), oracle.all_to_all_ref(xs)[rank])
        assert torch.equal(b.cpu(), xs[world - 1])
        # the same operations below and above the sizes at which the in-switch kernels take over, and the
        # two-shot all-reduce (16 MiB), against the oracle
        for numel in (1 << 10, 1 << 23):
            ys = [torch.randn(numel, generator=g).to(torch.bfloat16) for g in gens]
            y = ys[rank].cuda()
            got_ar = txr.all_reduce(comm, y)
            got_ag = txr.all_gather(comm, y)
            got_rs = txr.reduce_scatter(comm, y)
            bb = y.clone()
            txr.broadcast(comm, bb, root=0)
            torch.cuda.synchronize()
            assert comm.device_status() == 0
            want = oracle.all_reduce_ref(ys)
            assert torch.allclose(got_ar.cpu().float(), want.float(), rtol=2 ** -7, atol=1e-6)
            assert torch.equal(got_ag.cpu().reshape(-1), oracle.all_gather_ref(ys))
            m = numel // world
            assert torch.allclose(got_rs.cpu().float(), want[rank * m:(rank + 1) * m].float(), rtol=2 ** -7, atol=1e-6)
            assert torch.equal(bb.cpu(), ys[0])
        # a back-to-back pair of zero-copy all-gathers into one registered output with a long reader in between on
        # the last rank: the second gather must not overwrite what the reader still reads
        first, second = xs[rank].cuda(), (xs[rank].float() + 1).to(torch.bfloat16).cuda()
        txr.all_gather(comm, first, out=sym)
        if rank == world - 1:
            torch.cuda._sleep(200_000_000)                     # about a tenth of a second of device time
        snapshot = sym.clone()
        txr.all_gather(comm, second, out=sym)
        torch.cuda.synchronize()
        assert comm.device_status() == 0
        assert torch.equal(snapshot.cpu().reshape(-1), oracle.all_gather_ref(xs))

        bs, h, E, K = 64, 1024, 8 * world, 4
        tok = [torch.randn(bs, h, generator=g).to(torch.bfloat16) for g in gens]
        logits = [torch.randn(bs, E, generator=g) for g in gens]
        routed = [oracle.routing_topk_ref(l, K, 1, True) for l in logits]
        d = ep.dispatch(comm, tok[rank].cuda(), gate_logits=logits[rank].cuda(), num_experts=E, top_k=K,
                        quant_mode=ep.QUANT_FP8_1X128, score_func=1)
        rows = txr.quant.fp8_dequant_1x128(d.expand_x, d.dynamic_scales, torch.bfloat16)
        y = ep.combine(comm, rows, d, expert_scales=d.topk_weights)
        torch.cuda.synchronize()
        assert comm.device_status() == 0
        ref = oracle.ep_dispatch_ref(tok, [r[0] for r in routed], E)[rank]
        cnt = int(d.recv_total.item())
        assert cnt == len(ref["rows"])
        assert torch.equal(d.assist[:cnt].cpu(), ref["assist"])
        # identity expert: y = sum_k w_k * bf16(dequant(quant(x))), weights renormalised to one
        rq, rs_ = oracle.fp8_quant_1x128_ref(tok[rank])
        deq = oracle.fp8_dequant_1x128_ref(rq, rs_).to(torch.bfloat16).float()
        want_y = deq * routed[rank][1].sum(dim=1, keepdim=True)
        assert torch.allclose(y.cpu().float(), want_y, rtol=2e-2, atol=2e-2), (y.cpu().float() - want_y).abs().max()
        src_rows = torch.stack([tok[int(s)][int(t)] for s, t, _, _ in ref["assist"].tolist()])
        wq, ws_ = oracle.fp8_quant_1x128_ref(src_rows)
        assert torch.equal(d.expand_x[:cnt].cpu().view(torch.uint8), wq.view(torch.uint8))
        assert torch.equal(d.dynamic_scales[:cnt].cpu(), ws_)
        # The same step captured in a CUDA graph and replayed on fresh inputs: launches carry no per-call host
        # state (epochs live on the device), so every replay is a new launch for the flag protocol.
        x_static = tok[rank].cuda()
        lg_static = logits[rank].cuda()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            def graph_step():
                dd = ep.dispatch(comm, x_static, gate_logits=lg_static, num_experts=E, top_k=K,
                                 quant_mode=ep.QUANT_FP8_1X128, score_func=1)
                rr = txr.quant.fp8_dequant_1x128(dd.expand_x, dd.dynamic_scales, torch.bfloat16)
                return ep.combine(comm, rr, dd, expert_scales=dd.topk_weights), txr.all_reduce(comm, x_static)
            graph_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y_static, ar_static = graph_step()
        for it in range(3):
            fresh = [torch.randn(bs, h, generator=gg).to(torch.bfloat16) for gg in gens]
            x_static.copy_(fresh[rank])
            g.replay()
            torch.cuda.synchronize()
            assert comm.device_status() == 0
            assert (y_static.cpu().float() - fresh[rank].float()).abs().max().item() < 0.35
            assert torch.allclose(ar_static.cpu().float(), oracle.all_reduce_ref(fresh).float(), rtol=2 ** -7, atol=1e-6)
        eager = txr.all_reduce(comm, x_static)          # eager launches keep working after replays
        torch.cuda.synchronize()
        assert torch.equal(eager.cpu(), ar_static.cpu())
        comm.destroy()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def test_process_per_gpu_collectives_and_ep():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = min(torch.cuda.device_count(), 4)
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
        assert status == "ok", f"rank {rank}:\n{status}"
