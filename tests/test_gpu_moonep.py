"""MoonEP stages on emulated worlds: planner kernel vs the CPU plan, dispatch/combine round trip,
weight prefetch and owner-pull gradient reduction."""
import pytest
import torch

from conftest import require_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def txr():
    require_cuda()
    import tilexr_b200

    return tilexr_b200


def _topk(r, s, k, e, seed, skew=True):
    g = torch.Generator().manual_seed(seed)
    p = torch.ones(e)
    if skew:
        p[: max(1, e // 8)] = 10.0
    return [torch.multinomial(p, s * k, replacement=True, generator=g).to(torch.int32).view(s, k) for _ in range(r)]


@pytest.mark.parametrize("r,s,k,e,b,pad", [(2, 32, 2, 8, 4, 1), (4, 64, 4, 32, 8, 16), (8, 48, 8, 64, 8, 8)])
def test_planner_matches_cpu_plan_and_stages_round_trip(txr, r, s, k, e, b, pad):
    C = txr._C
    world = txr.init_emulated_world(r, device=0, buffer_mb=64)
    topk = _topk(r, s, k, e, 3)
    all_topk = torch.stack([t.reshape(-1) for t in topk])
    topk_dev = [t.cuda() for t in topk]
    for _ in range(2):
        plans = world.run(lambda c, rank: C.moonep_planning(c, topk_dev[rank], e, b, pad))
        world.check()
    nvs = plans[0]["NvS"]
    n = s * k
    for rank in range(r):
        ref = C.moonep_reference_plan(all_topk, rank, s, k, e, b, pad)
        p = plans[rank]
        assert int(p["status"].item()) == 0
        for key in ("dst", "cu_seqlens", "experts_to_copy", "zero_fill_ranges", "remote_stats"):
            assert torch.equal(p[key].cpu(), ref[key]), key
    # dst_local is the inverse of dst
    for rank in range(r):
        dl = plans[rank]["dst_local"].cpu()
        filled = 0
        for src in range(r):
            dst = plans[src]["dst"].cpu()
            for i, raw in enumerate(dst.tolist()):
                if raw // nvs == rank:
                    assert int(dl[raw % nvs]) == src * n + i
                    filled += 1
        assert int((dl >= 0).sum()) == filled

    # dispatch -> identity expert -> combine returns K * hidden; weights come back bit-exact
    h = 256
    g = torch.Generator().manual_seed(5)
    hidden = [torch.randn(s, h, generator=g).to(torch.bfloat16).cuda() for _ in range(r)]
    weights = [torch.rand(s, k, generator=g).cuda() for _ in range(r)]
    for symmetric in (False, True):
        if symmetric:
            rows = world.symm_empty((nvs, h), torch.bfloat16)
            wrow = world.symm_empty((nvs,), torch.float32)
        else:
            rows = [torch.empty(nvs, h, dtype=torch.bfloat16, device="cuda") for _ in range(r)]
            wrow = [torch.empty(nvs, dtype=torch.float32, device="cuda") for _ in range(r)]
        for x in rows:
            x.fill_(7.0)
        world.run(lambda c, rank: C.moonep_dispatch(c, plans[rank], hidden[rank], weights[rank], rows[rank], wrow[rank]))
        world.check()
        for rank in range(r):
            dl = plans[rank]["dst_local"].cpu()
            got = rows[rank].cpu()
            for slot in range(nvs):
                v = int(dl[slot])
                if v < 0:
                    assert torch.all(got[slot] == 0), "padding rows are cleared"
                else:
                    src, route = divmod(v, n)
                    assert torch.equal(got[slot], hidden[src].cpu()[route // k])
                    assert float(wrow[rank][slot]) == float(weights[src].reshape(-1)[route])
        outs = [torch.empty(s, h, dtype=torch.bfloat16, device="cuda") for _ in range(r)]
        wout = [torch.empty(s, k, dtype=torch.float32, device="cuda") for _ in range(r)]
        world.run(lambda c, rank: C.moonep_combine(c, plans[rank], rows[rank], wrow[rank], outs[rank], wout[rank]))
        world.check()
        for rank in range(r):
            want = (hidden[rank].float() * k).to(torch.bfloat16)
            assert torch.allclose(outs[rank].float(), want.float(), rtol=1e-2, atol=1e-2)
            assert torch.equal(wout[rank], weights[rank])

    # prefetch: slot rows receive the owner's rows; reduce-grad: owners add the slot rows back
    L = e // r
    gate = world.symm_empty((L + b, 64), torch.bfloat16)
    up = world.symm_empty((L + b, 32), torch.bfloat16)
    for rank in range(r):
        gate[rank].copy_((torch.arange((L + b) * 64).view(L + b, 64) % 97 + 1000 * rank).to(torch.bfloat16))
        up[rank].copy_((torch.arange((L + b) * 32).view(L + b, 32) % 31 + 10 * rank).to(torch.bfloat16))
    before = [t.clone() for t in gate]
    world.run(lambda c, rank: C.moonep_prefetch_weight(c, plans[rank], gate[rank], up[rank], None))
    world.check()
    etc = plans[0]["experts_to_copy"].cpu()
    for rank in range(r):
        for slot in range(b):
            ex = int(etc[rank, slot])
            if ex >= 0:
                assert torch.equal(gate[rank][L + slot], before[ex // L][ex % L])
    grads = world.symm_empty((L + b, 48), torch.float32)
    for rank in range(r):
        grads[rank].copy_(torch.randn(L + b, 48, generator=g))
    snap = [t.clone() for t in grads]
    world.run(lambda c, rank: C.moonep_reduce_grad(c, plans[rank], grads[rank], None, None))
    world.check()
    for rank in range(r):
        want = snap[rank][:L].clone()
        for src in range(r):
            for slot in range(b):
                ex = int(etc[src, slot])
                if ex >= 0 and ex // L == rank and src != rank:
                    want[ex % L] += snap[src][L + slot]
        assert torch.equal(grads[rank][:L], want)
        assert torch.all(grads[rank][L:] == 0)
    world.destroy()


def test_buffer_facade_single_rank(txr, port):
    from tilexr_b200.integrations.moonep import Buffer

    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{port}", buffer_mb=64, device=0)
    S, H, K, E = 32, 128, 2, 8
    buf = Buffer(S, H, K, E, 1, token_padding=4, comm=comm)
    g = torch.Generator().manual_seed(1)
    hidden = torch.randn(S, H, generator=g).to(torch.bfloat16).cuda()
    w = torch.rand(S, K, generator=g).cuda()
    topk = torch.randint(0, E, (S, K), generator=g, dtype=torch.int32).cuda()
    rows, wn, cu, plan = buf.dispatch(hidden, w, topk)
    assert rows.shape == (buf.native.NvS, H) and cu.shape == (E + buf.B,)
    y, wk, ev = buf.combine(plan, rows, wn)
    torch.cuda.synchronize()
    buf.native.check_pending_status(plan)
    assert torch.allclose(y.float(), hidden.float() * K, rtol=1e-2, atol=1e-2)
    assert torch.equal(wk, w)
    again = buf.dispatch(hidden, w, plan=plan.clone())
    torch.cuda.synchronize()
    assert torch.equal(again[0], rows)
    buf.destroy()
    comm.destroy()


def test_context_owned_buffer_forward_and_backward(txr, port):
    """The reference's construction order: a context from the launcher's environment, a buffer that owns it, forward and
    backward with state objects (integrations/moonep_torch/tilexr_moonep/torch_api.py:284-304, 388-443, 1612-1683)."""
    from tilexr_b200.integrations import moonep

    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{port}", buffer_mb=64, device=0)
    S, H, K, E = 32, 128, 2, 8
    ctx = moonep.TileXRMoonEPContext.from_env(tokens_per_rank=S, hidden_size=H, topk=K, expert_count=E, dtype=torch.bfloat16,
                                              token_padding=4, runtime=comm)
    buf = moonep.TileXRMoonEPBuffer.from_context(ctx)
    assert buf.NvS == ctx.nv_s and buf.B == ctx.prefetch_slots == E
    with pytest.raises(RuntimeError):
        moonep.TileXRMoonEPBuffer.from_context(ctx)                   # one owner at a time
    g = torch.Generator().manual_seed(4)
    hidden = torch.randn(S, H, generator=g).to(torch.bfloat16).cuda()
    w = torch.rand(S, K, generator=g).cuda()
    topk = torch.randint(0, E, (S, K), generator=g, dtype=torch.int32).cuda()
    fwd = buf.forward_state(hidden, w, topk, None, None, lambda rows, cu, proj: rows.clone())
    torch.cuda.synchronize()
    buf.check_pending_status(fwd.state.plan)
    want = hidden.float() * w.sum(dim=1, keepdim=True)                 # identity experts, rows weighted before the sum
    assert torch.allclose(fwd.hidden.float(), want, rtol=2e-2, atol=2e-2)
    bwd = buf.backward_state(hidden, fwd.state, lambda rows, cu: rows.clone())
    torch.cuda.synchronize()
    buf.check_pending_status(bwd.plan)
    assert torch.allclose(bwd.grad_hidden.float(), hidden.float() * K, rtol=1e-2, atol=1e-2)
    assert buf.reduce_grad_info()["owned_rows"] == E
    buf.close()
    ctx.close()
    comm.destroy()


def test_harness_correctness_runner_single_rank(txr, port):
    """The harness compares the library with the torch reference, artifact by artifact."""
    from tilexr_b200.tools.moonep.contracts import MoonEPCase
    from tilexr_b200.tools.moonep.correctness import CorrectnessRunner
    from tilexr_b200.tools.moonep.tilexr_backend import TileXRBackend
    from tilexr_b200.tools.moonep.torch_reference_backend import TorchReferenceBackend

    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{port}", buffer_mb=64, device=0)
    backend = TileXRBackend(comm)
    runner = CorrectnessRunner(TorchReferenceBackend(), backend)
    for case in (MoonEPCase("r1_k2", 1, 32, 256, 2, 4, 2, token_padding=4, ffn=8, seed=3),
                 MoonEPCase("r1_k4_fp16", 1, 24, 512, 4, 8, 8, token_padding=1, dtype="float16", seed=4)):
        result = runner.run_case(case)
        assert result["ok_all_ranks"], result
    backend.close()
    comm.destroy()


@pytest.mark.parametrize("r,s,k,e,b,dtype", [(2, 40, 8, 8, 2, torch.bfloat16), (4, 64, 8, 16, 4, torch.bfloat16), (4, 48, 4, 32, 4, torch.float32)])
def test_combine_folds_duplicates_and_leaves_a_profile(txr, r, s, k, e, b, dtype):
    """Second-generation combine: the rows a token has on one rank come back as one.  Against the first generation
    (one rounding) the result may move by about a unit in the last place; the weights return bit-exact; every block
    leaves a profile record whose counters add up to the rows of the plan."""
    C = txr._C
    from tilexr_b200.tools.moonep import combine_v2_trace

    world = txr.init_emulated_world(r, device=0, buffer_mb=64)
    topk = _topk(r, s, k, e, 13)
    topk_dev = [t.cuda() for t in topk]
    plans = world.run(lambda c, rank: C.moonep_planning(c, topk_dev[rank], e, b, 4))
    world.check()
    nvs, n, h = plans[0]["NvS"], s * k, 512
    g = torch.Generator().manual_seed(21)
    hidden = [torch.randn(s, h, generator=g).to(dtype).cuda() for _ in range(r)]
    weights = [torch.rand(s, k, generator=g).cuda() for _ in range(r)]
    rows = world.symm_empty((nvs, h), dtype)
    wrow = world.symm_empty((nvs,), torch.float32)
    world.run(lambda c, rank: C.moonep_dispatch(c, plans[rank], hidden[rank], weights[rank], rows[rank], wrow[rank]))
    world.check()
    # a stand-in expert that makes every row different: scale by 1 + slot / 64
    processed = [(rows[rank].float() * (1 + torch.arange(nvs, device="cuda").unsqueeze(1) / 64)).to(dtype) for rank in range(r)]
    out1 = [torch.empty(s, h, dtype=dtype, device="cuda") for _ in range(r)]
    w1 = [torch.empty(s, k, dtype=torch.float32, device="cuda") for _ in range(r)]
    world.run(lambda c, rank: C.moonep_combine(c, plans[rank], processed[rank], wrow[rank], out1[rank], w1[rank]))
    world.check()
    nbytes, prof_off, _, _, rec_bytes, rec_max = C.moonep_combine_v2_workspace(s, h, k, nvs, dtype)
    assert rec_bytes == combine_v2_trace.RECORD_BYTES
    ws = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(r)]
    for launch in range(2):                                         # the index is rebuilt by every launch
        out2 = [torch.full((s, h), float("nan"), dtype=dtype, device="cuda") for _ in range(r)]
        w2 = [torch.empty(s, k, dtype=torch.float32, device="cuda") for _ in range(r)]
        world.run(lambda c, rank: C.moonep_combine_v2(c, plans[rank]["dst_local"], processed[rank], wrow[rank], out2[rank], w2[rank], ws[rank], k))
        world.check()
        for rank in range(r):
            assert torch.equal(w2[rank], weights[rank])
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert torch.allclose(out2[rank].float(), out1[rank].float(), rtol=tol, atol=tol), (out2[rank].float() - out1[rank].float()).abs().max()
    folded_total = 0
    for rank in range(r):
        raw = ws[rank][prof_off:prof_off + rec_bytes * rec_max].cpu().numpy().tobytes()
        recs = combine_v2_trace.decode_profile_records(raw)
        assert recs and all(x["rank"] == rank and "failure" not in x for x in recs)
        assert {x["block"] for x in recs} == set(range(recs[0]["grid_dim"]))
        tot = combine_v2_trace.totals(recs)
        valid = int((plans[rank]["dst_local"] >= 0).sum())
        assert tot["rows_indexed"] == valid and tot["groups_sent"] + tot["rows_folded"] == valid
        assert tot["tokens_reduced"] == s and tot["bytes_sent"] == tot["groups_sent"] * h * hidden[0].element_size()
        folded_total += tot["rows_folded"]
        t = recs[0]["time_ns"]
        assert t["begin"] <= t["index_cleared"] <= t["index_built"] <= t["send_end"] <= t["reduce_end"] <= t["end"]
        assert [row["stage"] for row in combine_v2_trace.stage_table(recs)] == [st[0] for st in combine_v2_trace.STAGES]
        assert combine_v2_trace.chrome_trace(recs)["traceEvents"]
    # the expected number of folded rows from the plans themselves: routes of a token that share a destination rank
    want_folded = 0
    for src in range(r):
        dst = plans[src]["dst"].cpu()
        dest = (torch.where(dst >= 0, dst, ~dst) // nvs).view(s, k)
        for t_ in range(s):
            want_folded += k - len(set(dest[t_].tolist()))
    assert folded_total == want_folded and (k <= r or folded_total > 0)
    world.destroy()


def test_dispatch_event_trace_decodes(txr):
    """The dispatch kernel's event trace: header, one record per block, route-send events whose rows add up to the
    routes of the plan; a short buffer is refused before anything is launched."""
    C = txr._C
    from tilexr_b200.tools.moonep import dispatch_trace

    r, s, k, e, b, h = 4, 64, 4, 16, 4, 256
    world = txr.init_emulated_world(r, device=0, buffer_mb=32)
    topk_dev = [t.cuda() for t in _topk(r, s, k, e, 17)]
    plans = world.run(lambda c, rank: C.moonep_planning(c, topk_dev[rank], e, b, 1))
    world.check()
    nvs = plans[0]["NvS"]
    g = torch.Generator().manual_seed(2)
    hidden = [torch.randn(s, h, generator=g).to(torch.bfloat16).cuda() for _ in range(r)]
    rows = world.symm_empty((nvs, h), torch.bfloat16)
    blocks, cap, iters = 128, 32, 2
    assert dispatch_trace.trace_layout(iters, blocks, cap)["trace_bytes"] == C.moonep_trace_layout(iters, blocks, cap)[2]
    bufs = [torch.zeros(C.moonep_trace_layout(iters, blocks, cap)[2], dtype=torch.uint8, device="cuda") for _ in range(r)]
    for it in range(iters):
        world.run(lambda c, rank: C.moonep_dispatch(c, plans[rank], hidden[rank], None, rows[rank], None, bufs[rank], it, iters, cap))
        world.check()
    for rank in range(r):
        trace = dispatch_trace.decode_trace(bufs[rank].cpu().numpy().tobytes())
        assert trace["header"]["rank"] == rank and trace["header"]["rank_size"] == r and trace["header"]["iterations"] == iters
        grid = trace["header"]["blocks"]
        assert len(trace["blocks"]) == iters * grid and all(blk["status"] == 0 and blk["dropped"] == 0 for blk in trace["blocks"])
        for it in range(iters):
            sent = sum(ev["rows"] for blk in trace["blocks"] if blk["iteration"] == it for ev in blk["events"] if ev["phase_name"] == "route-send")
            assert sent == s * k
        names = {row["phase"] for row in dispatch_trace.phase_summary(trace)}
        assert {"plan-check", "zero-fill", "route-send", "flag-raise", "flag-wait"} <= names and "output-copy" not in names
        assert all(ev["end_ns"] >= ev["begin_ns"] for blk in trace["blocks"] for ev in blk["events"])
        assert dispatch_trace.chrome_trace(trace)["traceEvents"]
    small = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        with txr.group():
            for rank, c in enumerate(world.comms):
                C.moonep_dispatch(c, plans[rank], hidden[rank], None, rows[rank], None, small, 0, 1, cap)
    world.destroy()


def test_dispatch_reports_a_destination_outside_the_communicator(txr):
    C = txr._C
    r, s, k, e, b, h = 2, 16, 2, 4, 2, 128
    world = txr.init_emulated_world(r, device=0, buffer_mb=32)
    topk_dev = [t.cuda() for t in _topk(r, s, k, e, 19)]
    plans = world.run(lambda c, rank: C.moonep_planning(c, topk_dev[rank], e, b, 1))
    world.check()
    nvs = plans[0]["NvS"]
    plans[1]["dst"][3] = 5 * nvs + 1                                    # rank 5 of 2
    hidden = [torch.randn(s, h).to(torch.bfloat16).cuda() for _ in range(r)]
    rows = world.symm_empty((nvs, h), torch.bfloat16)
    world.run(lambda c, rank: C.moonep_dispatch(c, plans[rank], hidden[rank], None, rows[rank], None))
    torch.cuda.synchronize()
    assert world.comms[1].device_status() == 4                          # TILEXR_DEV_BAD_ARGUMENT, not a silent skip
    assert world.comms[1].dfx()[6] == 3                                 # the failing route
    for c in world.comms:
        c.reset_status()
    world.destroy()
