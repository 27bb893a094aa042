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
