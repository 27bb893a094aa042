"""Expert-parallel dispatch / combine and the local hot ops against fp32 PyTorch references."""
import pytest
import torch

from conftest import require_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def txr():
    require_cuda()
    import tilexr_b200

    return tilexr_b200


@pytest.mark.parametrize("score_func,renorm,bias", [(0, True, False), (1, True, False), (1, False, True)])
def test_routing_topk(txr, score_func, renorm, bias):
    from tilexr_b200.utils import oracle

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(333, 256, generator=g)
    b = torch.randn(256, generator=g) * 0.1 if bias else None
    ids, w = txr.quant.routing_topk(logits.cuda(), 8, score_func, renorm, 2.5, None if b is None else b.cuda())
    rids, rw = oracle.routing_topk_ref(logits, 8, score_func, renorm, 2.5, b)
    assert torch.equal(ids.cpu(), rids)
    assert torch.allclose(w.cpu(), rw, rtol=1e-5, atol=1e-7)


def test_fp8_quant_1x128_matches_reference(txr):
    from tilexr_b200.utils import oracle

    g = torch.Generator().manual_seed(1)
    x = (torch.randn(257, 7168, generator=g) * 3).to(torch.bfloat16)
    x[5] = 0       # an all-zero row hits the amax floor
    q, s = txr.quant.fp8_quant_1x128(x.cuda())
    rq, rs = oracle.fp8_quant_1x128_ref(x)
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    back = txr.quant.fp8_dequant_1x128(q, s, torch.bfloat16)
    ref_back = oracle.fp8_dequant_1x128_ref(rq, rs).to(torch.bfloat16)
    assert torch.equal(back.cpu(), ref_back)
    rel = (back.cpu().float() - x.float()).abs().max() / x.float().abs().max()
    assert rel < 0.07


@pytest.mark.parametrize("e5m2", [False, True])
def test_mxfp8_matches_reference(txr, e5m2):
    from tilexr_b200.utils import oracle

    g = torch.Generator().manual_seed(2)
    x = (torch.randn(64, 1000, generator=g) * torch.logspace(-3, 3, 1000)).to(torch.float16)
    q, s = txr.quant.mxfp8_quant(x.cuda(), e5m2)
    rq, rs = oracle.mxfp8_quant_ref(x, e5m2)
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    back = txr.quant.mxfp8_dequant(q, s, torch.float16)
    assert torch.allclose(back.cpu().float(), oracle.mxfp8_dequant_ref(rq, rs).to(torch.float16).float(), rtol=0, atol=0)


@pytest.mark.parametrize("with_residual", [False, True])
def test_rmsnorm(txr, with_residual):
    from tilexr_b200.utils import oracle

    g = torch.Generator().manual_seed(3)
    x = torch.randn(37, 8192, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(8192, generator=g)).to(torch.bfloat16)
    res = torch.randn(37, 8192, generator=g).to(torch.bfloat16) if with_residual else None
    res_dev = res.cuda() if with_residual else None
    y = txr.quant.rmsnorm(x.cuda(), gamma.cuda(), 1e-6, res_dev)
    ry, rres = oracle.rmsnorm_ref(x, gamma, 1e-6, res)
    assert torch.allclose(y.cpu().float(), ry.float(), rtol=2e-2, atol=2e-2)
    assert (y.cpu().float() - ry.float()).abs().mean() < 2e-3
    if with_residual:
        assert torch.equal(res_dev.cpu(), rres)


def _ep_case(txr, ranks, bs, h, experts, top_k, quant, fused_routing, masks=False, zero_copy=False, dtype=torch.bfloat16,
             dedup=None, scales_at_dispatch=False):
    from tilexr_b200.ops import ep
    from tilexr_b200.utils import oracle

    world = txr.init_emulated_world(ranks, device=0, buffer_mb=128)
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(bs, h, generator=g).to(dtype) for _ in range(ranks)]
    logits = [torch.randn(bs, experts, generator=g) for _ in range(ranks)]
    routed = [oracle.routing_topk_ref(l, top_k, 1, True, 1.0) for l in logits]
    ids = [r[0] for r in routed]
    ws = [r[1] for r in routed]
    mask = None
    if masks:
        mask = [(torch.rand(bs, generator=g) > 0.3) for _ in range(ranks)]
    max_rows = bs * ranks * min(top_k, experts // ranks)
    outs = world.symm_empty((max_rows, h), torch.float8_e4m3fn if quant else dtype) if zero_copy else [None] * ranks
    for _ in range(2):
        def call(c, r):
            kw = dict(num_experts=experts, top_k=top_k, quant_mode=ep.QUANT_FP8_1X128 if quant else ep.QUANT_NONE,
                      score_func=1, renormalize=True, max_recv_rows=max_rows, expand_x_out=outs[r],
                      active_mask=None if mask is None else mask[r].cuda(), dedup=dedup)
            if scales_at_dispatch:
                kw["expert_scales"] = ws[r].cuda()
            if fused_routing:
                return ep.dispatch(c, xs[r].cuda(), gate_logits=logits[r].cuda(), **kw)
            return ep.dispatch(c, xs[r].cuda(), expert_ids=ids[r].cuda(), **kw)
        res = world.run(call)
        world.check()
    ref = oracle.ep_dispatch_ref(xs, ids, experts, mask)
    expert_outs = []
    for r in range(ranks):
        d = res[r]
        n = int(d.recv_total.item())
        assert n == len(ref[r]["rows"])
        assert torch.equal(d.assist[:n].cpu(), ref[r]["assist"])
        assert torch.equal(d.expert_token_nums.cpu(), ref[r]["token_nums"])
        assert torch.equal(d.send_counts.cpu(), ref[r]["send_counts"])
        if fused_routing or scales_at_dispatch:
            # the gate weight of every received row travelled with it
            a = ref[r]["assist"].long()
            want_w = torch.stack([ws[int(s)][int(t), int(k)] for s, t, k, _ in a.tolist()]) if n else torch.empty(0)
            assert torch.allclose(d.expand_scales[:n].cpu(), want_w, rtol=1e-5, atol=1e-7)
        if fused_routing:
            assert torch.equal(d.topk_ids.cpu(), ids[r])
            assert torch.allclose(d.topk_weights.cpu(), ws[r], rtol=1e-5, atol=1e-7)
        if quant:
            rq, rs = oracle.fp8_quant_1x128_ref(ref[r]["expand_x"]) if n else (None, None)
            if n:
                assert torch.equal(d.expand_x[:n].cpu().view(torch.uint8), rq.view(torch.uint8))
                assert torch.equal(d.dynamic_scales[:n].cpu(), rs)
            rows = txr.quant.fp8_dequant_1x128(d.expand_x, d.dynamic_scales, dtype)
        else:
            assert torch.equal(d.expand_x[:n].cpu(), ref[r]["expand_x"])
            rows = d.expand_x
        # stand-in expert: scale by (1 + local expert index / 8)
        e_local = (d.assist[:, 3] % (experts // ranks)).clamp(min=0).float().cuda()
        out = (rows.float() * (1 + e_local / 8).unsqueeze(1)).to(dtype)
        expert_outs.append(out)

    ys = world.run(lambda c, r: ep.combine(c, expert_outs[r], res[r], expert_scales=ws[r].cuda(),
                                           active_mask=None if mask is None else mask[r].cuda()))
    world.check()
    ref_outs = [expert_outs[r][: len(ref[r]["rows"])].cpu() for r in range(ranks)]
    yref = oracle.ep_combine_ref(ref, ref_outs, ids, ws, dtype)
    for r in range(ranks):
        got = ys[r].cpu().float()
        want = yref[r].float()
        if mask is not None:
            want = want * mask[r].unsqueeze(1).float()
        assert torch.allclose(got, want, rtol=2e-2, atol=2e-2), (got - want).abs().max()
        assert (got - want).abs().mean() < 1e-3
    world.destroy()


def test_ep_bf16_explicit_ids(txr):
    _ep_case(txr, ranks=4, bs=48, h=256, experts=16, top_k=2, quant=False, fused_routing=False)


def test_ep_fp8_fused_routing(txr):
    _ep_case(txr, ranks=4, bs=40, h=1024, experts=32, top_k=4, quant=True, fused_routing=True)


def test_ep_token_mask(txr):
    _ep_case(txr, ranks=2, bs=33, h=512, experts=8, top_k=2, quant=True, fused_routing=False, masks=True)


def test_ep_zero_copy_output(txr):
    _ep_case(txr, ranks=4, bs=64, h=512, experts=16, top_k=4, quant=True, fused_routing=True, zero_copy=True)


def test_ep_eight_ranks_fp16(txr):
    _ep_case(txr, ranks=8, bs=24, h=512, experts=64, top_k=8, quant=False, fused_routing=True, dtype=torch.float16)


def test_ep_dedup_explicit_ids_with_scales(txr):
    # top-8 over 2 ranks: nearly every token has several experts on the remote rank
    _ep_case(txr, ranks=2, bs=40, h=512, experts=16, top_k=8, quant=True, fused_routing=False, scales_at_dispatch=True,
             zero_copy=True)


def test_ep_dedup_staged_output_and_masks(txr):
    _ep_case(txr, ranks=4, bs=37, h=256, experts=32, top_k=6, quant=False, fused_routing=True, masks=True)


def test_ep_large_batch_overlapped_combine(txr):
    # enough routes for combine's bucketed send order with dedicated reducer blocks
    _ep_case(txr, ranks=2, bs=1536, h=512, experts=16, top_k=8, quant=True, fused_routing=True, zero_copy=True)


def test_ep_dedup_off_matches(txr):
    _ep_case(txr, ranks=4, bs=40, h=1024, experts=32, top_k=4, quant=True, fused_routing=True, dedup=False)


@pytest.mark.parametrize("e5m2", [False, True])
def test_ep_dispatch_fused_mxfp8(txr, e5m2):
    """quantMode 3 / 4: rows arrive as MXFP8 with one E8M0 exponent byte per 32 elements, bit-exact vs the reference."""
    from tilexr_b200.ops import ep
    from tilexr_b200.utils import oracle

    ranks, bs, h, experts, top_k = 4, 36, 1024, 16, 4
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=64)
    g = torch.Generator().manual_seed(21)
    xs = [(torch.randn(bs, h, generator=g) * (1 + 3 * torch.rand(bs, 1, generator=g))).to(torch.bfloat16) for _ in range(ranks)]
    xs[0][0, :40] = 0                                  # an all-zero block
    logits = [torch.randn(bs, experts, generator=g) for _ in range(ranks)]
    ids = [oracle.routing_topk_ref(l, top_k, 1, True, 1.0)[0] for l in logits]
    mode = ep.QUANT_MXFP8_E5M2 if e5m2 else ep.QUANT_MXFP8_E4M3
    res = world.run(lambda c, r: ep.dispatch(c, xs[r].cuda(), gate_logits=logits[r].cuda(), num_experts=experts, top_k=top_k,
                                             quant_mode=mode, score_func=1))
    world.check()
    ref = oracle.ep_dispatch_ref(xs, ids, experts, None)
    for r in range(ranks):
        d = res[r]
        n = int(d.recv_total.item())
        assert n == len(ref[r]["rows"]) and n > 0
        assert d.expand_x.dtype == (torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn)
        assert d.dynamic_scales.dtype == torch.uint8 and tuple(d.dynamic_scales.shape[1:]) == (h // 32,)
        rq, rs = oracle.mxfp8_quant_ref(ref[r]["expand_x"], e5m2)
        assert torch.equal(d.expand_x[:n].cpu().view(torch.uint8), rq.view(torch.uint8))
        assert torch.equal(d.dynamic_scales[:n].cpu(), rs)
    world.destroy()


@pytest.mark.parametrize("dynamic,smooth", [(True, False), (True, True), (False, True)])
def test_ep_dispatch_int8_modes(txr, dynamic, smooth):
    """quantMode 1 (static) and 2 (per-row dynamic) int8, with per-expert smoothing scales."""
    from tilexr_b200.ops import ep
    from tilexr_b200.utils import oracle

    ranks, bs, h, experts, top_k = 2, 20, 512, 8, 3
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=64)
    g = torch.Generator().manual_seed(31)
    xs = [torch.randn(bs, h, generator=g).to(torch.bfloat16) for _ in range(ranks)]
    ids = [torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(bs)]).to(torch.int32) for _ in range(ranks)]
    ws = [torch.rand(bs, top_k, generator=g) for _ in range(ranks)]
    smooth_scales = (0.5 + torch.rand(experts, h, generator=g)) * (1.0 if dynamic else 20.0) if smooth else None
    mode = ep.QUANT_DYNAMIC_INT8 if dynamic else ep.QUANT_STATIC_INT8
    res = world.run(lambda c, r: ep.dispatch(c, xs[r].cuda(), expert_ids=ids[r].cuda(), expert_scales=ws[r].cuda(),
                                             num_experts=experts, top_k=top_k, quant_mode=mode,
                                             scales=None if smooth_scales is None else smooth_scales.cuda()))
    world.check()
    ref = oracle.ep_dispatch_ref(xs, ids, experts, None)
    for r in range(ranks):
        d = res[r]
        n = int(d.recv_total.item())
        assert n == len(ref[r]["rows"]) and d.expand_x.dtype == torch.int8
        v = ref[r]["expand_x"].float()
        if smooth_scales is not None:
            v = v * smooth_scales[ref[r]["assist"][:, 3].long()]
        if dynamic:
            amax = v.abs().amax(dim=1)
            inv = torch.where(amax > 0, torch.full_like(amax, 127.0) / amax, torch.ones_like(amax))   # tensor / tensor: IEEE division
            want = torch.round(v * inv.unsqueeze(1)).clamp(-128, 127).to(torch.int8)
            assert torch.equal(d.dynamic_scales[:n].cpu(), torch.where(amax > 0, amax / 127.0, torch.ones_like(amax)))
        else:
            want = torch.round(v).clamp(-128, 127).to(torch.int8)
            assert d.dynamic_scales is None
        assert torch.equal(d.expand_x[:n].cpu(), want)
        assert d.dedup == (smooth_scales is None)
    world.destroy()


def test_ep_shared_expert_ranks(txr):
    """Two leading ranks hold the shared expert (one copy each), two hold the routed experts: every token also
    goes to its copy of the shared expert (slot top_k, weight 1), cf. the reference's destination rule."""
    from tilexr_b200.ops import ep
    from tilexr_b200.utils import oracle

    ranks, shared_ranks, shared_experts, bs, h, experts, top_k = 4, 2, 1, 24, 256, 8, 2
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=64)
    g = torch.Generator().manual_seed(41)
    xs = [torch.randn(bs, h, generator=g).to(torch.bfloat16) for _ in range(ranks)]
    logits = [torch.randn(bs, experts, generator=g) for _ in range(ranks)]
    routed = [oracle.routing_topk_ref(l, top_k, 1, True, 1.0) for l in logits]
    ids, ws = [r[0] for r in routed], [r[1] for r in routed]
    res = world.run(lambda c, r: ep.dispatch(c, xs[r].cuda(), gate_logits=logits[r].cuda(), num_experts=experts, top_k=top_k,
                                             score_func=1, shared_expert_num=shared_experts, shared_expert_rank_num=shared_ranks))
    world.check()
    per_shared = shared_ranks // shared_experts
    moe_per_rank = experts // (ranks - shared_ranks)
    # expected rows per destination: local expert major, then source rank, then token order
    for dst in range(ranks):
        want = []      # (src, token, slot, expert id)
        local = [None] if dst < shared_ranks else list(range((dst - shared_ranks) * moe_per_rank, (dst - shared_ranks + 1) * moe_per_rank))
        for e in local:
            for src in range(ranks):
                for t in range(bs):
                    if e is None:
                        if src % per_shared + 0 * per_shared == dst:
                            want.append((src, t, top_k, 0))
                    else:
                        for k in range(top_k):
                            if int(ids[src][t, k]) == e:
                                want.append((src, t, k, e))
        d = res[dst]
        n = int(d.recv_total.item())
        assert n == len(want), (dst, n, len(want))
        assert d.assist[:n].cpu().tolist() == [list(w) for w in want]
        rows = torch.stack([xs[s][t] for s, t, _, _ in want]) if want else torch.empty(0, h, dtype=torch.bfloat16)
        assert torch.equal(d.expand_x[:n].cpu(), rows)
        assert d.expert_token_nums.numel() == (1 if dst < shared_ranks else moe_per_rank)
    # identity experts: y = sum_k w_k x + x (the shared expert's copy)
    ys = world.run(lambda c, r: ep.combine(c, res[r].expand_x, res[r], expert_scales=ws[r].cuda()))
    world.check()
    for r in range(ranks):
        want = (xs[r].float() * (ws[r].sum(dim=1, keepdim=True) + 1.0))
        assert torch.allclose(ys[r].cpu().float(), want, rtol=2e-2, atol=2e-2)
    world.destroy()


def test_ep_overflow_is_reported_not_written(txr):
    from tilexr_b200.ops import ep

    world = txr.init_emulated_world(2, device=0, buffer_mb=64)
    x = [torch.randn(16, 256).to(torch.bfloat16).cuda() for _ in range(2)]
    ids = [torch.zeros(16, 2, dtype=torch.int32).cuda() for _ in range(2)]     # every route to expert 0
    ids[0][:, 1] = 1
    ids[1][:, 1] = 1
    world.run(lambda c, r: ep.dispatch(c, x[r], expert_ids=ids[r], num_experts=4, top_k=2, max_recv_rows=8))
    torch.cuda.synchronize()
    assert all(c.device_status() == 4 for c in world.comms)      # TILEXR_DEV_BAD_ARGUMENT on every rank
    for c in world.comms:
        c.reset_status()
    world.destroy()


def test_reset_status_keeps_flags_meaningful(txr):
    """After a failed launch and reset_status the next launches must still WAIT for their flags: the reset keeps
    the launch epoch, so flags left by earlier launches stay older than anything a new launch waits for."""
    from tilexr_b200.ops import ep
    from tilexr_b200.utils import oracle

    ranks = 4
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=64)
    g = torch.Generator().manual_seed(5)
    # a few launches first, so that flags and done epochs of earlier launches exist
    for i in range(5):
        xs = [torch.randn(3000, generator=g).cuda() for _ in range(ranks)]
        outs = world.run(lambda c, r: txr.all_reduce(c, xs[r]))
        world.check()
        assert torch.allclose(outs[0], sum(xs), rtol=1e-5, atol=1e-5)
    epoch_before = [c.dfx()[0] for c in world.comms]
    x = [torch.randn(16, 256, generator=g).to(torch.bfloat16).cuda() for _ in range(ranks)]
    ids = [torch.zeros(16, 2, dtype=torch.int32).cuda() for _ in range(ranks)]
    for r in range(ranks):
        ids[r][:, 1] = 1
    world.run(lambda c, r: ep.dispatch(c, x[r], expert_ids=ids[r], num_experts=8, top_k=2, max_recv_rows=8))
    torch.cuda.synchronize()
    assert all(c.device_status() == 4 for c in world.comms)
    for c in world.comms:
        c.reset_status()
    assert all(c.device_status() == 0 for c in world.comms)
    for i in range(3):
        xs = [torch.randn(5000, generator=g).cuda() for _ in range(ranks)]
        outs = world.run(lambda c, r: txr.all_reduce(c, xs[r]))
        gathered = world.run(lambda c, r: txr.all_gather(c, xs[r]))
        world.check()
        for r in range(ranks):
            assert torch.allclose(outs[r], sum(xs), rtol=1e-5, atol=1e-5)
            assert torch.equal(gathered[r], torch.stack(xs))
    assert all(c.dfx()[0] > e for c, e in zip(world.comms, epoch_before))      # the epoch went on, it did not restart
    xs = [torch.randn(24, 256, generator=g).to(torch.bfloat16) for _ in range(ranks)]
    ids = [torch.randint(0, 8, (24, 2), generator=g, dtype=torch.int32) for _ in range(ranks)]
    for t in ids:
        t[:, 1] = (t[:, 0] + 1 + t[:, 1] % 7) % 8                                # two different experts per token
    res = world.run(lambda c, r: ep.dispatch(c, xs[r].cuda(), expert_ids=ids[r].cuda(), num_experts=8, top_k=2))
    world.check()
    ref = oracle.ep_dispatch_ref(xs, ids, 8, None)
    for r in range(ranks):
        n = int(res[r].recv_total.item())
        assert n == len(ref[r]["rows"])
        assert torch.equal(res[r].assist[:n].cpu(), ref[r]["assist"])
        assert torch.equal(res[r].expand_x[:n].cpu(), ref[r]["expand_x"])
    world.destroy()


@pytest.mark.parametrize("fp8", [False, True])
def test_moe_layer_matches_a_dense_reference(txr, fp8):
    """The MoE block (routing, dispatch, expert FFN on the tcgen05 GEMM, combine) against plain PyTorch in fp32."""
    from conftest import free_port
    from tilexr_b200.models import ExpertParallelMoE, MoEConfig
    from tilexr_b200.utils import oracle

    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{free_port()}", buffer_mb=64, device=0)
    cfg = MoEConfig(hidden=512, ffn=256, num_experts=8, top_k=2, fp8_dispatch=fp8)
    layer = ExpertParallelMoE(comm, cfg, seed=3)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(96, cfg.hidden, generator=g).to(torch.bfloat16)
    y = layer(x.cuda())
    torch.cuda.synchronize()
    assert comm.device_status() == 0
    logits = x.float() @ layer.gate.detach().cpu().t()
    ids, ws = oracle.routing_topk_ref(logits, cfg.top_k, cfg.score_func, cfg.renormalize, cfg.routed_scale)
    xin = x.float()
    if fp8:
        q, s = oracle.fp8_quant_1x128_ref(x)
        xin = oracle.fp8_dequant_1x128_ref(q, s).to(torch.bfloat16).float()
    w13, w2 = layer.w13.detach().cpu().float(), layer.w2.detach().cpu().float()
    want = torch.zeros(96, cfg.hidden)
    for t in range(96):
        for k in range(cfg.top_k):
            e = int(ids[t, k])
            gu = xin[t] @ w13[e].t()                                  # gate and up rows interleaved; the activation runs in fp32
            hmid = (torch.nn.functional.silu(gu[0::2]) * gu[1::2]).to(torch.bfloat16).float()
            want[t] += float(ws[t, k]) * (hmid @ w2[e].t()).to(torch.bfloat16).float()
    got = y.cpu().float()
    assert torch.allclose(got, want, rtol=3e-2, atol=3e-3), (got - want).abs().max()
    comm.destroy()


@pytest.mark.parametrize("dedup", [False, True])
def test_ep_with_tensor_parallel_groups(txr, dedup):
    """tpWorldSize 2 on four ranks: two expert groups of two ranks.  Every route reaches both ranks of its group, sorted
    by local expert; the lane counts come back; combine adds the two partial outputs of every row."""
    from tilexr_b200.ops import ep
    from tilexr_b200.utils import oracle

    ranks, T, bs, h, experts, top_k = 4, 2, 24, 512, 8, 2
    groups, per = ranks // T, experts // (ranks // T)
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=64)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(bs, h, generator=g).to(torch.bfloat16) for _ in range(ranks)]
    routed = [oracle.routing_topk_ref(torch.randn(bs, experts, generator=g), top_k, 1, True, 1.0) for _ in range(ranks)]
    ids, ws = [r[0] for r in routed], [r[1] for r in routed]
    ids[1][3, 1] = -1                                     # an inactive route
    res = world.run(lambda c, r: ep.dispatch(c, xs[r].cuda(), expert_ids=ids[r].cuda(), expert_scales=ws[r].cuda(),
                                             num_experts=experts, top_k=top_k, tp_world_size=T, dedup=dedup))
    world.check()
    # the same dispatch stated on lane experts: route (t, k) -> slots k * T + l on expert ((group * T + l) * per + local)
    wide = []
    for r in range(ranks):
        e = ids[r].long()
        lane = torch.arange(T).view(1, 1, T)
        v = ((e // per).unsqueeze(-1) * T + lane) * per + (e % per).unsqueeze(-1)
        v = torch.where(e.unsqueeze(-1) >= 0, v, torch.full_like(v, -1))
        wide.append(v.reshape(bs, top_k * T).to(torch.int32))
    ref = oracle.ep_dispatch_ref(xs, wide, experts * T)
    for r in range(ranks):
        d = res[r]
        n = int(d.recv_total.item())
        assert n == len(ref[r]["rows"]) and n > 0
        assert torch.equal(d.assist[:n].cpu(), ref[r]["assist"])
        assert torch.equal(d.expand_x[:n].cpu(), ref[r]["expand_x"])
        assert torch.equal(d.expert_token_nums.cpu(), ref[r]["token_nums"]) and d.expert_token_nums.numel() == per
        assert torch.equal(d.send_counts.cpu(), ref[r]["send_counts"])
        by_lane = [sum(1 for (s, _, _, _) in ref[r]["rows"] if s % T == l) for l in range(T)]
        assert d.tp_recv_counts.cpu().tolist() == by_lane
        # both ranks of a group hold the same rows
        mate = res[r ^ 1]
        assert torch.equal(mate.expand_x[:n].cpu(), d.expand_x[:n].cpu())
    # each rank returns its "partial output": the row scaled by a factor of its own
    factor = [1.0 + r / 8 for r in range(ranks)]
    outs = [(res[r].expand_x.float() * factor[r]).to(torch.bfloat16) for r in range(ranks)]
    ys = world.run(lambda c, r: ep.combine(c, outs[r], res[r], expert_scales=ws[r].cuda()))
    world.check()
    for r in range(ranks):
        want = torch.zeros(bs, h)
        for t in range(bs):
            for k in range(top_k):
                e = int(ids[r][t, k])
                if e < 0:
                    continue
                for l in range(T):
                    owner = (e // per) * T + l
                    want[t] += float(ws[r][t, k]) * (xs[r][t].float() * factor[owner]).to(torch.bfloat16).float()
        got = ys[r].cpu().float()
        assert torch.allclose(got, want, rtol=2e-2, atol=2e-2), (got - want).abs().max()
    world.destroy()
