"""Collective kernels against plain PyTorch references, on emulated worlds: R ranks share one
GPU and every op is ONE cooperative launch that covers all ranks, so the flag protocol between
ranks runs for real without needing R GPUs."""
import pytest
import torch

from conftest import require_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def txr():
    require_cuda()
    import tilexr_b200

    return tilexr_b200


def _world(txr, ranks, buffer_mb=64):
    return txr.init_emulated_world(ranks, device=0, buffer_mb=buffer_mb)


def _inputs(ranks, numel, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    if dtype.is_floating_point:
        return [torch.randn(numel, generator=g).to(dtype).cuda() for _ in range(ranks)]
    return [torch.randint(-50, 50, (numel,), generator=g).to(dtype).cuda() for _ in range(ranks)]


@pytest.mark.parametrize("ranks,numel,dtype", [
    (2, 1000, torch.float32), (4, 8192, torch.bfloat16), (8, 70001, torch.int32), (4, 1 << 20, torch.bfloat16),
    (3, 12345, torch.int8),
])
def test_all_gather(txr, ranks, numel, dtype):
    from tilexr_b200.utils import oracle

    world = _world(txr, ranks)
    xs = _inputs(ranks, numel, dtype)
    for _ in range(3):   # three epochs: both data halves and the reuse guard
        outs = world.run(lambda c, r: txr.all_gather(c, xs[r]))
        world.check()
    ref = oracle.all_gather_ref(xs)
    for o in outs:
        assert torch.equal(o.cpu().reshape(-1), ref)
    world.destroy()


def test_all_gather_zero_copy_into_symmetric_memory(txr):
    from tilexr_b200.utils import oracle

    ranks, numel = 4, 300000
    world = _world(txr, ranks)
    xs = _inputs(ranks, numel, torch.bfloat16, seed=3)
    outs = world.symm_empty((ranks, numel), torch.bfloat16)
    assert all(c.is_registered(o) for c, o in zip(world.comms, outs))
    world.run(lambda c, r: txr.all_gather(c, xs[r], out=outs[r]))
    world.check()
    ref = oracle.all_gather_ref(xs)
    for o in outs:
        assert torch.equal(o.cpu().reshape(-1), ref)
    world.destroy()


@pytest.mark.parametrize("ranks,per_peer,dtype", [(2, 777, torch.float32), (4, 65536, torch.bfloat16), (8, 4099, torch.int16)])
def test_all_to_all(txr, ranks, per_peer, dtype):
    from tilexr_b200.utils import oracle

    world = _world(txr, ranks)
    xs = _inputs(ranks, per_peer * ranks, dtype, seed=1)
    for _ in range(2):
        outs = world.run(lambda c, r: txr.all_to_all(c, xs[r]))
        world.check()
    refs = oracle.all_to_all_ref(xs)
    for o, ref in zip(outs, refs):
        assert torch.equal(o.cpu().reshape(-1), ref)
    world.destroy()


@pytest.mark.parametrize("ranks,numel,dtype,op", [
    (2, 513, torch.float32, "sum"),          # one-shot
    (8, 4096, torch.bfloat16, "sum"),        # one-shot, decode sized
    (4, 1 << 20, torch.bfloat16, "sum"),     # two-shot
    (8, 300001, torch.float32, "sum"),       # two-shot with a ragged tail and empty slices
    (4, 5000, torch.int32, "max"),
    (2, 4000, torch.float16, "min"),
    (4, 3000, torch.int64, "sum"),
])
def test_all_reduce(txr, ranks, numel, dtype, op):
    from tilexr_b200.utils import oracle

    world = _world(txr, ranks)
    xs = _inputs(ranks, numel, dtype, seed=2)
    rop = {"sum": txr.ReduceOp.SUM, "max": txr.ReduceOp.MAX, "min": txr.ReduceOp.MIN}[op]
    for _ in range(3):
        outs = world.run(lambda c, r: txr.all_reduce(c, xs[r], op=rop))
        world.check()
    ref = oracle.all_reduce_ref(xs, op)
    for o in outs:
        # same accumulation order as the reference: bit-identical, and identical on every rank
        assert torch.equal(o.cpu(), ref), (o.cpu().float() - ref.float()).abs().max()
    world.destroy()


@pytest.mark.parametrize("ranks,per_rank,dtype", [(2, 1000, torch.float32), (4, 131072, torch.bfloat16), (8, 999, torch.int32)])
def test_reduce_scatter(txr, ranks, per_rank, dtype):
    from tilexr_b200.utils import oracle

    world = _world(txr, ranks)
    xs = _inputs(ranks, per_rank * ranks, dtype, seed=5)
    outs = world.run(lambda c, r: txr.reduce_scatter(c, xs[r]))
    world.check()
    full = oracle.all_reduce_ref(xs)
    for r, o in enumerate(outs):
        assert torch.equal(o.cpu(), full[r * per_rank:(r + 1) * per_rank])
    world.destroy()


@pytest.mark.parametrize("ranks,numel,root", [(2, 100, 1), (4, 500000, 0), (8, 4097, 5), (4, 1 << 20, 2), (8, 3 << 19, 7)])   # the last two: scatter + all-gather
def test_broadcast(txr, ranks, numel, root):
    world = _world(txr, ranks)
    xs = _inputs(ranks, numel, torch.float32, seed=7)
    ref = xs[root].cpu().clone()
    world.run(lambda c, r: txr.broadcast(c, xs[r], root=root))
    world.check()
    for x in xs:
        assert torch.equal(x.cpu(), ref)
    world.destroy()


def test_large_all_gather_is_split_into_launches(txr):
    """A message larger than a pair's share of the window runs as several launches."""
    from tilexr_b200.utils import oracle

    ranks = 2
    world = _world(txr, ranks, buffer_mb=8)          # 4 MiB per half, 2 MiB per pair
    numel = (5 << 20) // 4                            # 5 MiB per rank
    xs = _inputs(ranks, numel, torch.float32, seed=9)
    before = txr.launch_count()
    outs = world.run(lambda c, r: txr.all_gather(c, xs[r]))
    world.check()
    assert txr.launch_count() - before >= 3
    ref = oracle.all_gather_ref(xs)
    for o in outs:
        assert torch.equal(o.cpu().reshape(-1), ref)
    world.destroy()


def test_single_rank_process_communicator_and_probe(txr, port):
    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{port}", buffer_mb=16, device=0)
    x = torch.arange(100000, dtype=torch.float32, device="cuda")
    y = txr.all_reduce(comm, x)
    z = txr.profile_probe(comm, x)
    torch.cuda.synchronize()
    assert torch.equal(x, y) and torch.equal(x, z)
    assert comm.device_status() == 0
    comm.destroy()


def test_perf_session_writes_reports(txr, tmp_path):
    import json

    world = _world(txr, 2)
    xs = _inputs(2, 1 << 18, torch.float32)
    session = txr._C.perf_session_create(str(tmp_path), 1, True, "cat analysis.md")
    session.activate()
    world.run(lambda c, r: txr.all_gather(c, xs[r]))
    world.check()
    session.deactivate()
    session.write_report()
    session.destroy()
    trace = json.loads((tmp_path / "rank0" / "launch0" / "trace.json").read_text())
    assert trace["op"] == "TileXRAllGather" and trace["records"]
    stages = {r["stage"] for r in trace["records"]}
    assert 0 in stages and 3 in stages        # kernel_total and local_input_to_ipc
    assert (tmp_path / "rank1" / "launch1" / "summary.csv").exists()
    assert (tmp_path / "rank0" / "launch0" / "ai_prompt.md").exists()
    world.destroy()


@pytest.mark.parametrize("ranks,numel,scale_count,dtype", [
    (2, 4096, 1, torch.float16), (4, 16 * 1031, 1, torch.bfloat16), (8, 64 * 1024, 256, torch.bfloat16), (3, 48 * 7, 48, torch.float16),
])
def test_all_reduce_quant(txr, ranks, numel, scale_count, dtype):
    """int8 payloads, dequantised and summed in fp32: out = sum_r (x_r + offset) * scale[i % scale_count]."""
    world = _world(txr, ranks)
    g = torch.Generator().manual_seed(11)
    xs = [torch.randint(-128, 128, (numel,), generator=g, dtype=torch.int16).to(torch.int8).cuda() for _ in range(ranks)]
    scale = (0.01 + 0.02 * torch.rand(scale_count, generator=g)).to(dtype).cuda()
    offset = 3.0
    for _ in range(3):
        outs = world.run(lambda c, r: txr.collectives.all_reduce_quant(c, xs[r], scale, offset))
        world.check()
    ref = torch.zeros(numel, dtype=torch.float32)
    sc = scale.float().cpu().repeat(numel // scale_count)
    for x in xs:
        ref += (x.cpu().float() + offset) * sc
    ref = ref.to(dtype)
    for o in outs:
        assert o.dtype == dtype
        assert torch.equal(o.cpu(), ref), (o.cpu().float() - ref.float()).abs().max()
    world.destroy()


@pytest.mark.parametrize("ranks,rows,width,dtype", [
    (2, 7, 64, torch.bfloat16), (4, 129, 4 * 24, torch.float32), (8, 1024, 8 * 128, torch.bfloat16), (4, 3000, 4 * 1024, torch.float16),
])
def test_all_to_all_transpose(txr, ranks, rows, width, dtype):
    """Rank p receives column block p of every rank's [rows, width] matrix."""
    world = _world(txr, ranks)
    g = torch.Generator().manual_seed(23)
    xs = [torch.randn(rows, width, generator=g).to(dtype).cuda() for _ in range(ranks)]
    for _ in range(3):
        outs = world.run(lambda c, r: txr.collectives.all_to_all_transpose(c, xs[r]))
        world.check()
    burst = width // ranks
    for r, o in enumerate(outs):
        assert o.shape == (ranks, rows, burst)
        for s in range(ranks):
            assert torch.equal(o[s], xs[s][:, r * burst:(r + 1) * burst]), (r, s)
    world.destroy()
