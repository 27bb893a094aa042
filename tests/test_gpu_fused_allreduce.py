"""All-reduce + residual add + RMSNorm in one kernel, one-shot and two-shot, against fp32 PyTorch."""
import pytest
import torch

from conftest import require_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def txr():
    require_cuda()
    import tilexr_b200

    return tilexr_b200


def _reference(xs, residual, gamma, eps):
    acc = xs[0].float()
    for x in xs[1:]:
        acc = acc + x.float()
    if residual is not None:
        acc = acc + residual.float()
    s = acc.to(xs[0].dtype)
    xf = s.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(xs[0].dtype)
    return y, s


@pytest.mark.parametrize("ranks,rows,h,algo,with_res,symmetric", [
    (2, 1, 8192, 1, True, False),
    (8, 16, 8192, 1, True, False),
    (4, 256, 4096, 1, False, False),
    (4, 64, 8192, 2, True, False),
    (8, 203, 2048, 2, True, False),       # rows do not divide by the rank count
    (4, 128, 8192, 2, True, True),        # peers write y and the residual directly
    (8, 37, 1024, 0, True, False),
    (8, 1, 2048, 2, True, False),         # two-shot with fewer rows than ranks: most ranks own nothing
    (8, 3, 1024, 2, True, True),
])
def test_all_reduce_rmsnorm(txr, ranks, rows, h, algo, with_res, symmetric):
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=64)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(rows, h, generator=g).to(torch.bfloat16) for _ in range(ranks)]
    res = torch.randn(rows, h, generator=g).to(torch.bfloat16) if with_res else None
    gamma = (1 + 0.1 * torch.randn(h, generator=g)).to(torch.bfloat16)
    want_y, want_res = _reference(xs, res, gamma, 1e-6)
    xd = [x.cuda() for x in xs]
    gd = gamma.cuda()
    for rep in range(2):
        if symmetric:
            ys = world.symm_empty((rows, h), torch.bfloat16)
            rd = world.symm_empty((rows, h), torch.bfloat16)
            for r in rd:
                r.copy_(res)
        else:
            ys = [None] * ranks
            rd = [res.cuda() if with_res else None for _ in range(ranks)]
        out = world.run(lambda c, r: txr.collectives.all_reduce_rmsnorm(c, xd[r], gd, 1e-6, residual=rd[r], algo=algo, out=ys[r]))
        world.check()
        for r in range(ranks):
            if with_res:
                assert torch.equal(rd[r].cpu(), want_res), f"rank {r} residual"
            got = out[r].cpu().float()
            assert torch.allclose(got, want_y.float(), rtol=2e-2, atol=2e-2)
            assert torch.equal(out[r].cpu(), out[0].cpu())       # bit-identical on every rank
    world.destroy()


def test_choice_by_size(txr):
    assert txr._C.all_reduce_rmsnorm_choose(16 * 1024, 8) == 1
    assert txr._C.all_reduce_rmsnorm_choose(4 << 20, 8) == 2
    assert txr._C.all_reduce_rmsnorm_choose(4 << 20, 2) == 1
