"""tcgen05 GEMM and its all-gather / reduce-scatter fusions against an fp32 PyTorch matmul."""
import pytest
import torch

from conftest import require_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def txr():
    require_cuda()
    import tilexr_b200

    return tilexr_b200


def _close(got, want, k):
    got, want = got.float().cpu(), want.float().cpu()
    tol = 2e-2 * max(1.0, (k ** 0.5) / 8)
    assert torch.allclose(got, want, rtol=2e-2, atol=tol), (got - want).abs().max()
    assert (got - want).abs().mean() < 0.02 * want.abs().mean() + 1e-3


@pytest.mark.parametrize("m,n,k,dtype", [
    (128, 256, 64, torch.bfloat16),
    (512, 512, 256, torch.bfloat16),
    (300, 264, 200, torch.bfloat16),        # ragged in every dimension
    (2048, 2048, 1024, torch.float16),
    (1024, 7168, 2048, torch.bfloat16),     # more tiles than SMs: both accumulator buffers, ring wrap
])
def test_matmul(txr, m, n, k, dtype):
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * 0.5).to(dtype).cuda()
    b = (torch.randn(n, k, generator=g) * 0.5).to(dtype).cuda()
    for _ in range(2):
        c = txr.gemm.matmul(a, b)
    torch.cuda.synchronize()
    _close(c, a.float() @ b.float().t(), k)


@pytest.mark.parametrize("m,n,k,fmt", [
    (256, 256, 128, torch.float8_e4m3fn),
    (1000, 520, 400, torch.float8_e4m3fn),      # ragged in every dimension
    (2048, 4096, 2048, torch.float8_e5m2),
    (4096, 2048, 7168, torch.float8_e4m3fn),    # more tiles than CTA pairs, long K
])
def test_matmul_fp8(txr, m, n, k, fmt):
    """fp8 operands on the kind::f8f6f4 tensor-core path against an fp32 product of the same fp8 values."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(fmt).cuda()
    b = torch.randn(n, k, generator=g).to(fmt).cuda()
    alpha = 0.37
    for _ in range(2):
        c = txr.gemm.matmul_fp8(a, b, alpha)
    torch.cuda.synchronize()
    want = alpha * (a.float() @ b.float().t())
    got = c.float()
    # fp32 accumulation of exact fp8 products: only the final bf16 rounding differs
    assert torch.allclose(got, want, rtol=1e-2, atol=1e-2 * (k ** 0.5)), (got - want).abs().max()
    assert (got - want).abs().mean() < 4e-3 * want.abs().mean() + 1e-4


@pytest.mark.parametrize("ranks,shard_rows,n,k", [(2, 128, 256, 256), (2, 256, 512, 1024), (4, 128, 768, 512), (4, 512, 1024, 512)])
def test_all_gather_matmul(txr, ranks, shard_rows, n, k):
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    g = torch.Generator().manual_seed(7)
    shards = [(torch.randn(shard_rows, k, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(ranks)]
    bs = [(torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(ranks)]
    staging = world.symm_empty((ranks * shard_rows, k), torch.bfloat16)
    full = torch.cat(shards).float()
    for _ in range(3):
        outs = world.run(lambda c, r: txr.gemm.all_gather_matmul(c, shards[r], bs[r], staging[r]))
        world.check()
    for r in range(ranks):
        _close(outs[r], full @ bs[r].float().t(), k)
    world.destroy()


@pytest.mark.parametrize("ranks,shard_rows,n,k", [(2, 128, 256, 128), (2, 256, 512, 512), (4, 128, 512, 256), (4, 512, 1024, 768)])
def test_matmul_reduce_scatter(txr, ranks, shard_rows, n, k):
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    g = torch.Generator().manual_seed(9)
    m = ranks * shard_rows
    a = [(torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(ranks)]
    b = [(torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(ranks)]
    staging = world.symm_empty((m, n), torch.bfloat16)
    # partial products travel as bf16 and are summed in rank order in fp32
    partial = [(a[r].float() @ b[r].float().t()).to(torch.bfloat16).float() for r in range(ranks)]
    want = partial[0]
    for p in partial[1:]:
        want = want + p
    for _ in range(3):
        outs = world.run(lambda c, r: txr.gemm.matmul_reduce_scatter(c, a[r], b[r], staging[r]))
        world.check()
    for r in range(ranks):
        _close(outs[r], want[r * shard_rows:(r + 1) * shard_rows], k * ranks)
    world.destroy()


def test_matmul_all_reduce(txr):
    """GEMM with the reduce-scatter in its epilogue, then an all-gather of the reduced shards: every rank ends with the sum."""
    ranks, shard_rows, n, k = 2, 128, 256, 256
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    g = torch.Generator().manual_seed(21)
    m = ranks * shard_rows
    a = [(torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(ranks)]
    b = [(torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(ranks)]
    staging = world.symm_empty((m, n), torch.bfloat16)
    want = sum((a[r].float() @ b[r].float().t()).to(torch.bfloat16).float() for r in range(ranks))
    for _ in range(2):
        outs = world.run(lambda c, r: txr.gemm.matmul_all_reduce(c, a[r], b[r], staging[r]))
        world.check()
    for r in range(ranks):
        _close(outs[r], want, k * ranks)
    world.destroy()


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 256, 512), (300, 384, 1024), (1024, 2048, 7168), (96, 128, 256)])
def test_matmul_fp8_block_scaled(txr, m, n, k):
    """Block-scaled fp8 (1 x 128 activation scales, 128 x 128 weight scales, fp32) against the fp32 product of the
    dequantised operands.  Rows are given very different magnitudes, and so are the weight blocks, so that a scale
    applied to the wrong row, column group or block of K shows."""
    from tilexr_b200.utils import oracle

    g = torch.Generator().manual_seed(31)
    a = torch.randn(m, k, generator=g) * (0.25 + 4.0 * torch.rand(m, 1, generator=g)) * (0.5 + torch.rand(1, k // 128, generator=g)).repeat_interleave(128, dim=1)
    w = torch.randn(n, k, generator=g) * 0.5
    nb = (n + 127) // 128
    w = w * (0.2 + 3.0 * torch.rand(nb, k // 128, generator=g)).repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)
    qa, sa = txr.quant.fp8_quant_1x128(a.to(torch.bfloat16).cuda())
    qw, sw = txr.gemm.quantize_weight_128x128(w.cuda())
    got = txr.gemm.matmul_fp8_block(qa, sa, qw, sw).float().cpu()
    torch.cuda.synchronize()
    da = oracle.fp8_dequant_1x128_ref(qa.cpu(), sa.cpu())
    dw = qw.cpu().float().view(-1, k) * sw.cpu().repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)
    want = da @ dw.t()
    assert torch.allclose(got, want, rtol=1e-2, atol=1e-2 * want.abs().max().item()), (got - want).abs().max()
    assert (got - want).abs().mean() < 4e-3 * want.abs().mean() + 1e-4


@pytest.mark.parametrize("counts,n,k,swiglu", [
    ([300, 0, 17, 256, 1, 700], 512, 256, False),          # empty group, groups smaller and larger than a tile, ragged starts
    ([300, 0, 17, 256, 1, 700], 512, 256, True),
    ([5] * 70, 264, 128, False),                             # more groups than one launch holds, N not a multiple of the tile
    ([2000, 3000, 100, 4000], 4096, 1024, True),             # more tiles than CTA pairs
])
def test_grouped_matmul(txr, counts, n, k, swiglu):
    """One launch over all groups, row counts read on the device, against fp32 PyTorch; rows past the counts untouched."""
    g = torch.Generator().manual_seed(sum(counts) + n)
    total = sum(counts)
    rows = (torch.randn(total + 40, k, generator=g) * 0.5).to(torch.bfloat16).cuda()
    w = (torch.randn(len(counts), n, k, generator=g) * 0.2).to(torch.bfloat16).cuda()
    group_rows = torch.tensor(counts, dtype=torch.int64).cuda()
    epi = txr.gemm.EPILOGUE_SWIGLU if swiglu else txr.gemm.EPILOGUE_STORE
    out = torch.full((total + 40, n // 2 if swiglu else n), 7.0, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        got = txr.gemm.grouped_matmul(rows, w, group_rows, epilogue=epi, out=out)
    torch.cuda.synchronize()
    want = txr.gemm.grouped_matmul_ref(rows, w, group_rows, epi)
    _close(got[:total], want[:total], k)
    assert torch.all(got[total:] == 7.0)


def _block_operands(txr, rows, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(rows, k, generator=g) * (0.25 + 4.0 * torch.rand(rows, 1, generator=g))
    w = torch.randn(n, k, generator=g) * 0.5
    qa, sa = txr.quant.fp8_quant_1x128(a.to(torch.bfloat16).cuda())
    qw, sw = txr.gemm.quantize_weight_128x128(w.cuda())
    return qa, sa, qw, sw


def _block_product(qa, sa, qw, sw):
    k = qa.shape[1]
    da = qa.float().cpu().view(qa.shape[0], k // 128, 128) * sa.cpu().unsqueeze(-1)
    dw = qw.float().cpu() * sw.cpu().repeat_interleave(128, dim=0)[:qw.shape[0]].repeat_interleave(128, dim=1)
    return da.view(qa.shape[0], k) @ dw.t()


@pytest.mark.parametrize("ranks,shard_rows,n,k", [(2, 256, 256, 512), (2, 512, 640, 1024), (4, 256, 512, 1536)])
def test_all_gather_matmul_fp8_block(txr, ranks, shard_rows, n, k):
    """Block-scaled fp8 GEMM fused with the all-gather of A: every rank's rows AND scales travel into the others' staging
    buffers during the launch; three launches in a row reuse the buffers behind the reuse guard."""
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    ops = [_block_operands(txr, shard_rows, n, k, 50 + r) for r in range(ranks)]
    a_staging = world.symm_empty((ranks * shard_rows, k), torch.float8_e4m3fn)
    s_staging = world.symm_empty((ranks * shard_rows, k // 128), torch.float32)
    for _ in range(3):
        outs = world.run(lambda c, r: txr.gemm.all_gather_matmul_fp8_block(c, ops[r][0], ops[r][1], a_staging[r], s_staging[r], ops[r][2], ops[r][3]))
        world.check()
    qa_all = torch.cat([o[0] for o in ops])
    sa_all = torch.cat([o[1] for o in ops])
    for r in range(ranks):
        want = _block_product(qa_all, sa_all, ops[r][2], ops[r][3])
        got = outs[r].float().cpu()
        assert torch.allclose(got, want, rtol=1e-2, atol=1e-2 * want.abs().max().item()), (got - want).abs().max()
        assert (got - want).abs().mean() < 4e-3 * want.abs().mean() + 1e-4
    world.destroy()


@pytest.mark.parametrize("ranks,shard_rows,n,k", [(2, 256, 256, 256), (2, 256, 768, 1024), (4, 256, 512, 512)])
def test_matmul_reduce_scatter_fp8_block(txr, ranks, shard_rows, n, k):
    """Block-scaled fp8 GEMM fused with the reduce-scatter of its result: partial tiles travel as bf16 and are added in
    rank order in fp32."""
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    m = ranks * shard_rows
    ops = [_block_operands(txr, m, n, k, 70 + r) for r in range(ranks)]
    staging = world.symm_empty((m, n), torch.bfloat16)
    partial = [_block_product(*ops[r]).to(torch.bfloat16).float() for r in range(ranks)]
    want = partial[0]
    for p in partial[1:]:
        want = want + p
    for _ in range(3):
        outs = world.run(lambda c, r: txr.gemm.matmul_reduce_scatter_fp8_block(c, ops[r][0], ops[r][1], ops[r][2], ops[r][3], staging[r]))
        world.check()
    for r in range(ranks):
        got = outs[r].float().cpu()
        ref = want[r * shard_rows:(r + 1) * shard_rows]
        assert torch.allclose(got, ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item()), (got - ref).abs().max()
        assert (got - ref).abs().mean() < 6e-3 * ref.abs().mean() + 1e-4
    world.destroy()
