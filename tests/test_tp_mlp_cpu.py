"""The sequence-parallel MLP layer against a dense feed-forward, with the fused GEMMs replaced by plain PyTorch over a
simulated world (the kernels themselves are tested on the GPU in tests/test_gpu_gemm.py): sharding of the weights, the order
of gate and up columns, the rows each rank ends with."""
import pytest
import torch

from tilexr_b200.models.tp_mlp import SequenceParallelMLP, TPMlpConfig, shard_weights


class World:
    """Ranks of one process: the fake ops need every rank's operands to compute a rank's result."""

    def __init__(self, n):
        self.n = n
        self.x = [None] * n
        self.act = [None] * n
        self.w2 = [None] * n


class FakeComm:
    def __init__(self, world, rank):
        self.world, self.rank, self.world_size = world, rank, world.n

    def symm_empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype)


class FakeOps:
    """all_gather_matmul / matmul_reduce_scatter with the semantics of tilexr_b200.ops.gemm, computed in fp32."""

    def __init__(self, world):
        self.world = world

    def all_gather_matmul(self, comm, a_shard, b, staging):
        full = torch.cat([x.float() for x in self.world.x])
        assert torch.equal(self.world.x[comm.rank], a_shard) and staging.shape[0] == full.shape[0]
        return (full @ b.float().t()).to(a_shard.dtype)

    def matmul_reduce_scatter(self, comm, a, b, staging):
        total = sum(self.world.act[r].float() @ self.world.w2[r].float().t() for r in range(self.world.n))
        rows = total.shape[0] // self.world.n
        return total[comm.rank * rows:(comm.rank + 1) * rows].to(a.dtype)


@pytest.mark.parametrize("ranks", [1, 2, 4])
def test_layer_matches_a_dense_feed_forward(ranks):
    g = torch.Generator().manual_seed(5)
    T, H, F = 32, 16, 24
    x = torch.randn(T, H, generator=g)
    wg, wu, wd = torch.randn(F, H, generator=g) * 0.3, torch.randn(F, H, generator=g) * 0.3, torch.randn(H, F, generator=g) * 0.3
    want = (torch.nn.functional.silu(x @ wg.t()) * (x @ wu.t())) @ wd.t()
    world = World(ranks)
    cfg = TPMlpConfig(hidden=H, ffn=F, tokens=T, dtype=torch.float32)
    layers = []
    rows = T // ranks
    for r in range(ranks):
        w13, w2 = shard_weights(wg, wu, wd, r, ranks)
        assert w13.shape == (2 * F // ranks, H) and w2.shape == (H, F // ranks)
        world.w2[r] = w2
        world.x[r] = x[r * rows:(r + 1) * rows].contiguous()
        layers.append(SequenceParallelMLP(FakeComm(world, r), cfg, w13, w2, ops=FakeOps(world)))
    # the first GEMM and the activation of every rank, then the second GEMM (it needs every rank's activation)
    for r in range(ranks):
        gu = layers[r].ops.all_gather_matmul(layers[r].comm, world.x[r], layers[r].w13, layers[r].stage_rows)
        f = F // ranks
        world.act[r] = torch.nn.functional.silu(gu[:, :f]) * gu[:, f:]
    for r in range(ranks):
        y = layers[r](world.x[r])
        assert y.shape == (rows, H)
        assert torch.allclose(y, want[r * rows:(r + 1) * rows], rtol=1e-4, atol=1e-4)


def test_shapes_are_checked():
    world = World(2)
    comm = FakeComm(world, 0)
    cfg = TPMlpConfig(hidden=16, ffn=24, tokens=32, dtype=torch.float32)
    with pytest.raises(ValueError):
        SequenceParallelMLP(comm, cfg, torch.zeros(24, 16), torch.zeros(16, 10), ops=FakeOps(world))
    with pytest.raises(ValueError):
        SequenceParallelMLP(comm, TPMlpConfig(hidden=16, ffn=25, tokens=32), torch.zeros(24, 16), torch.zeros(16, 12), ops=FakeOps(world))
    with pytest.raises(ValueError):
        shard_weights(torch.zeros(25, 16), torch.zeros(25, 16), torch.zeros(16, 25), 0, 2)
    layer = SequenceParallelMLP(comm, cfg, torch.zeros(24, 16), torch.zeros(16, 12), ops=FakeOps(world))
    with pytest.raises(ValueError):
        layer(torch.zeros(8, 16))
    with pytest.raises(ValueError):
        SequenceParallelMLP(comm, TPMlpConfig(hidden=16, ffn=24, tokens=32, fp8_block=True), torch.zeros(24, 16), torch.zeros(16, 12), ops=FakeOps(world),
                            quant_ops=object())
