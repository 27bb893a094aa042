"""The vLLM communicator patch with a fake communicator: gating, fallback and route counters."""
import torch

from tilexr_b200.integrations import vllm_collectives as vc


class FakeCommunicator:
    def all_reduce(self, t):
        return ("stock", t)

    def all_gather(self, t, dim=-1):
        return ("stock", t)

    def reduce_scatter(self, t, dim=-1):
        return ("stock", t)

    def broadcast(self, t, src=0):
        return ("stock", t)


def test_patch_falls_back_for_cpu_tensors_and_counts(monkeypatch):
    vc.route_counters.clear()
    assert vc.patch_communicator(FakeCommunicator, get_comm=lambda self, t: None)
    assert vc.patch_communicator(FakeCommunicator, get_comm=lambda self, t: None)     # idempotent
    c = FakeCommunicator()
    x = torch.ones(4)
    monkeypatch.delenv(vc.ENV_GATE, raising=False)
    assert c.all_reduce(x)[0] == "stock"
    monkeypatch.setenv(vc.ENV_GATE, "1")
    assert c.all_gather(x, 0)[0] == "stock"          # CPU tensor: not eligible
    assert vc.route_counters["all_reduce"]["fallback"] == 1
    assert vc.route_counters["all_gather"]["fallback"] == 1
    assert vc.route_counters["all_gather"]["tilexr"] == 0


def test_errors_in_the_fast_path_fall_back(monkeypatch):
    class Cuda(torch.Tensor):
        @property
        def is_cuda(self):
            return True

    class Comm2:
        def all_reduce(self, t):
            return "stock"

    def boom(self, t):
        raise RuntimeError("no communicator")

    vc.route_counters.clear()
    vc.patch_communicator(Comm2, get_comm=boom)
    monkeypatch.setenv(vc.ENV_GATE, "1")
    t = torch.ones(2).as_subclass(Cuda)
    assert Comm2().all_reduce(t) == "stock"
    assert vc.route_counters["all_reduce"]["error"] == 1


def test_autopatch_without_vllm_gate(monkeypatch):
    monkeypatch.delenv(vc.ENV_GATE, raising=False)
    assert vc.autopatch() is False


def test_adapter_returns_none_where_the_fast_path_does_not_apply(monkeypatch):
    """None means "use your own path": gate off, CPU tensor, non-contiguous, ragged sizes, different dimensions, an error."""

    class Cuda(torch.Tensor):
        @property
        def is_cuda(self):
            return True

    class FakeComm:
        rank, world_size = 0, 2

    a = vc.TileXRVllmCollectivesAdapter(FakeComm())
    x = torch.ones(4, 4)
    monkeypatch.delenv(vc.ENV_GATE, raising=False)
    assert a.should_fallback(x.as_subclass(Cuda))                     # gate off
    monkeypatch.setenv(vc.ENV_GATE, "1")
    assert a.should_fallback(None) and a.should_fallback(x)            # nothing, CPU tensor
    assert a.should_fallback(x.t().as_subclass(Cuda))                  # not contiguous
    t = x.as_subclass(Cuda)
    assert not a.should_fallback(t)
    assert a.should_fallback(t, scatter_sizes=[1, 3]) and a.all_to_all(t, 0, 0, scatter_sizes=[1, 3]) is None
    assert a.all_to_all(t, 0, 1) is None and a.last_error is None      # different dimensions: not an error, just not ours
    monkeypatch.setattr(vc, "all_reduce", lambda comm, tensor: (_ for _ in ()).throw(RuntimeError("no device")))
    assert a.all_reduce(t) is None and isinstance(a.last_error, RuntimeError)
    monkeypatch.setattr(vc, "all_gather", lambda comm, tensor, dim: ("fast", dim))
    assert a.all_gather(t, 1) == ("fast", 1) and a.last_error is None
    err = vc.TileXRCollectivesError("TileXRAllReduce", 3, "bad count")
    assert err.ret == 3 and "TileXRAllReduce" in str(err)


def test_smoke_values_have_the_closed_forms_the_checks_use():
    """The smoke tool's expected values against the collectives stated with torch on the CPU."""
    from tilexr_b200.tools import vllm_collectives_smoke as sm

    world, n, dt = 4, 35, torch.float32
    xs = [sm.make_values(r, n, dt) for r in range(world)]
    assert torch.equal(sm.expected_all_reduce(world, n, dt), sum(xs))
    assert torch.equal(sm.expected_all_gather(world, n, dt), torch.cat(xs))
    big = [sm.make_values(r, n * world, dt) for r in range(world)]
    total = sum(big)
    for r in range(world):
        assert torch.equal(sm.expected_reduce_scatter(world, r, n, dt), total[r * n:(r + 1) * n])
        assert torch.equal(sm.expected_all_to_all(world, r, n, dt), torch.cat([big[s][r * n:(r + 1) * n] for s in range(world)]))
    assert torch.equal(sm.expected_broadcast(2, n, dt), xs[2])
