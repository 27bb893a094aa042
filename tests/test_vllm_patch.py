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
