"""vLLM integration: tensor-level collectives with vLLM's calling conventions and a patch that
routes ``CudaCommunicator`` through them.

Mirrors the reference's vLLM-Ascend glue (integrations/vllm_ascend/tilexr_collectives/
torch_collectives.py:22-233, vllm_adapter.py:13-117, vllm_patch.py:14-120): an environment
gate, one cached runtime per (rank, world, prefix, device), a fallback to the original
communicator method whenever the fast path does not apply (not CUDA, uneven sizes, any error),
and per-method route counters (``tilexr`` / ``fallback`` / ``error``).
"""
from __future__ import annotations

import functools
import os
from collections import defaultdict
from typing import Callable, Dict, Optional

import torch

ENV_GATE = "VLLM_TILEXR_COLLECTIVES"
ENV_TRACE = "TILEXR_VLLM_TRACE"

route_counters: Dict[str, Dict[str, int]] = defaultdict(lambda: {"tilexr": 0, "fallback": 0, "error": 0})


ENV_GATE_REFERENCE = "VLLM_ASCEND_TILEXR_COLLECTIVES"      # the reference's name for the same gate: honoured too


def enabled() -> bool:
    return any(os.environ.get(name, "0").strip().lower() not in ("", "0", "false", "no", "off") for name in (ENV_GATE, ENV_GATE_REFERENCE))


def _trace(msg: str) -> None:
    if os.environ.get(ENV_TRACE, "0") not in ("", "0"):
        print(f"[tilexr-vllm] {msg}", flush=True)


@functools.lru_cache(maxsize=None)
def _runtime(rank: int, world_size: int, prefix: str, device_index: int, group_id: int):
    """One communicator per (rank, world, prefix, device).  ``group_id`` is ``id()`` of the
    process group the caller uses, so that different groups get different communicators."""
    import tilexr_b200 as txr

    group = _GROUPS.get(group_id)
    return txr.init_from_torch_distributed(group=group, device=device_index, domain=abs(hash(prefix)) % 1000)


_GROUPS: Dict[int, object] = {}


def runtime_for(group, device: torch.device, prefix: str = "vllm"):
    import torch.distributed as dist

    _GROUPS[id(group)] = group
    return _runtime(dist.get_rank(group), dist.get_world_size(group), prefix, device.index or 0, id(group))


def _front(t: torch.Tensor, dim: int) -> torch.Tensor:
    return t.movedim(dim, 0).contiguous()


def all_reduce(comm, t: torch.Tensor) -> torch.Tensor:
    import tilexr_b200 as txr

    return txr.all_reduce(comm, t.contiguous()).view_as(t)


def all_gather(comm, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """vLLM semantics: the gathered pieces are concatenated along ``dim``."""
    import tilexr_b200 as txr

    dim = dim % t.dim()
    world = comm.world_size
    gathered = txr.all_gather(comm, t.contiguous())                    # [world, *t.shape]
    out = gathered.movedim(0, dim)                                     # [..., world, size_dim, ...]
    shape = list(t.shape)
    shape[dim] *= world
    return out.reshape(shape)


def reduce_scatter(comm, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
    import tilexr_b200 as txr

    dim = dim % t.dim()
    if t.shape[dim] % comm.world_size != 0:
        raise ValueError("reduce_scatter: the scattered dimension must divide by the world size")
    moved = _front(t, dim)
    out = txr.reduce_scatter(comm, moved)
    return out.movedim(0, dim).contiguous()


def broadcast(comm, t: torch.Tensor, root: int = 0) -> torch.Tensor:
    import tilexr_b200 as txr

    if t.is_contiguous():
        return txr.broadcast(comm, t, root)
    buf = t.contiguous()
    txr.broadcast(comm, buf, root)
    t.copy_(buf)
    return t


def all_to_all(comm, t: torch.Tensor, scatter_dim: int = 0, gather_dim: int = 0) -> torch.Tensor:
    """Equal split; only ``scatter_dim == gather_dim`` is supported, like the reference glue."""
    import tilexr_b200 as txr

    scatter_dim %= t.dim()
    gather_dim %= t.dim()
    if scatter_dim != gather_dim:
        raise ValueError("all_to_all: scatter_dim must equal gather_dim")
    if t.shape[scatter_dim] % comm.world_size != 0:
        raise ValueError("all_to_all: the split dimension must divide by the world size")
    moved = _front(t, scatter_dim)
    out = txr.all_to_all(comm, moved)
    return out.movedim(0, scatter_dim).contiguous()


class TileXRCollectivesError(RuntimeError):
    """A collective of this library refused its arguments or failed on the device."""

    def __init__(self, operation: str, ret: int, detail: str = ""):
        super().__init__(f"{operation} failed with {ret}" + (f": {detail}" if detail else ""))
        self.operation, self.ret, self.detail = operation, ret, detail


class TileXRVllmCollectivesAdapter:
    """The collectives with "None means use your own path" semantics, for callers that keep their stock implementation
    beside this one (the reference's adapter: integrations/vllm_ascend/tilexr_collectives/vllm_adapter.py:34-117).
    Every method returns the result, or None when the fast path does not apply (gate off, not a contiguous CUDA tensor,
    uneven split sizes, different scatter and gather dimensions) or raised; the exception is kept in ``last_error``."""

    def __init__(self, comm):
        self.comm = comm
        self.rank, self.world_size = comm.rank, comm.world_size
        self.last_error: Optional[BaseException] = None

    def should_fallback(self, tensor=None, *, scatter_sizes=None, gather_sizes=None) -> bool:
        self.last_error = None
        if not enabled() or tensor is None or not getattr(tensor, "is_cuda", False):
            return True
        contiguous = getattr(tensor, "is_contiguous", None)
        if not callable(contiguous) or not contiguous():
            return True
        return scatter_sizes is not None or gather_sizes is not None      # ragged exchanges stay on the stock path

    def _try(self, fn: Callable):
        try:
            return fn()
        except (OSError, RuntimeError, TypeError, ValueError) as exc:
            self.last_error = exc
            return None

    def all_reduce(self, input_):
        return None if self.should_fallback(input_) else self._try(lambda: all_reduce(self.comm, input_))

    def all_gather(self, input_, dim: int = -1):
        return None if self.should_fallback(input_) else self._try(lambda: all_gather(self.comm, input_, dim))

    def reduce_scatter(self, input_, dim: int = -1):
        return None if self.should_fallback(input_) else self._try(lambda: reduce_scatter(self.comm, input_, dim))

    def broadcast(self, tensor, src: int = 0):
        return None if self.should_fallback(tensor) else self._try(lambda: broadcast(self.comm, tensor, src))

    def all_to_all(self, input_, scatter_dim: int = 0, gather_dim: int = -1, scatter_sizes=None, gather_sizes=None):
        if self.should_fallback(input_, scatter_sizes=scatter_sizes, gather_sizes=gather_sizes):
            return None
        try:
            if scatter_dim % input_.dim() != gather_dim % input_.dim():
                return None
        except (AttributeError, TypeError, ZeroDivisionError) as exc:
            self.last_error = exc
            return None
        return self._try(lambda: all_to_all(self.comm, input_, scatter_dim, gather_dim))


def _wrap(name: str, fast: Callable, original: Callable, get_comm: Callable):
    def method(self, tensor, *args, **kwargs):
        counters = route_counters[name]
        if not enabled() or not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
            counters["fallback"] += 1
            return original(self, tensor, *args, **kwargs)
        try:
            comm = get_comm(self, tensor)
            out = fast(comm, tensor, *args, **kwargs)
            counters["tilexr"] += 1
            _trace(f"{name}: tilexr {tuple(tensor.shape)}")
            return out
        except Exception as exc:  # any problem falls back to the stock path
            counters["error"] += 1
            _trace(f"{name}: error {exc!r}, falling back")
            return original(self, tensor, *args, **kwargs)

    method.__name__ = name
    method._tilexr_patched = True
    return method


def patch_communicator(communicator_cls=None, get_comm: Optional[Callable] = None) -> bool:
    """Patches ``all_reduce``, ``all_gather``, ``reduce_scatter``, ``broadcast`` and (where the class has one) ``all_to_all`` of vLLM's
    ``CudaCommunicator`` (or of ``communicator_cls``).  Returns False when vLLM is absent."""
    if communicator_cls is None:
        try:
            from vllm.distributed.device_communicators.cuda_communicator import CudaCommunicator as communicator_cls
        except Exception:
            return False
    if get_comm is None:
        def get_comm(self, tensor):
            return runtime_for(self.device_group, tensor.device, getattr(self, "unique_name", "vllm"))
    def equal_all_to_all(comm, t, scatter_dim: int = 0, gather_dim: int = -1, scatter_sizes=None, gather_sizes=None):
        if scatter_sizes is not None or gather_sizes is not None:
            raise ValueError("ragged all_to_all stays on the stock path")
        return all_to_all(comm, t, scatter_dim, gather_dim)

    table = {"all_reduce": all_reduce, "all_gather": all_gather, "reduce_scatter": reduce_scatter, "broadcast": broadcast,
             "all_to_all": equal_all_to_all}
    for name, fast in table.items():
        original = getattr(communicator_cls, name, None)
        if original is None or getattr(original, "_tilexr_patched", False):
            continue
        setattr(communicator_cls, name, _wrap(name, fast, original, get_comm))
    return True


def autopatch() -> bool:
    """What a ``sitecustomize`` hook calls: patch when the gate is set."""
    return patch_communicator() if enabled() else False
