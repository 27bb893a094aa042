"""MoonEP-compatible torch facade over the native five-stage kernels.

``Buffer`` keeps the call signatures of the reference's compatibility layer
(integrations/moonep_torch/tilexr_moonep/compat.py:135-501) so that training code written
against it runs unchanged; ``TileXRMoonEPBuffer`` is the native facade with real remote weight
prefetch and owner-pull gradient reduction (torch_api.py:591-1808).  Differences: there is no
host synchronisation between planning and dispatch (every later stage checks ``plan.status`` on
the device), and the dispatch outputs are persistent symmetric tensors that peers write
directly, so ``dispatch`` returns views that stay valid until the next ``dispatch``.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional

import torch

from .. import _C
from ..ops import collectives


@dataclasses.dataclass
class MoonEPCommPlan:
    dst: torch.Tensor
    experts_to_copy: torch.Tensor
    zero_fill_ranges: torch.Tensor
    remote_stats: torch.Tensor
    N: int
    R: int
    E: int
    B: int
    NvS: int
    K: int
    dup_groups: Optional[torch.Tensor] = None
    dup_loffs: Optional[torch.Tensor] = None
    dup_counts: Optional[torch.Tensor] = None
    status: Optional[torch.Tensor] = None
    dst_local: Optional[torch.Tensor] = None
    cu_seqlens: Optional[torch.Tensor] = None

    def clone(self) -> "MoonEPCommPlan":
        def c(t):
            return None if t is None else t.clone()

        return MoonEPCommPlan(c(self.dst), c(self.experts_to_copy), c(self.zero_fill_ranges), c(self.remote_stats), self.N,
                              self.R, self.E, self.B, self.NvS, self.K, c(self.dup_groups), c(self.dup_loffs),
                              c(self.dup_counts), c(self.status), c(self.dst_local), c(self.cu_seqlens))

    def as_dict(self) -> dict:
        return {"dst": self.dst, "experts_to_copy": self.experts_to_copy, "zero_fill_ranges": self.zero_fill_ranges,
                "remote_stats": self.remote_stats, "dup_counts": self.dup_counts, "status": self.status,
                "dst_local": self.dst_local, "cu_seqlens": self.cu_seqlens, "N": self.N, "R": self.R, "E": self.E,
                "B": self.B, "NvS": self.NvS, "K": self.K}

    @staticmethod
    def from_dict(d: dict) -> "MoonEPCommPlan":
        return MoonEPCommPlan(d["dst"], d["experts_to_copy"], d["zero_fill_ranges"], d["remote_stats"], d["N"], d["R"], d["E"],
                              d["B"], d["NvS"], d["K"], None, None, d["dup_counts"], d["status"], d["dst_local"], d["cu_seqlens"])


    # -- a plan on disk: the routing of a step, to dispatch again later without planning (a plan holds no pointers) -----------
    _TENSORS = ("dst", "experts_to_copy", "zero_fill_ranges", "remote_stats", "dup_groups", "dup_loffs", "dup_counts", "status", "dst_local",
                "cu_seqlens")
    _SHAPE = ("N", "R", "E", "B", "NvS", "K")
    FILE_VERSION = 1

    def save(self, path: str) -> None:
        """Writes every table of the plan (on the CPU) and its shape.  Wait for the planning kernel first: the tables are read
        as they are."""
        doc = {"version": self.FILE_VERSION, "shape": {k: int(getattr(self, k)) for k in self._SHAPE},
               "tensors": {k: (None if getattr(self, k) is None else getattr(self, k).detach().cpu()) for k in self._TENSORS}}
        torch.save(doc, path)

    @classmethod
    def load(cls, path: str, device=None, expect: Optional[dict] = None) -> "MoonEPCommPlan":
        """Reads a plan written by `save`, checks that its tables have the sizes its shape implies and, with `expect`
        (a dict of N / R / E / B / NvS / K), that it was made for this buffer; moves the tables to `device`."""
        doc = torch.load(path, map_location="cpu", weights_only=True)
        if not isinstance(doc, dict) or doc.get("version") != cls.FILE_VERSION:
            raise TileXRMoonEPError(f"{path}: not a plan file of version {cls.FILE_VERSION}")
        shape, t = doc["shape"], doc["tensors"]
        for k, want in (expect or {}).items():
            if int(shape[k]) != int(want):
                raise TileXRMoonEPError(f"{path}: the plan was made for {k} = {shape[k]}, this buffer has {want}")
        sizes = {"dst": shape["N"], "experts_to_copy": shape["R"] * shape["B"], "dst_local": shape["NvS"]}
        for k, n in sizes.items():
            if t.get(k) is not None and t[k].numel() != n:
                raise TileXRMoonEPError(f"{path}: table {k} has {t[k].numel()} entries, its shape implies {n}")
        if t.get("dst") is None or t.get("experts_to_copy") is None:
            raise TileXRMoonEPError(f"{path}: the plan has no destination table")
        move = (lambda x: x) if device is None else (lambda x: None if x is None else x.to(device))
        return cls(*[move(t.get(k)) for k in ("dst", "experts_to_copy", "zero_fill_ranges", "remote_stats")], *[int(shape[k]) for k in cls._SHAPE],
                   *[move(t.get(k)) for k in ("dup_groups", "dup_loffs", "dup_counts", "status", "dst_local", "cu_seqlens")])


class TileXRMoonEPError(RuntimeError):
    """A native MoonEP call refused its arguments or a stage failed on the device."""


STAGE_BITS = {"planning": 1 << 0, "dispatch": 1 << 1, "prefetch_weight": 1 << 2, "combine": 1 << 3, "reduce_grad": 1 << 4}


@dataclasses.dataclass(frozen=True)
class NativeCapabilities:
    """What the native library serves itself (reference: integrations/moonep_torch/tilexr_moonep/runtime.py:54-112):
    ``stage_mask`` has a bit per stage with a kernel of its own, ``stub_mask`` a bit per stage that only has a stand-in."""
    abi_version: int
    stage_mask: int
    stub_mask: int

    @staticmethod
    def query() -> "NativeCapabilities":
        abi, native, stub = _C.moonep_capabilities()
        return NativeCapabilities(int(abi), int(native), int(stub))

    def implementation(self, stage: str) -> str:
        if stage not in STAGE_BITS:
            raise KeyError(f"unknown MoonEP stage: {stage}")
        bit = STAGE_BITS[stage]
        return "stub" if self.stub_mask & bit else "native" if self.stage_mask & bit else "unavailable"

    @property
    def transport_correctness_valid(self) -> bool:
        """Every stage moves its data with a kernel of the library (no stand-in), so a correctness run judges the transport."""
        every = sum(STAGE_BITS.values())
        return (self.stage_mask & every) == every and (self.stub_mask & every) == 0

    @property
    def transport_performance_valid(self) -> bool:
        """Native coverage alone does not make a number publishable: the harness gates on precision and on its sample filter."""
        return False

    def as_dict(self) -> dict:
        return {"abi_version": self.abi_version, "stage_mask": self.stage_mask, "stub_mask": self.stub_mask,
                "implementations": {stage: self.implementation(stage) for stage in STAGE_BITS},
                "transport_correctness_valid": self.transport_correctness_valid,
                "transport_performance_valid": self.transport_performance_valid}


@dataclasses.dataclass
class TileXRMoonEPContext:
    """Shape and placement of one MoonEP instance, with the fields and checks of the reference's context
    (integrations/moonep_torch/tilexr_moonep/torch_api.py:306-590).  ``runtime`` is a communicator of this package
    (``tilexr_b200.init_from_torch_distributed`` or an emulated world's rank); the planner group is the set of ranks that
    plan together (the communicator's ranks), the lane group the tensor-parallel lanes of one expert group.

    One buffer at a time may own a context (``attach_buffer``); a context whose buffer saw a failed stage is poisoned and
    refuses further owners, because the windows' contents are then undefined for the other ranks too."""
    runtime: object
    global_rank: int
    global_world_size: int
    node_rank: int
    node_count: int
    local_rank: int
    local_world_size: int
    planner_group_rank: int
    planner_group_size: int
    lane_group_rank: int
    lane_group_size: int
    device_index: int
    tokens_per_rank: int
    hidden_size: int
    topk: int
    expert_count: int
    dtype: object
    token_padding: int = 1
    prefetch_slots: Optional[int] = None

    def __post_init__(self) -> None:
        self._owner = None
        self._stream = None
        self._poisoned = False
        self._closed = False
        if not 1 <= self.planner_group_size <= 128:
            raise ValueError(f"planner_group_size must be in [1, 128], got {self.planner_group_size}")
        if not 0 <= self.planner_group_rank < self.planner_group_size:
            raise ValueError("planner_group_rank is outside the planner group")
        if self.tokens_per_rank <= 0 or self.hidden_size <= 0 or not 1 <= self.topk <= 32:
            raise ValueError("tokens_per_rank and hidden_size must be positive; topk must be in [1, 32]")
        if self.expert_count <= 0 or self.expert_count % self.planner_group_size != 0:
            raise ValueError("expert_count must be positive and divisible by planner_group_size")
        if self.token_padding <= 0:
            raise ValueError("token_padding must be positive")
        if self.prefetch_slots is None:
            self.prefetch_slots = self.experts_per_rank
        if not 1 <= self.prefetch_slots <= self.experts_per_rank:
            raise ValueError("prefetch_slots must be in [1, E/R]")
        if self.planner_group_size * self.nv_s > 2 ** 31:
            raise OverflowError("the int32 destination encoding needs planner_group_size * NvS <= 2^31")
        rank = getattr(self.runtime, "rank", self.planner_group_rank)
        world = getattr(self.runtime, "world_size", self.planner_group_size)
        if int(rank) != self.planner_group_rank or int(world) != self.planner_group_size:
            raise ValueError("the communicator's rank and size do not match the planner group")

    @property
    def experts_per_rank(self) -> int:
        return self.expert_count // self.planner_group_size

    @property
    def route_count(self) -> int:
        return self.tokens_per_rank * self.topk

    @property
    def nv_s(self) -> int:
        """Rows of a rank's receive buffer: its routes plus the padding behind every local group and slot."""
        return self.route_count + (self.token_padding - 1) * 2 * self.experts_per_rank

    @property
    def dispatched_capacity(self) -> int:
        return self.nv_s

    @classmethod
    def from_env(cls, *, tokens_per_rank: int, hidden_size: int, topk: int, expert_count: int, dtype, token_padding: int = 1,
                 prefetch_slots: Optional[int] = None, runtime=None, buffer_mb: Optional[int] = None) -> "TileXRMoonEPContext":
        """Ranks from the launcher's environment (RANK, WORLD_SIZE, LOCAL_RANK, LOCAL_WORLD_SIZE, NODE_RANK, NODE_COUNT,
        TILEXR_PLANNER_GROUP_RANK / _SIZE, TILEXR_LANE_GROUP_RANK / _SIZE).  Without ``runtime`` a communicator is created
        over the initialised ``torch.distributed`` world."""
        import os

        env = os.environ
        global_rank, global_world = int(env.get("RANK", "0")), int(env.get("WORLD_SIZE", "1"))
        local_rank = int(env.get("LOCAL_RANK", str(global_rank)))
        device = torch.cuda.current_device() if torch.cuda.is_available() else local_rank
        if local_rank != device:
            raise ValueError(f"LOCAL_RANK={local_rank} does not match the current CUDA device {device}")
        group_rank = int(env.get("TILEXR_PLANNER_GROUP_RANK", str(global_rank)))
        group_size = int(env.get("TILEXR_PLANNER_GROUP_SIZE", str(global_world)))
        if runtime is None:
            from ..parallel.comm import init_from_torch_distributed

            per = tokens_per_rank * topk * hidden_size * torch.empty((), dtype=dtype).element_size()
            runtime = init_from_torch_distributed(buffer_mb=buffer_mb if buffer_mb is not None else max(64, int(3 * per / (1 << 20)) + 16))
        return cls(runtime=runtime, global_rank=global_rank, global_world_size=global_world, node_rank=int(env.get("NODE_RANK", "0")),
                   node_count=int(env.get("NODE_COUNT", "1")), local_rank=local_rank,
                   local_world_size=int(env.get("LOCAL_WORLD_SIZE", str(global_world))), planner_group_rank=group_rank,
                   planner_group_size=group_size, lane_group_rank=int(env.get("TILEXR_LANE_GROUP_RANK", "0")),
                   lane_group_size=int(env.get("TILEXR_LANE_GROUP_SIZE", "1")), device_index=int(device),
                   tokens_per_rank=int(tokens_per_rank), hidden_size=int(hidden_size), topk=int(topk), expert_count=int(expert_count),
                   dtype=dtype, token_padding=int(token_padding), prefetch_slots=None if prefetch_slots is None else int(prefetch_slots))

    # -- ownership ---------------------------------------------------------------------------------------
    def attach_buffer(self, owner) -> None:
        if self._closed or self._poisoned:
            raise RuntimeError("this MoonEP context is closed or saw a failed stage; create a new one")
        if self._owner is not None and self._owner is not owner:
            raise RuntimeError("this MoonEP context already belongs to a buffer")
        self._owner = owner

    def detach_buffer(self, owner) -> None:
        if self._owner is owner:
            self._owner = None
            self._stream = None

    def bind_stream(self, owner, stream_ptr: int) -> None:
        """All stages of one buffer run on one stream: the flag epochs of the windows follow that stream's order."""
        if self._owner is not owner:
            raise RuntimeError("only the owning buffer binds a stream")
        if self._stream is not None and self._stream != int(stream_ptr):
            raise RuntimeError("this MoonEP context is bound to another stream; release it first")
        self._stream = int(stream_ptr)

    def release_stream(self, owner) -> None:
        if self._owner is owner:
            self._stream = None

    def mark_poisoned(self) -> None:
        self._poisoned = True

    def capabilities(self) -> NativeCapabilities:
        return NativeCapabilities.query()

    def close(self) -> None:
        if self._closed:
            return
        if self._owner is not None:
            raise RuntimeError("close the owning MoonEP buffer before its context")
        self._closed = True


@dataclasses.dataclass
class DispatchResult:
    hidden: torch.Tensor
    route_weights: Optional[torch.Tensor]
    plan: "MoonEPCommPlan"


@dataclasses.dataclass
class CombineResult:
    hidden: torch.Tensor
    route_weights: Optional[torch.Tensor]


@dataclasses.dataclass
class ForwardState:
    """What backward needs from forward: the plan, the weight buffers and the route weights as dispatched."""
    plan: "MoonEPCommPlan"
    projections: Optional["ProjectionBuffers"]
    dispatched_route_weights: Optional[torch.Tensor] = None
    apply_route_weights: bool = True
    expert_cache: object = None


@dataclasses.dataclass
class ForwardResult:
    hidden: torch.Tensor
    route_weights: Optional[torch.Tensor]
    state: ForwardState


@dataclasses.dataclass
class BackwardResult:
    grad_hidden: torch.Tensor
    plan: "MoonEPCommPlan"


@dataclasses.dataclass
class ProjectionBuffers:
    """gate / up / down as ``[E/R + B, ...]`` tensors in symmetric memory: rows ``[0, E/R)`` are the
    rank's own experts, rows ``E/R + b`` the prefetch slots."""
    gate: torch.Tensor
    up: torch.Tensor
    down: torch.Tensor


class TileXRMoonEPBuffer:
    """Native facade: planning, dispatch, prefetch_weight, combine, reduce_grad, forward, backward."""

    def __init__(self, comm, S: int, H: int, K: int, E: int, token_padding: int = 128, B: Optional[int] = None,
                 dtype=torch.bfloat16):
        self.comm = comm
        self.S, self.H, self.K, self.E = S, H, K, E
        self.R = comm.world_size
        if E % self.R != 0:
            raise ValueError("E must divide by the number of ranks")
        self.B = E // self.R if B is None else B
        self.token_padding = token_padding
        self.NvS = S * K + (token_padding - 1) * 2 * (E // self.R)
        self.dtype = dtype
        self._poisoned = False
        self.context: Optional[TileXRMoonEPContext] = None
        from .moonep_capture import StageCapture

        self._capture = StageCapture(comm.rank)          # stage tracing / latency capture, switched on from the environment
        self._direction = "forward"
        # persistent receive tensors: peers write into them directly
        self.hidden_nvsh = comm.symm_empty([self.NvS, H], dtype)
        self.weights_nvs = comm.symm_empty([self.NvS], torch.float32)
        self._grad_nvsh = None

    @classmethod
    def from_context(cls, context: TileXRMoonEPContext) -> "TileXRMoonEPBuffer":
        """The buffer of a :class:`TileXRMoonEPContext` (the reference's constructor form, torch_api.py:591-640): the context
        gives the shape, the buffer becomes its owner until :meth:`close`."""
        self = cls(context.runtime, context.tokens_per_rank, context.hidden_size, context.topk, context.expert_count,
                   token_padding=context.token_padding, B=context.prefetch_slots, dtype=context.dtype)
        context.attach_buffer(self)
        if torch.cuda.is_available():
            context.bind_stream(self, torch.cuda.current_stream().cuda_stream)
        self.context = context
        return self

    def forward_state(self, hidden, route_weights, topk_experts, tokens_per_expert, projections: Optional[ProjectionBuffers],
                      expert_forward: Callable, apply_route_weights: bool = True) -> ForwardResult:
        """:meth:`forward` with the reference's result objects (torch_api.py:284-304): the state goes to
        :meth:`backward_state`."""
        plan = self.planning(topk_experts, tokens_per_expert)
        rows, w = self.dispatch(hidden, route_weights, plan)
        if projections is not None:
            self.prefetch_weight(plan, projections)
        out = expert_forward(rows, plan.cu_seqlens, projections)
        if apply_route_weights and w is not None:
            out = (out.float() * w.unsqueeze(1)).to(out.dtype)
        y, wy = self.combine(plan, out, None if apply_route_weights else w)
        return ForwardResult(y, wy, ForwardState(plan, projections, w, apply_route_weights))

    def backward_state(self, grad_output, state: ForwardState, expert_backward: Callable, grads: Optional[ProjectionBuffers] = None) -> BackwardResult:
        return BackwardResult(self.backward(grad_output, state.plan, expert_backward, grads), state.plan)

    def reduce_grad_info(self) -> dict:
        """Sizes of the gradient reduction of this shape: per projection, rows a rank owns and rows it may borrow."""
        L = self.E // self.R
        return {"owned_rows": L, "slot_rows": self.B, "ranks": self.R, "dtype": "float32"}

    # -- stages ------------------------------------------------------------------------------------
    def planning(self, topk_experts_sk: torch.Tensor, tokens_per_expert: Optional[torch.Tensor] = None) -> MoonEPCommPlan:
        self._check_alive()
        topk = topk_experts_sk.to(torch.int32).contiguous()
        token = self._capture.begin("planning") if self._capture.active else None
        plan = MoonEPCommPlan.from_dict(_C.moonep_planning(self.comm, topk, self.E, self.B, self.token_padding))
        self._capture.end(token)
        return plan

    def dispatch(self, hidden_sh: torch.Tensor, route_weights_sk: Optional[torch.Tensor], plan: MoonEPCommPlan,
                 out: Optional[torch.Tensor] = None, trace: Optional["DispatchTrace"] = None):
        """``trace`` (a :class:`DispatchTrace`) makes the kernel record its phases, one traced launch per call until the
        trace's iterations are used up."""
        self._check_alive()
        hidden_out = self.hidden_nvsh if out is None else out
        w_out = self.weights_nvs if route_weights_sk is not None else None
        kw = {}
        if trace is not None and trace.iteration < trace.iterations:
            kw = dict(trace_buffer=trace.buffer, trace_iteration=trace.iteration, trace_iterations=trace.iterations,
                      trace_event_capacity=trace.event_capacity)
            trace.iteration += 1
        token = self._capture.begin(f"dispatch_{self._direction}") if self._capture.active else None
        _C.moonep_dispatch(self.comm, plan.as_dict(), hidden_sh.contiguous(),
                           None if route_weights_sk is None else route_weights_sk.float().contiguous(), hidden_out, w_out, **kw)
        self._capture.end(token)
        return hidden_out, w_out

    def dispatch_trace(self, iterations: int = 1, event_capacity: int = 64, blocks: int = 128) -> "DispatchTrace":
        """A device buffer for the event trace of ``iterations`` dispatch launches (``blocks`` must be at least the grid of
        the kernel: 128 unless TILEXR_MOONEP_DISPATCH_BLOCKS says otherwise)."""
        return DispatchTrace(self.hidden_nvsh.device, iterations, event_capacity, blocks)

    def register_projection_buffers(self, rows_gate, rows_up, rows_down, dtype=torch.bfloat16) -> ProjectionBuffers:
        L = self.E // self.R
        mk = lambda shape: self.comm.symm_empty([L + self.B] + list(shape), dtype)
        return ProjectionBuffers(mk(rows_gate), mk(rows_up), mk(rows_down))

    def prefetch_weight(self, plan: MoonEPCommPlan, projections: ProjectionBuffers) -> None:
        self._check_alive()
        token = self._capture.begin("prefetch_weight") if self._capture.active else None
        _C.moonep_prefetch_weight(self.comm, plan.as_dict(), projections.gate, projections.up, projections.down)
        self._capture.end(token)

    def combine(self, plan: MoonEPCommPlan, hidden_nvsh: torch.Tensor, route_weights_nvs: Optional[torch.Tensor] = None,
                fold_duplicates: bool = False):
        """``fold_duplicates`` runs the second-generation kernel: the rows that a token has on one expert rank are summed
        there (fp32, route order, one rounding) and travel back as one row, so a token costs one row per distinct rank
        instead of one per route; the result may differ from the single-rounding sum by about one unit in the last
        place (csrc/moonep/moonep_combine_v2.cu).  Each block leaves a profile record: :meth:`combine_profile`."""
        self._check_alive()
        hidden_sh = torch.empty(self.S, hidden_nvsh.shape[1], dtype=hidden_nvsh.dtype, device=hidden_nvsh.device)
        w_sk = None
        if route_weights_nvs is not None:
            w_sk = torch.empty(self.S, self.K, dtype=torch.float32, device=hidden_nvsh.device)
        token = self._capture.begin(f"combine_{self._direction}") if self._capture.active else None
        if fold_duplicates:
            ws = self._combine_workspace(hidden_nvsh.shape[1], hidden_nvsh.dtype)
            _C.moonep_combine_v2(self.comm, plan.dst_local, hidden_nvsh.contiguous(), route_weights_nvs, hidden_sh, w_sk, ws, self.K)
        else:
            _C.moonep_combine(self.comm, plan.as_dict(), hidden_nvsh.contiguous(), route_weights_nvs, hidden_sh, w_sk)
        self._capture.end(token)
        return hidden_sh, w_sk

    def _combine_workspace(self, h: int, dtype) -> torch.Tensor:
        key = (h, dtype)
        if getattr(self, "_combine_ws_key", None) != key:
            nbytes, self._profile_off, _, _, self._profile_bytes, self._profile_max = _C.moonep_combine_v2_workspace(self.S, h, self.K, self.NvS, dtype)
            self._combine_ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.hidden_nvsh.device)
            self._combine_ws_key = key
        return self._combine_ws

    def combine_profile(self):
        """Decoded profile records of the last ``combine(..., fold_duplicates=True)`` (synchronises with the device)."""
        from ..tools.moonep.combine_v2_trace import decode_profile_records

        if getattr(self, "_combine_ws", None) is None:
            return []
        torch.cuda.synchronize()
        raw = self._combine_ws[self._profile_off:self._profile_off + self._profile_bytes * self._profile_max].cpu().numpy().tobytes()
        return decode_profile_records(raw)

    def prepare_reduce_grad(self, projections: ProjectionBuffers) -> ProjectionBuffers:
        """Gradient tensors must be fp32 and symmetric; returns zero-filled ones of the right shape."""
        L = self.E // self.R
        mk = lambda t: self.comm.symm_empty([L + self.B] + list(t.shape[1:]), torch.float32).zero_()
        return ProjectionBuffers(mk(projections.gate), mk(projections.up), mk(projections.down))

    def reduce_grad(self, plan: MoonEPCommPlan, grads: ProjectionBuffers) -> None:
        self._check_alive()
        token = self._capture.begin("reduce_grad") if self._capture.active else None
        _C.moonep_reduce_grad(self.comm, plan.as_dict(), grads.gate, grads.up, grads.down)
        self._capture.end(token)

    # -- composed flows -------------------------------------------------------------------------------
    def forward(self, hidden, route_weights, topk_experts, tokens_per_expert, projections: Optional[ProjectionBuffers],
                expert_forward: Callable, apply_route_weights: bool = True):
        plan = self.planning(topk_experts, tokens_per_expert)
        rows, w = self.dispatch(hidden, route_weights, plan)
        if projections is not None:
            self.prefetch_weight(plan, projections)
        out = expert_forward(rows, plan.cu_seqlens, projections)
        if apply_route_weights and w is not None:
            out = (out.float() * w.unsqueeze(1)).to(out.dtype)
        y, _ = self.combine(plan, out)
        return y, plan

    def backward(self, grad_output, plan: MoonEPCommPlan, expert_backward: Callable, grads: Optional[ProjectionBuffers] = None):
        if self._grad_nvsh is None or self._grad_nvsh.dtype != grad_output.dtype:
            self._grad_nvsh = self.comm.symm_empty([self.NvS, self.H], grad_output.dtype)
        self._direction = "backward"
        try:
            rows, _ = self.dispatch(grad_output, None, plan, out=self._grad_nvsh)
            grad_rows = expert_backward(rows, plan.cu_seqlens)
            gx, _ = self.combine(plan, grad_rows)
            if grads is not None:
                self.reduce_grad(plan, grads)
        finally:
            self._direction = "forward"
        return gx

    # -- housekeeping ------------------------------------------------------------------------------------
    def check_pending_status(self, plan: Optional[MoonEPCommPlan] = None) -> None:
        """Call after a stream synchronisation: raises if a stage gave up on the device."""
        status = self.comm.device_status()
        plan_status = int(plan.status.item()) if plan is not None and plan.status is not None else 0
        if status != 0 or plan_status != 0:
            self._poisoned = True
            if self.context is not None:
                self.context.mark_poisoned()
            from ..utils import failure_dump

            failure_dump.dump(self.comm, None, {"what": "MoonEP stage", "plan_status": plan_status, "S": self.S, "H": self.H, "K": self.K,
                                                "E": self.E})
            self.comm.print_dfx()
            raise TileXRMoonEPError(f"MoonEP stage failed: device status {status}, plan status {plan_status}")

    def synchronize(self) -> None:
        torch.cuda.synchronize()
        self.check_pending_status()

    quiesce = synchronize

    def _check_alive(self):
        if self._poisoned:
            raise RuntimeError("this MoonEP buffer saw a failed stage; create a new one")

    def close(self) -> None:
        if self._capture.dir and not self._poisoned:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._capture.write()
        self._poisoned = True
        if self.context is not None:
            self.context.release_stream(self)
            self.context.detach_buffer(self)
            self.context = None


class DispatchTrace:
    """Device buffer of the dispatch event trace (csrc/include/tilexr_moonep_trace.h) with its host-side decoding."""

    def __init__(self, device, iterations: int = 1, event_capacity: int = 64, blocks: int = 128):
        _, _, total = _C.moonep_trace_layout(iterations, blocks, event_capacity)
        self.buffer = torch.zeros(total, dtype=torch.uint8, device=device)
        self.iterations, self.event_capacity, self.blocks = iterations, event_capacity, blocks
        self.iteration = 0

    def raw(self) -> bytes:
        torch.cuda.synchronize()
        return self.buffer.cpu().numpy().tobytes()

    def decode(self):
        from ..tools.moonep.dispatch_trace import decode_trace

        return decode_trace(self.raw())


class Buffer:
    """Drop-in for the MoonEP ``Buffer``: same constructor and method signatures."""

    def __init__(self, S, H, K, E, num_ep_ranks, num_sms=None, token_padding=128, B=None, group=None,
                 comm_stream_priority=-1, enable_pdl=True, explicitly_destroy=False, comm=None, dtype=torch.bfloat16):
        if comm is None:
            import torch.distributed as dist

            from ..parallel.comm import init_from_torch_distributed

            if not dist.is_initialized():
                raise RuntimeError("Buffer needs an initialised torch.distributed (or pass comm=)")
            pg = group if group is not None else dist.group.WORLD
            if dist.get_world_size(pg) != num_ep_ranks:
                raise ValueError("group size must equal num_ep_ranks")
            need = max(S * K * H * 2 + S * K * 4, 64 << 20)
            comm = init_from_torch_distributed(pg, buffer_mb=int(2 * need / (1 << 20)) + 16)
        if comm.world_size != num_ep_ranks:
            raise ValueError("communicator size must equal num_ep_ranks")
        self.num_sms = 32 if num_sms is None else num_sms
        self.explicitly_destroy = explicitly_destroy
        self.native = TileXRMoonEPBuffer(comm, S, H, K, E, token_padding, B, dtype)
        self.S, self.H, self.K, self.E, self.R = S, H, K, E, num_ep_ranks
        self.B = self.native.B

    def dispatch(self, hidden_sh, route_weights_sk=None, topk_experts_sk=None, tokens_per_expert=None, plan=None,
                 async_finish=False, *, inter_rank_sync=True, zero_copy=False):
        """``zero_copy`` and ``inter_rank_sync`` are accepted as in the reference's drop-in (compat.py:264-330): the rows always
        land directly in the returned tensors (there is no boundary copy to leave out), and the kernels meet their peers through
        flags whether or not the caller asks for a synchronisation.  With ``zero_copy=True`` the returned tensors are remembered,
        and ``combine(zero_copy=True)`` insists on getting exactly them."""
        del inter_rank_sync
        self._zero_copy_aliases = None
        if plan is None:
            if topk_experts_sk is None:
                raise ValueError("a fresh dispatch needs topk_experts_sk")
            plan = self.native.planning(topk_experts_sk, tokens_per_expert)
        rows, w = self.native.dispatch(hidden_sh, route_weights_sk, plan)
        if zero_copy:
            self._zero_copy_aliases = (plan, rows, w)
        out = (rows, w, plan.cu_seqlens, plan)
        if async_finish:
            ev = torch.cuda.Event()
            ev.record()
            out = out + (ev,)
        return out

    def prefetch_weight(self, plan, async_finish=False, *, full_gate_weight, full_up_weight, full_down_weight):
        """Every rank holds all E experts in rows [0, E); rows [E, E+B) receive this rank's
        borrowed experts (a local copy, as in the reference's compatibility layer)."""
        idx = plan.experts_to_copy[self.native.comm.rank].long()
        valid = idx >= 0
        src = idx.clamp(min=0)
        for t in (full_gate_weight, full_up_weight, full_down_weight):
            rows = t.index_select(0, src)
            rows[~valid] = 0
            t[self.E:self.E + self.B].copy_(rows)
        if async_finish:
            ev = torch.cuda.Event()
            ev.record()
            return ev
        return None

    def combine(self, plan, hidden_nvsh, route_weights_nvs=None, async_finish=False, inter_rank_sync=True, *, zero_copy=False):
        del inter_rank_sync
        if zero_copy:
            aliases = getattr(self, "_zero_copy_aliases", None)
            if aliases is None or aliases[0] is not plan or hidden_nvsh.data_ptr() != aliases[1].data_ptr():
                raise AssertionError("combine(zero_copy=True): hidden_nvsh must be the output of the latest zero-copy dispatch of this plan")
            if route_weights_nvs is not None and (aliases[2] is None or route_weights_nvs.data_ptr() != aliases[2].data_ptr()):
                raise AssertionError("combine(zero_copy=True): route_weights_nvs must be the weights of the latest zero-copy dispatch")
        self._zero_copy_aliases = None
        # TILEXR_MOONEP_COMBINE_VERSION=2 selects the second-generation kernel (duplicates folded on the expert rank); the
        # default here is the first, whose sum is rounded once
        import os

        fold = os.environ.get("TILEXR_MOONEP_COMBINE_VERSION", "1").strip() == "2"
        y, w = self.native.combine(plan, hidden_nvsh, route_weights_nvs, fold_duplicates=fold)
        ev = None
        if async_finish:
            ev = torch.cuda.Event()
            ev.record()
        return y, w, ev

    def reduce_grad(self, plan, async_finish=False, *, full_gate_grad, full_up_grad, full_down_grad, gate_reduce_buffer,
                    up_reduce_buffer, down_reduce_buffer):
        """Slot rows [E, E+B) of every rank are gathered into the ``[R, B, ...]`` reduce buffers and
        each owner adds the rows of its experts in ascending (rank, slot) order."""
        comm = self.native.comm
        L = self.E // self.R
        etc = plan.experts_to_copy
        for grad, buf in ((full_gate_grad, gate_reduce_buffer), (full_up_grad, up_reduce_buffer),
                          (full_down_grad, down_reduce_buffer)):
            collectives.all_gather(comm, grad[self.E:self.E + self.B].contiguous(), out=buf)
            owner_rows = (etc >= comm.rank * L) & (etc < (comm.rank + 1) * L)
            rr, bb = owner_rows.nonzero(as_tuple=True)
            for r, b in zip(rr.tolist(), bb.tolist()):
                if r == comm.rank:
                    continue
                grad[int(etc[r, b])] += buf[r, b]
            grad[self.E:self.E + self.B].zero_()
        if async_finish:
            ev = torch.cuda.Event()
            ev.record()
            return ev
        return None

    def destroy(self):
        self.native.close()
        self._destroyed = True

    @property
    def destroyed(self) -> bool:
        return getattr(self, "_destroyed", False)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.destroy()
        return False


# ---- planner, second generation ---------------------------------------------------------------------------------

PLAN_STATUS_NAMES = ("PLAN_OK", "PLAN_PARTIAL_NO_FEASIBLE_PAIR", "PLAN_PARTIAL_PREFETCH_SLOT_EXHAUSTED", "PLAN_PARTIAL_TOKEN_SUPPLY",
                     "PLAN_ERROR_CONFIG_MISMATCH", "PLAN_ERROR_TPE_MISMATCH", "PLAN_ERROR_LAYOUT_EXCEEDS_NVS",
                     "PLAN_ERROR_MOVE_RECORD_OVERFLOW", "PLAN_ERROR_INTERNAL_INVARIANT")


@dataclasses.dataclass
class MoonEPPlanV2:
    """Tables of the topology-aware planner (C API ``TileXRMoeEpPlanV2WithMetadata``, csrc/include/tilexr_ep_plan.h;
    reference: src/include/tilexr_ep_plan.h:27-58).  ``dst`` holds ``dst_rank * nvs + row`` per route, ``~raw`` for a
    route whose token already has an earlier route to the same rank."""
    dst: torch.Tensor
    cu_seqlens: torch.Tensor
    experts_to_copy: torch.Tensor
    remote_stats: torch.Tensor
    remote_experts: torch.Tensor
    expert_targets: torch.Tensor
    status: torch.Tensor
    nvs: int
    workspace: Optional[torch.Tensor] = None
    stage_plan: Optional[dict] = None      # the tables the dispatch / combine / prefetch / reduce-grad stages take

    def comm_plan(self) -> MoonEPCommPlan:
        """The plan in the form ``TileXRMoonEPBuffer`` passes to the stage kernels: destinations with duplicates
        decoded (every route carries its hidden state), zero-fill ranges, the row -> route table and a one-word status."""
        return MoonEPCommPlan.from_dict(self.stage_plan)

    def status_name(self) -> str:
        """Reads the status word (synchronises with the stream that planned)."""
        return PLAN_STATUS_NAMES[int(self.status[0].item())]

    def decode(self, world_size: int):
        """(dst_rank, row, sends_hidden) per route, as tensors on the plan's device."""
        raw = torch.where(self.dst >= 0, self.dst, ~self.dst)
        return raw // self.nvs, raw % self.nvs, self.dst >= 0


def planning_v2(comm, topk_experts_sk: torch.Tensor, tokens_per_expert_re: torch.Tensor, global_rank_ids: Optional[torch.Tensor] = None,
                prefetch_slots: int = 8, nvs: Optional[int] = None, token_padding: int = 1, route_limit_per_pair: int = 0) -> MoonEPPlanV2:
    """Plans one step on this rank of ``comm`` (every rank calls it with the same ``tokens_per_expert_re`` [R, E]).

    ``global_rank_ids`` places the ranks in servers of 8 consecutive ids; the default is the communicator's own
    numbering, i.e. one server per 8 ranks.  Nothing synchronises with the host: read ``plan.status`` when needed.
    """
    S, K = topk_experts_sk.shape
    R, E = tokens_per_expert_re.shape
    if global_rank_ids is None:
        global_rank_ids = torch.arange(R, dtype=torch.int32, device=topk_experts_sk.device)
    if nvs is None:
        nvs = S * K + (E + prefetch_slots) * token_padding
    d = _C.moonep_plan_v2(comm, topk_experts_sk.to(torch.int32).contiguous(), tokens_per_expert_re.to(torch.int32).contiguous(),
                          global_rank_ids.to(torch.int32).contiguous(), prefetch_slots, nvs, token_padding, route_limit_per_pair)
    return MoonEPPlanV2(dst=d["dst"], cu_seqlens=d["cu_seqlens"], experts_to_copy=d["experts_to_copy"], remote_stats=d["remote_stats"],
                        remote_experts=d["remote_experts"], expert_targets=d["expert_targets"], status=d["status"], nvs=nvs,
                        workspace=d["workspace"], stage_plan=d["stage_plan"])
