"""The library under test behind the harness contract (reference: tools/moonep/tilexr_backend.py)."""
from __future__ import annotations

import torch

from ...integrations.moonep import ProjectionBuffers, TileXRMoonEPBuffer
from .contracts import MoonEPCase, RankInputs, StageArtifacts


class TileXRBackend:
    name = "tilexr"

    def __init__(self, comm):
        self.comm = comm
        self._buffers = {}

    def _buffer(self, case: MoonEPCase) -> TileXRMoonEPBuffer:
        key = (case.tokens, case.hidden, case.top_k, case.experts, case.token_padding, case.prefetch_slots, case.dtype)
        if key not in self._buffers:
            self._buffers[key] = TileXRMoonEPBuffer(self.comm, case.tokens, case.hidden, case.top_k, case.experts,
                                                    token_padding=case.token_padding, B=case.prefetch_slots,
                                                    dtype=case.torch_dtype())
        return self._buffers[key]

    def run(self, case: MoonEPCase, inputs: RankInputs, expert_fn=None) -> StageArtifacts:
        buf = self._buffer(case)
        dev = buf.hidden_nvsh.device
        L, B = case.local_experts, case.prefetch_slots
        plan = buf.planning(inputs.topk_experts_sk.to(dev))
        rows, w = buf.dispatch(inputs.hidden_sh.to(dev), inputs.route_weights_sk.to(dev), plan)
        dispatched_hidden, dispatched_weights = rows.clone(), w.clone()
        processed = rows if expert_fn is None else expert_fn(rows, plan)
        combined, wback = buf.combine(plan, processed, w)
        prefetched = reduced = None
        if inputs.gate is not None:
            proj = buf.register_projection_buffers(inputs.gate.shape[1:], inputs.gate.shape[1:], inputs.gate.shape[1:],
                                                   dtype=inputs.gate.dtype)
            for t, src in ((proj.gate, inputs.gate), (proj.up, inputs.up), (proj.down, inputs.down)):
                t.zero_()
                t[:L].copy_(src.to(dev))
            self.comm.barrier()                       # every owner's rows are in place before anyone pulls
            buf.prefetch_weight(plan, proj)
            prefetched = proj.gate.clone()
            grads = buf.prepare_reduce_grad(proj)
            grads.gate.copy_(inputs.grad_rows.to(dev))
            torch.cuda.synchronize()
            self.comm.barrier()
            buf.reduce_grad(plan, ProjectionBuffers(grads.gate, None, None))
            reduced = grads.gate.clone()
        buf.synchronize()
        d = plan.as_dict()
        tensors = {k: v.cpu() for k, v in d.items() if isinstance(v, torch.Tensor)}
        return StageArtifacts(plan=tensors, dispatched_hidden=dispatched_hidden.cpu(), dispatched_weights=dispatched_weights.cpu(),
                              prefetched_gate=None if prefetched is None else prefetched.cpu(), combined_hidden=combined.cpu(),
                              combined_weights=wback.cpu(), reduced_grad=None if reduced is None else reduced.cpu())

    def close(self) -> None:
        for b in self._buffers.values():
            b.close()
        self._buffers.clear()
