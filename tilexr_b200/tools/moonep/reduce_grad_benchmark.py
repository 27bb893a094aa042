"""ReduceGrad on its own (reference: tools/moonep/reduce_grad_benchmark.py).

With the synthetic borrow table of :mod:`prefetch_weight_benchmark` every rank holds fp32 gradient rows in its
``B`` slots that belong to remote owners; the stage makes each owner add, in ascending (rank, slot) order, the slot
rows of everybody who borrowed one of its experts, and clears the slots.  Bytes per rank and round by the
reference's formula: borrowed slots x 3 x ffn x hidden x 4.
"""
from __future__ import annotations

from typing import Dict

import torch

from ...integrations.moonep import ProjectionBuffers, TileXRMoonEPBuffer
from .benchmark import summarise
from .contracts import MoonEPCase
from .prefetch_weight_benchmark import synthetic_borrow_table


def reduce_grad_benchmark(comm, case: MoonEPCase, iters: int = 20, warmup: int = 5) -> Dict[str, object]:
    if case.ffn <= 0:
        raise ValueError("the case has no projection tensors (ffn = 0)")
    rank, R, L, B = comm.rank, case.ranks, case.local_experts, case.prefetch_slots
    buf = TileXRMoonEPBuffer(comm, case.tokens, case.hidden, case.top_k, case.experts, token_padding=case.token_padding, B=B,
                             dtype=case.torch_dtype())
    dev = buf.hidden_nvsh.device
    g = torch.Generator().manual_seed(case.seed * 31 + rank)
    topk = torch.randint(0, case.experts, (case.tokens, case.top_k), generator=g, dtype=torch.int32).to(dev)
    plan = buf.planning(topk)
    buf.synchronize()
    table = synthetic_borrow_table(R, L, B)
    plan.experts_to_copy.copy_(table.to(dev))
    shape = (case.ffn, case.hidden)
    proj = buf.register_projection_buffers(shape, shape, shape, dtype=case.torch_dtype())
    grads = buf.prepare_reduce_grad(proj)
    samples = {"reduce_grad": []}
    ok = True
    for it in range(warmup + iters):
        for t in (grads.gate, grads.up, grads.down):
            t[:L].zero_()
            t[L:].fill_(float(rank + 1))                  # slot rows carry the borrower's rank + 1
        torch.cuda.synchronize()
        comm.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        buf.reduce_grad(plan, ProjectionBuffers(grads.gate, grads.up, grads.down))
        e1.record()
        buf.synchronize()
        if it >= warmup:
            samples["reduce_grad"].append(e0.elapsed_time(e1) * 1e3)
        if it == 0:
            want = torch.zeros(L)
            for r in range(R):
                for b in range(B):
                    e = int(table[r, b])
                    if e >= 0 and e // L == rank and r != rank:
                        want[e % L] += r + 1
            got = grads.gate[:L].float().mean(dim=(1, 2)).cpu()
            ok = bool(torch.equal(got, want)) and float(grads.gate[L:].abs().max().item()) == 0.0
    nbytes = {"reduce_grad": int((table[rank] >= 0).sum()) * 3 * case.ffn * case.hidden * 4}
    out = summarise(case, samples, nbytes, iters, warmup, dev)
    out["verified"] = ok
    buf.close()
    return out
