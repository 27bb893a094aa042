"""PrefetchWeight on its own (reference: tools/moonep/prefetch_weight_benchmark.py).

Every rank owns ``E/R`` experts with gate / up / down rows of ``ffn x hidden`` elements and pulls ``B`` borrowed
experts into its slots; which ones is fixed by a synthetic plan (slot b of rank r borrows expert
``((r + 1 + b) % R) * E/R + b % (E/R)``, i.e. always a remote one, a different owner per slot), so that the
stage is measured at a known byte count: ``B x 3 x ffn x hidden x element size`` per rank and round.  The
reference publishes this stage at 4 slots x 3 x 28 MiB = 336 MiB per rank (EP8, bf16, hidden 7168, ffn 2048).
"""
from __future__ import annotations

from typing import Dict

import torch

from ...integrations.moonep import TileXRMoonEPBuffer
from .benchmark import summarise
from .contracts import MoonEPCase


def synthetic_borrow_table(ranks: int, local_experts: int, slots: int) -> torch.Tensor:
    etc = torch.full((ranks, slots), -1, dtype=torch.int32)
    if ranks > 1:
        for r in range(ranks):
            for b in range(slots):
                owner = (r + 1 + b % (ranks - 1)) % ranks
                etc[r, b] = owner * local_experts + b % local_experts
    return etc


def prefetch_weight_benchmark(comm, case: MoonEPCase, iters: int = 20, warmup: int = 5) -> Dict[str, object]:
    if case.ffn <= 0:
        raise ValueError("the case has no projection tensors (ffn = 0)")
    rank, R, L, B = comm.rank, case.ranks, case.local_experts, case.prefetch_slots
    buf = TileXRMoonEPBuffer(comm, case.tokens, case.hidden, case.top_k, case.experts, token_padding=case.token_padding, B=B,
                             dtype=case.torch_dtype())
    dev = buf.hidden_nvsh.device
    g = torch.Generator().manual_seed(case.seed * 31 + rank)
    topk = torch.randint(0, case.experts, (case.tokens, case.top_k), generator=g, dtype=torch.int32).to(dev)
    plan = buf.planning(topk)                  # a real plan gives the tables their shapes; the borrow table is replaced
    buf.synchronize()
    plan.experts_to_copy.copy_(synthetic_borrow_table(R, L, B).to(dev))
    shape = (case.ffn, case.hidden)
    proj = buf.register_projection_buffers(shape, shape, shape, dtype=case.torch_dtype())
    for t in (proj.gate, proj.up, proj.down):
        t.zero_()
        t[:L].fill_(float(rank + 1))
    torch.cuda.synchronize()
    comm.barrier()
    samples = {"prefetch_weight": []}
    for it in range(warmup + iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        buf.prefetch_weight(plan, proj)
        e1.record()
        buf.synchronize()
        if it >= warmup:
            samples["prefetch_weight"].append(e0.elapsed_time(e1) * 1e3)
    # what arrived is the owner's fill value
    etc = plan.experts_to_copy.cpu()
    ok = all(float(proj.gate[L + b].float().mean().item()) == float(int(etc[rank, b]) // L + 1) for b in range(B) if int(etc[rank, b]) >= 0)
    esize = torch.tensor([], dtype=case.torch_dtype()).element_size()
    pulled = int((etc[rank] >= 0).sum())
    nbytes = {"prefetch_weight": pulled * 3 * case.ffn * case.hidden * esize}
    out = summarise(case, samples, nbytes, iters, warmup, dev)
    out["verified"] = bool(ok)
    buf.close()
    return out
