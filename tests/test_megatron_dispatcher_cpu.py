"""The Megatron-style dispatcher's autograd rules, route recorder and replay on the CPU: the two kernels are replaced by a
one-rank PyTorch statement of dispatch and combine, and the gradients are compared with a dense MoE under autograd."""
import dataclasses

import torch

from tilexr_b200.integrations.megatron_dispatcher import RouteRecorder, RouteReplay, TileXRTokenDispatcher
from tilexr_b200.ops import ep


class _OneRankOps:
    """dispatch / combine of tilexr_b200.ops.ep for a world of one rank, in plain PyTorch."""

    def dispatch(self, comm, x, *, num_experts, top_k, expert_ids, expert_scales=None, quant_mode=0, max_recv_rows=None,
                 dedup=None, tp_world_size=1):
        bs = x.shape[0]
        flat = expert_ids.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                       # by expert, then (token, k)
        tokens, slots = order // top_k, order % top_k
        rows = max_recv_rows or bs * top_k
        expand = torch.zeros(rows, x.shape[1], dtype=x.dtype)
        expand[: order.numel()] = x[tokens]
        assist = torch.zeros(rows, 4, dtype=torch.int32)
        assist[: order.numel()] = torch.stack([torch.zeros_like(tokens), tokens, slots, flat[order]], dim=1).to(torch.int32)
        scales = torch.zeros(rows)
        if expert_scales is not None:
            scales[: order.numel()] = expert_scales.reshape(-1)[order]
        route_rows = torch.empty(bs * top_k, dtype=torch.int32)
        route_rows[order] = torch.arange(order.numel(), dtype=torch.int32)
        none = torch.zeros(1, dtype=torch.int32)
        return ep.DispatchResult(expand, None, assist, torch.bincount(flat, minlength=num_experts), none, torch.tensor([order.numel()], dtype=torch.int32),
                                 expert_ids, none, route_rows.view(bs, top_k), none, scales, none, bs=bs, top_k=top_k,
                                 num_experts=num_experts, dedup=False)

    def combine(self, comm, expert_out, d, *, expert_scales=None):
        rows = d.route_rows.long()
        picked = expert_out.float()[rows]                              # [bs, k, h]
        w = torch.ones(rows.shape) if expert_scales is None else expert_scales.float()
        return (picked * w.unsqueeze(-1)).sum(dim=1).to(expert_out.dtype)


@dataclasses.dataclass
class _Comm:
    world_size: int = 1
    rank: int = 0


def _setup(seed=0, tokens=12, h=16, E=4, K=2):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, h, generator=g, requires_grad=True)
    logits = torch.randn(tokens, E, generator=g, requires_grad=True)
    w = torch.randn(E, h, h, generator=g) / h ** 0.5
    return x, logits, w, E, K


def test_gradients_match_a_dense_moe():
    x, logits, w, E, K = _setup()
    probs_all = torch.softmax(logits, -1)
    probs, idx = probs_all.topk(K, dim=-1)
    disp = TileXRTokenDispatcher(_Comm(), E, K, x.shape[1], ops=_OneRankOps())
    rows, counts = disp.token_permutation(x, probs, idx)
    out = torch.zeros_like(rows)
    first = 0
    for e, n in enumerate(counts.tolist()):
        out[first:first + n] = torch.tanh(rows[first:first + n] @ w[e].t())
        first += n
    y, _ = disp.token_unpermutation(out)
    target = torch.randn(y.shape, generator=torch.Generator().manual_seed(1))
    (y * target).sum().backward()
    gx, gl = x.grad.clone(), logits.grad.clone()

    x.grad = logits.grad = None
    probs2, idx2 = torch.softmax(logits, -1).topk(K, dim=-1)
    dense = torch.zeros_like(x)
    for k in range(K):
        per_tok = torch.stack([torch.tanh(x[t] @ w[idx2[t, k]].t()) for t in range(x.shape[0])])
        dense = dense + probs2[:, k:k + 1] * per_tok
    (dense * target).sum().backward()
    assert torch.allclose(y, dense, atol=1e-5)
    assert torch.allclose(gx, x.grad, atol=1e-5)
    # the probability gradients return as (high, low) bf16 pairs: about 16 bits of mantissa
    assert torch.allclose(gl, logits.grad, rtol=1e-3, atol=1e-4)


def test_route_recorder_and_replay(tmp_path):
    x, logits, w, E, K = _setup(seed=3)
    rec = RouteRecorder(str(tmp_path), rank=0, max_steps=2)
    disp = TileXRTokenDispatcher(_Comm(), E, K, x.shape[1], ops=_OneRankOps(), recorder=rec, stage_barrier=True)
    seen = []
    for step in range(3):                                              # the third step is past max_steps
        probs, idx = torch.softmax(logits.detach() + step, -1).topk(K, dim=-1)
        rows, _ = disp.token_permutation(x.detach(), probs, idx)
        disp.token_unpermutation(rows)
        seen.append((idx.to(torch.int32), probs))
    rec.close()
    replay = RouteReplay(rec.path)
    assert len(replay) == 2
    for step in (0, 1, 0):                                             # wraps around
        ids, probs = replay.next()
        assert torch.equal(ids, seen[step][0]) and torch.allclose(probs, seen[step][1])
