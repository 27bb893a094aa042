"""The Megatron-Core style token dispatcher over the fused dispatch / combine kernels, against a dense PyTorch MoE."""
import pytest
import torch

from conftest import free_port, require_cuda

pytestmark = pytest.mark.gpu


def test_dispatcher_round_trip_matches_dense_moe():
    require_cuda()
    import tilexr_b200 as txr
    from tilexr_b200.integrations.megatron_dispatcher import TileXRTokenDispatcher

    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{free_port()}", buffer_mb=64, device=0)
    try:
        s, b, h, E, K = 24, 2, 256, 8, 2
        g = torch.Generator().manual_seed(4)
        hidden = torch.randn(s, b, h, generator=g).to(torch.bfloat16).cuda()
        logits = torch.randn(s * b, E, generator=g)
        probs, idx = torch.softmax(logits, -1).topk(K, dim=-1)
        probs = (probs / probs.sum(-1, keepdim=True)).cuda()
        idx = idx.cuda()
        w = (torch.randn(E, h, h, generator=g) / h ** 0.5).to(torch.bfloat16).cuda()

        disp = TileXRTokenDispatcher(comm, E, K, h)
        for _ in range(2):
            rows, counts = disp.token_permutation(hidden, probs, idx)
            torch.cuda.synchronize()
            assert counts.tolist() == torch.bincount(idx.reshape(-1).cpu(), minlength=E).tolist()
            assert disp.ctx() is not None and int(disp.ctx().recv_total.item()) == s * b * K
            out_rows = torch.zeros_like(rows)
            first = 0
            for e, n in enumerate(counts.tolist()):          # what a grouped GEMM does with the sorted rows
                out_rows[first:first + n] = rows[first:first + n] @ w[e].t()
                first += n
            y, _ = disp.token_unpermutation(out_rows)
            torch.cuda.synchronize()
            assert comm.device_status() == 0
        x = hidden.reshape(-1, h).float()
        ref = torch.zeros_like(x)
        for k in range(K):
            per_tok = torch.stack([(x[t].to(torch.bfloat16) @ w[idx[t, k]].t()).float() for t in range(x.shape[0])])
            ref += probs[:, k:k + 1].float() * per_tok
        assert y.shape == hidden.shape
        assert torch.allclose(y.float().reshape(-1, h), ref, rtol=3e-2, atol=3e-2)
        with pytest.raises(RuntimeError):
            disp.token_unpermutation(out_rows)
    finally:
        comm.destroy()


def test_dispatcher_backward_matches_dense_moe():
    """Loss gradients with respect to the hidden states, the router probabilities and the expert outputs through the two
    autograd functions (dispatch and combine in swapped roles), against a dense MoE under PyTorch autograd."""
    require_cuda()
    import tilexr_b200 as txr
    from tilexr_b200.integrations.megatron_dispatcher import TileXRTokenDispatcher

    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{free_port()}", buffer_mb=64, device=0)
    try:
        tokens, h, E, K = 64, 256, 8, 2
        g = torch.Generator().manual_seed(8)
        x = torch.randn(tokens, h, generator=g).to(torch.bfloat16).cuda().requires_grad_(True)
        logits = torch.randn(tokens, E, generator=g).cuda().requires_grad_(True)
        w = (torch.randn(E, h, h, generator=g) / h ** 0.5).to(torch.bfloat16).cuda()
        target = torch.randn(tokens, h, generator=g).cuda()

        probs, idx = torch.softmax(logits, -1).topk(K, dim=-1)
        disp = TileXRTokenDispatcher(comm, E, K, h)
        rows, counts = disp.token_permutation(x, probs, idx)
        pieces, first = [], 0
        for e, n in enumerate(counts.tolist()):
            pieces.append(rows[first:first + n] @ w[e].t())
            first += n
        out = torch.cat(pieces + [rows[first:] * 0])
        y, _ = disp.token_unpermutation(out)
        (y.float() * target).sum().backward()
        torch.cuda.synchronize()
        assert comm.device_status() == 0
        gx, gl = x.grad.float().clone(), logits.grad.clone()

        x.grad = logits.grad = None
        probs2, idx2 = torch.softmax(logits, -1).topk(K, dim=-1)
        dense = torch.zeros(tokens, h, device="cuda")
        for k in range(K):
            per_tok = torch.bmm(x.unsqueeze(1), w[idx2[:, k]].transpose(1, 2)).squeeze(1).float()
            dense = dense + probs2[:, k:k + 1] * per_tok
        (dense * target).sum().backward()
        assert torch.allclose(y.float(), dense, rtol=3e-2, atol=3e-2)
        assert torch.allclose(gx, x.grad.float(), rtol=5e-2, atol=5e-2), (gx - x.grad.float()).abs().max()
        assert torch.allclose(gl, logits.grad, rtol=5e-2, atol=2e-2), (gl - logits.grad).abs().max()
    finally:
        comm.destroy()
