"""tcgen05 GEMM and its fusions with collectives (csrc/include/tilexr_fused.h).

Weights follow the ``torch.nn.Linear`` convention: ``b`` is ``[N, K]`` and the product is
``a @ b.T``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _C


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a[M,K] @ b[N,K].T`` on the tensor cores (fp16 / bf16, fp32 accumulation)."""
    return _C.matmul(a.contiguous(), b.contiguous())


EPILOGUE_STORE = 0
EPILOGUE_SWIGLU = 1


def grouped_matmul(rows: torch.Tensor, weights: torch.Tensor, group_rows: torch.Tensor, epilogue: int = EPILOGUE_STORE,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """Grouped GEMM of an expert feed-forward in one launch: ``rows`` [R, K] hold ``group_rows[0]`` rows of group 0, then
    ``group_rows[1]`` rows of group 1, ...; group g is multiplied with ``weights[g]`` ([groups, N, K]).  ``group_rows`` is
    an int64 tensor ON THE DEVICE (``DispatchResult.expert_token_nums``): the tile list is built inside the kernel and
    nothing is read back to the host.  Rows past the sum of the counts are left as they are.

    ``epilogue=EPILOGUE_SWIGLU`` reads weight row 2i as gate row i and row 2i+1 as up row i (see
    :func:`interleave_gate_up`) and returns ``silu(gate) * up`` [R, N/2] without the [R, N] intermediate."""
    return _C.grouped_matmul(rows.contiguous(), weights.contiguous(), group_rows, int(epilogue), out)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[..., F, K] gate and up projections -> [..., 2F, K] with gate row i at 2i and up row i at 2i+1, the layout the
    SwiGLU epilogue of :func:`grouped_matmul` expects."""
    return torch.stack((w_gate, w_up), dim=-2).reshape(*w_gate.shape[:-2], 2 * w_gate.shape[-2], w_gate.shape[-1]).contiguous()


def grouped_matmul_ref(rows: torch.Tensor, weights: torch.Tensor, group_rows, epilogue: int = EPILOGUE_STORE) -> torch.Tensor:
    """Plain PyTorch statement of :func:`grouped_matmul` in fp32 (rows past the counts come back as zeros)."""
    n = weights.shape[1] // 2 if epilogue == EPILOGUE_SWIGLU else weights.shape[1]
    out = torch.zeros(rows.shape[0], n, dtype=torch.float32, device=rows.device)
    start = 0
    for g, count in enumerate(int(v) for v in group_rows.tolist()):
        count = max(0, min(count, rows.shape[0] - start))
        prod = rows[start:start + count].float() @ weights[g].float().t()
        if epilogue == EPILOGUE_SWIGLU:
            prod = torch.nn.functional.silu(prod[:, 0::2]) * prod[:, 1::2]
        out[start:start + count] = prod
        start += count
    return out


def matmul_fp8(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``alpha * a @ b.T`` for fp8 operands (both float8_e4m3fn or both float8_e5m2; a [M, K], b [N, K], K % 16 == 0) with fp32
    accumulation on the 8-bit tensor-core path; ``alpha`` is the product of the two per-tensor dequantisation scales."""
    return _C.matmul_fp8(a.contiguous(), b.contiguous(), float(alpha), out_dtype)


def matmul_fp8_block(a: torch.Tensor, scale_a: torch.Tensor, b: torch.Tensor, scale_b: torch.Tensor,
                     out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Block-scaled fp8 product ``(a * scale_a) @ (b * scale_b).T`` with fp32 scales: ``a`` [M, K] with one scale per row and
    128 elements of K (``scale_a`` [M, K/128], what ``ep.dispatch(..., quant_mode=QUANT_FP8_1X128)`` and
    ``quant.fp8_quant_1x128`` produce), ``b`` [N, K] with one scale per 128 x 128 block (``scale_b`` [ceil(N/128), K/128],
    see :func:`quantize_weight_128x128`).  The tensor cores multiply one block of K at a time in fp32; the blocks are folded
    together with their scales on the CUDA cores while the next block is being multiplied."""
    return _C.matmul_fp8_block(a.contiguous(), scale_a.contiguous(), b.contiguous(), scale_b.contiguous(), out_dtype)


def quantize_weight_128x128(w: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn):
    """``w`` [N, K] (K a multiple of 128) -> (fp8 [N, K], fp32 scales [ceil(N/128), K/128]): one scale per 128 x 128 block,
    the block's largest magnitude mapped to the largest finite value of the fp8 type."""
    n, k = w.shape
    if k % 128 != 0:
        raise ValueError("K must be a multiple of 128")
    fmax = torch.finfo(dtype).max
    nb = (n + 127) // 128
    wp = torch.nn.functional.pad(w.float(), (0, 0, 0, nb * 128 - n))
    blocks = wp.view(nb, 128, k // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-4)
    scale = amax / fmax
    q = (blocks / scale[:, None, :, None]).clamp(-fmax, fmax).to(dtype).view(nb * 128, k)[:n].contiguous()
    return q, scale.contiguous()


def all_gather_matmul(comm, a_shard: torch.Tensor, b: torch.Tensor, staging: torch.Tensor) -> torch.Tensor:
    """``all_gather(a_shard) @ b.T`` with the gather overlapped tile by tile.

    ``staging`` is a ``comm.symm_empty([world * rows, K], dtype)`` buffer reused across calls.
    """
    return _C.all_gather_matmul(comm, a_shard.contiguous(), staging, b.contiguous())


def matmul_reduce_scatter(comm, a: torch.Tensor, b: torch.Tensor, staging: torch.Tensor) -> torch.Tensor:
    """``reduce_scatter(a @ b.T)`` along rows; ``staging`` is ``comm.symm_empty([M, N], dtype)``."""
    return _C.matmul_reduce_scatter(comm, a.contiguous(), b.contiguous(), staging)


def matmul_all_reduce(comm, a: torch.Tensor, b: torch.Tensor, staging: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``all_reduce(a @ b.T)`` (the reference's MATMUL_ALL_REDUCE operator id): the reduce-scatter runs in the GEMM's epilogue
    (:func:`matmul_reduce_scatter`), the reduced row shards are then all-gathered.  A registered ``out``
    (``comm.symm_empty([M, N], dtype)``) is written by the peers directly."""
    from .collectives import all_gather
    shard = matmul_reduce_scatter(comm, a, b, staging)
    world = comm.world_size
    if out is None:
        out = torch.empty((world * shard.shape[0], shard.shape[1]), dtype=shard.dtype, device=shard.device)
    all_gather(comm, shard, out=out.view(world, shard.shape[0], shard.shape[1]))
    return out


def all_gather_matmul_fp8_block(comm, a_shard: torch.Tensor, scale_a_shard: torch.Tensor, a_staging: torch.Tensor, scale_staging: torch.Tensor,
                                b: torch.Tensor, scale_b: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``all_gather(a_shard) @ b.T`` with block scales (see :func:`matmul_fp8_block`): the shard's fp8 rows and their 1 x 128
    scales are written into every rank's staging buffers (``comm.symm_empty([world * rows, K], fp8)`` and
    ``comm.symm_empty([world * rows, K // 128], float32)``) by otherwise idle warps of the GEMM's own CTAs, through the NVLink
    multicast alias of the buffers where there is one, and each tile starts when its rows have landed."""
    return _C.all_gather_matmul_fp8_block(comm, a_shard.contiguous(), scale_a_shard.contiguous(), a_staging, scale_staging, b.contiguous(),
                                          scale_b.contiguous(), out_dtype)


def matmul_reduce_scatter_fp8_block(comm, a: torch.Tensor, scale_a: torch.Tensor, b: torch.Tensor, scale_b: torch.Tensor,
                                    staging: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``reduce_scatter(a @ b.T)`` along rows with block scales; ``staging`` is ``comm.symm_empty([M, N], out_dtype)``.  Partial
    tiles are stored into the row owner's staging slots from the GEMM's epilogue and added there in rank order in fp32."""
    return _C.matmul_reduce_scatter_fp8_block(comm, a.contiguous(), scale_a.contiguous(), b.contiguous(), scale_b.contiguous(), staging, out_dtype)
