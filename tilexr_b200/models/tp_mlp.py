"""Tensor-parallel SwiGLU feed-forward with sequence-parallel activations, built on the fused GEMMs.

The layout is Megatron's sequence parallelism: every rank holds ``tokens / world`` rows of the activations, a column
shard of the gate / up projection and a row shard of the down projection.

    x_shard [T/R, H]  --all-gather -> GEMM-->  [T, 2F/R]  --SwiGLU-->  [T, F/R]  --GEMM -> reduce-scatter-->  y_shard [T/R, H]

Both collectives run inside the GEMM kernels (csrc/gemm/gemm_tcgen05_pair.cu: the gather is pushed by warps of the GEMM's own
CTAs tile by tile, the partial products are stored to the row owners from the epilogue and added there in rank order), so
the layer issues two GEMM launches and one elementwise kernel and no separate collective.  With ``fp8_block=True`` the
operands are e4m3 with 1 x 128 activation scales and 128 x 128 weight scales (csrc/gemm/gemm_tcgen05_fp8_block.cu): the
gather then moves half the bytes, rows and scales together.

The reference names these fusions only as operator ids (ALL_GATHER_MATMUL, MATMUL_REDUCE_SCATTER; its
src/include/tilexr_types.h:108-125); `tilexr_b200/tools/tp_mlp_perf.py` times the same two launches against NCCL + cuBLAS.
"""
from __future__ import annotations

import dataclasses

import torch


@dataclasses.dataclass
class TPMlpConfig:
    hidden: int = 8192
    ffn: int = 28672                 # the full width; every rank holds ffn / world columns
    tokens: int = 8192               # global rows per call (the staging buffers are sized for it)
    dtype: torch.dtype = torch.bfloat16
    fp8_block: bool = False


def shard_weights(w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, rank: int, world: int):
    """This rank's shards of full weights: gate / up [F, H] are cut by rows (output columns of the first GEMM) and stacked as
    [2F/R, H] (gate rows first), down [H, F] is cut by columns (the contraction of the second GEMM)."""
    f = w_gate.shape[0]
    if f % world != 0:
        raise ValueError("the feed-forward width must divide by the number of ranks")
    lo, hi = rank * f // world, (rank + 1) * f // world
    return torch.cat([w_gate[lo:hi], w_up[lo:hi]], dim=0).contiguous(), w_down[:, lo:hi].contiguous()


class SequenceParallelMLP(torch.nn.Module):
    """``ops`` is the module that provides ``all_gather_matmul`` / ``matmul_reduce_scatter`` (and their ``_fp8_block`` forms);
    the default is ``tilexr_b200.ops.gemm``.  Tests inject a plain PyTorch stand-in."""

    def __init__(self, comm, cfg: TPMlpConfig, w13: torch.Tensor, w2: torch.Tensor, ops=None, quant_ops=None):
        super().__init__()
        world = comm.world_size
        if cfg.tokens % world != 0 or cfg.ffn % world != 0:
            raise ValueError("tokens and ffn must divide by the number of ranks")
        f_loc = cfg.ffn // world
        if tuple(w13.shape) != (2 * f_loc, cfg.hidden) or tuple(w2.shape) != (cfg.hidden, f_loc):
            raise ValueError(f"expected w13 [{2 * f_loc}, {cfg.hidden}] and w2 [{cfg.hidden}, {f_loc}]")
        if ops is None:
            from ..ops import gemm as ops
        if quant_ops is None and cfg.fp8_block:
            from ..ops import quant as quant_ops
        self.comm, self.cfg, self.ops, self.quant = comm, cfg, ops, quant_ops
        self.f_loc = f_loc
        if cfg.fp8_block:
            if (cfg.tokens // world) % 256 != 0 or cfg.hidden % 512 != 0 or f_loc % 128 != 0:
                raise ValueError("block-scaled fp8 needs 256-row shards, hidden a multiple of 512 and ffn / world a multiple of 128")
            self.w13, self.s13 = ops.quantize_weight_128x128(w13.float())
            self.w2, self.s2 = ops.quantize_weight_128x128(w2.float())
            self.stage_rows = comm.symm_empty([cfg.tokens, cfg.hidden], torch.float8_e4m3fn)
            self.stage_scales = comm.symm_empty([cfg.tokens, cfg.hidden // 128], torch.float32)
        else:
            self.w13 = torch.nn.Parameter(w13.to(cfg.dtype), requires_grad=False)
            self.w2 = torch.nn.Parameter(w2.to(cfg.dtype), requires_grad=False)
            self.stage_rows = comm.symm_empty([cfg.tokens, cfg.hidden], cfg.dtype)
        self.stage_out = comm.symm_empty([cfg.tokens, cfg.hidden], cfg.dtype)

    @torch.no_grad()
    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        rows = cfg.tokens // self.comm.world_size
        if tuple(x_shard.shape) != (rows, cfg.hidden):
            raise ValueError(f"expected this rank's [{rows}, {cfg.hidden}] rows")
        if cfg.fp8_block:
            qx, sx = self.quant.fp8_quant_1x128(x_shard)
            gu = self.ops.all_gather_matmul_fp8_block(self.comm, qx, sx, self.stage_rows, self.stage_scales, self.w13, self.s13, cfg.dtype)
        else:
            gu = self.ops.all_gather_matmul(self.comm, x_shard, self.w13, self.stage_rows)
        act = (torch.nn.functional.silu(gu[:, :self.f_loc].float()) * gu[:, self.f_loc:].float()).to(cfg.dtype)
        if cfg.fp8_block:
            qa, sa = self.quant.fp8_quant_1x128(act)
            return self.ops.matmul_reduce_scatter_fp8_block(self.comm, qa, sa, self.w2, self.s2, self.stage_out, cfg.dtype)
        return self.ops.matmul_reduce_scatter(self.comm, act, self.w2, self.stage_out)
