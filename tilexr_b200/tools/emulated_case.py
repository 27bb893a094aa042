"""Runs one operator a few times on an emulated world (R ranks sharing one GPU, one cooperative
launch per call).  Small and self-contained: meant for profilers and for trying the library on
a single GPU.

    python -m tilexr_b200.tools.emulated_case --op all_gather --ranks 4 --mbytes 64 --launches 3
    python -m tilexr_b200.tools.emulated_case --op ep --ranks 4 --tokens 1024 --hidden 7168
    python -m tilexr_b200.tools.emulated_case --op ar_norm --ranks 8 --tokens 64 --hidden 8192
    python -m tilexr_b200.tools.emulated_case --op gemm --m 4096 --n 4096 --k 4096
    python -m tilexr_b200.tools.emulated_case --op gemm_fp8_block --m 4096 --n 4096 --k 4096
    python -m tilexr_b200.tools.emulated_case --op grouped_gemm --m 8192 --n 4096 --k 2048 --groups 8
    python -m tilexr_b200.tools.emulated_case --op ag_gemm_fp8_block --ranks 2 --m 4096 --n 4096 --k 4096
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--op", default="all_gather",
                   choices=["all_gather", "all_to_all", "all_reduce", "reduce_scatter", "ep", "ar_norm", "gemm", "ag_gemm", "gemm_rs", "gemm_fp8_block",
                            "grouped_gemm", "ag_gemm_fp8_block", "gemm_rs_fp8_block"])
    p.add_argument("--groups", type=int, default=8, help="grouped_gemm: experts; the m rows are split evenly, SwiGLU epilogue on")
    p.add_argument("--ranks", type=int, default=4)
    p.add_argument("--mbytes", type=float, default=64.0, help="per-rank message for the collectives")
    p.add_argument("--tokens", type=int, default=1024)
    p.add_argument("--hidden", type=int, default=7168)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--m", type=int, default=4096)
    p.add_argument("--n", type=int, default=4096)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--launches", type=int, default=3)
    p.add_argument("--buffer-mb", type=int, default=512)
    a = p.parse_args(argv)
    import tilexr_b200 as txr
    from tilexr_b200.ops import collectives as coll
    from tilexr_b200.ops import ep, quant

    R = a.ranks
    times = []

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1000.0)
        return out

    g = torch.Generator(device="cuda").manual_seed(0)
    if a.op == "gemm":
        x = (torch.randn(a.m, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        w = (torch.randn(a.n, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        for _ in range(a.launches):
            timed(lambda: txr.gemm.matmul(x, w))
        print(json.dumps({"op": a.op, "us": times, "tflops": 2.0 * a.m * a.n * a.k / times[-1] / 1e6}))
        return 0

    if a.op == "gemm_fp8_block":
        qx, sx = quant.fp8_quant_1x128((torch.randn(a.m, a.k, device="cuda", generator=g) * 0.5).to(torch.bfloat16))
        qw, sw = txr.gemm.quantize_weight_128x128(torch.randn(a.n, a.k, device="cuda", generator=g) * 0.5)
        for _ in range(a.launches):
            timed(lambda: txr.gemm.matmul_fp8_block(qx, sx, qw, sw))
        print(json.dumps({"op": a.op, "us": times, "tflops": 2.0 * a.m * a.n * a.k / times[-1] / 1e6}))
        return 0
    if a.op == "grouped_gemm":
        per = a.m // a.groups
        x = (torch.randn(per * a.groups, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        w = (torch.randn(a.groups, a.n, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        counts = torch.full((a.groups,), per, dtype=torch.int64, device="cuda")
        for _ in range(a.launches):
            timed(lambda: txr.gemm.grouped_matmul(x, w, counts, epilogue=txr.gemm.EPILOGUE_SWIGLU))
        print(json.dumps({"op": a.op, "us": times, "tflops": 2.0 * per * a.groups * a.n * a.k / times[-1] / 1e6}))
        return 0

    world = txr.init_emulated_world(R, device=0, buffer_mb=a.buffer_mb)
    n = int(a.mbytes * (1 << 20)) // 2
    if a.op in ("all_gather", "all_to_all", "all_reduce", "reduce_scatter"):
        n = n // R * R
        xs = [(torch.rand(n, device="cuda", generator=g) - 0.5).to(torch.bfloat16) for _ in range(R)]
        fn = {"all_gather": txr.all_gather, "all_to_all": txr.all_to_all, "all_reduce": txr.all_reduce,
              "reduce_scatter": txr.reduce_scatter}[a.op]
        for _ in range(a.launches):
            timed(lambda: world.run(lambda c, r: fn(c, xs[r])))
    elif a.op == "ep":
        xs = [torch.randn(a.tokens, a.hidden, device="cuda", generator=g).to(torch.bfloat16) for _ in range(R)]
        lg = [torch.randn(a.tokens, a.experts, device="cuda", generator=g) for _ in range(R)]
        cap = a.tokens * a.topk * 2
        recv = world.symm_empty((cap, a.hidden), torch.float8_e4m3fn)
        for _ in range(a.launches):
            ds = timed(lambda: world.run(lambda c, r: ep.dispatch(c, xs[r], gate_logits=lg[r], num_experts=a.experts, top_k=a.topk,
                                                                   quant_mode=ep.QUANT_FP8_1X128, score_func=1, max_recv_rows=cap,
                                                                   expand_x_out=recv[r])))
            rows = [quant.fp8_dequant_1x128(d.expand_x, d.dynamic_scales, torch.bfloat16) for d in ds]
            timed(lambda: world.run(lambda c, r: ep.combine(c, rows[r], ds[r], expert_scales=ds[r].topk_weights)))
    elif a.op == "ar_norm":
        xs = [torch.randn(a.tokens, a.hidden, device="cuda", generator=g).to(torch.bfloat16) for _ in range(R)]
        res = [torch.randn(a.tokens, a.hidden, device="cuda", generator=g).to(torch.bfloat16) for _ in range(R)]
        gamma = torch.ones(a.hidden, device="cuda", dtype=torch.bfloat16)
        for _ in range(a.launches):
            timed(lambda: world.run(lambda c, r: coll.all_reduce_rmsnorm(c, xs[r], gamma, 1e-6, residual=res[r])))
    elif a.op == "ag_gemm":
        rows = a.m // R // 128 * 128
        sh = [(torch.randn(rows, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16) for _ in range(R)]
        w = [(torch.randn(a.n, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16) for _ in range(R)]
        st = world.symm_empty((R * rows, a.k), torch.bfloat16)
        for _ in range(a.launches):
            timed(lambda: world.run(lambda c, r: txr.gemm.all_gather_matmul(c, sh[r], w[r], st[r])))
    elif a.op == "gemm_rs":
        rows = a.m // R // 128 * 128
        x = [(torch.randn(R * rows, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16) for _ in range(R)]
        w = [(torch.randn(a.n, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16) for _ in range(R)]
        st = world.symm_empty((R * rows, a.n), torch.bfloat16)
        for _ in range(a.launches):
            timed(lambda: world.run(lambda c, r: txr.gemm.matmul_reduce_scatter(c, x[r], w[r], st[r])))
    elif a.op in ("ag_gemm_fp8_block", "gemm_rs_fp8_block"):
        rows = a.m // R // 256 * 256
        total = R * rows
        ops = []
        for r in range(R):
            acts = (torch.randn(rows if a.op == "ag_gemm_fp8_block" else total, a.k, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
            ops.append(quant.fp8_quant_1x128(acts) + txr.gemm.quantize_weight_128x128(torch.randn(a.n, a.k, device="cuda", generator=g) * 0.5))
        if a.op == "ag_gemm_fp8_block":
            st_q = world.symm_empty((total, a.k), torch.float8_e4m3fn)
            st_s = world.symm_empty((total, a.k // 128), torch.float32)
            for _ in range(a.launches):
                timed(lambda: world.run(lambda c, r: txr.gemm.all_gather_matmul_fp8_block(c, ops[r][0], ops[r][1], st_q[r], st_s[r], ops[r][2], ops[r][3])))
        else:
            st = world.symm_empty((total, a.n), torch.bfloat16)
            for _ in range(a.launches):
                timed(lambda: world.run(lambda c, r: txr.gemm.matmul_reduce_scatter_fp8_block(c, ops[r][0], ops[r][1], ops[r][2], ops[r][3], st[r])))
    world.check()
    print(json.dumps({"op": a.op, "ranks": R, "us": times}))
    world.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
