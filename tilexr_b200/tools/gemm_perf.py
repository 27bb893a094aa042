"""tcgen05 GEMM against cuBLAS (torch.matmul) on one GPU: CUDA-event medians with an L2 flush between
iterations, bit comparison of the results.

    python -m tilexr_b200.tools.gemm_perf [--shapes 4096x4096x4096,8192x8192x8192] [--iters 8]

`TILEXR_GEMM_PAIR=0` selects the one-CTA kernel, `TILEXR_GEMM_GROUP=n` the raster group of the CTA-pair kernel.
"""
from __future__ import annotations

import argparse
import json

import torch

import tilexr_b200 as txr

DEFAULT = "4096x4096x4096,8192x8192x8192,8192x28672x8192,8192x8192x14336,16384x7168x2048"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default=DEFAULT, help="comma separated MxNxK")
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float8_e4m3fn", "float8_e5m2", "fp8_block"],
                    help="operand type; the fp8 types run the kind::f8f6f4 path against torch._scaled_mm (cuBLASLt); fp8_block "
                         "is e4m3 with fp32 block scales (1 x 128 activations, 128 x 128 weights) against torch._scaled_mm "
                         "with the same scales where this torch / cuBLASLt accepts them, else against its per-tensor fp8 GEMM")
    ap.add_argument("--groups", type=int, default=0,
                    help="grouped GEMM: the M rows split evenly over this many groups with one [N, K] weight each (bf16), one launch "
                         "with the row counts on the device, against torch.bmm (cuBLAS batched) on the same equal split; "
                         "--swiglu adds the fused activation (N counts gate and up rows) against bmm + silu * mul")
    ap.add_argument("--swiglu", action="store_true")
    args = ap.parse_args()
    block = args.dtype == "fp8_block"
    dtype = torch.float8_e4m3fn if block else getattr(torch, args.dtype)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")       # larger than the 126 MB L2

    def median_ms(fn):
        for _ in range(3):
            fn()
        times = []
        for _ in range(args.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        times.sort()
        return times[len(times) // 2]

    for shape in args.shapes.split(","):
        m, n, k = (int(v) for v in shape.split("x"))
        a = (torch.randn(m, k, device="cuda") * 0.5).to(dtype)
        b = (torch.randn(n, k, device="cuda") * 0.5).to(dtype)
        baseline = "torch.matmul (cuBLAS)"
        if args.groups > 0:
            G = args.groups
            per = m // G
            a = a[:per * G].contiguous()
            wg = (torch.randn(G, n, k, device="cuda") * 0.2).to(dtype)
            counts = torch.full((G,), per, dtype=torch.int64, device="cuda")
            epi = txr.gemm.EPILOGUE_SWIGLU if args.swiglu else txr.gemm.EPILOGUE_STORE
            out = torch.empty(per * G, n // 2 if args.swiglu else n, dtype=dtype, device="cuda")
            run_ours = lambda: txr.gemm.grouped_matmul(a, wg, counts, epilogue=epi, out=out)
            a3, wt = a.view(G, per, k), wg.transpose(1, 2)
            if args.swiglu:
                def run_lib():
                    p = torch.bmm(a3, wt)
                    return torch.nn.functional.silu(p[..., 0::2]) * p[..., 1::2]
                baseline = "torch.bmm + silu * mul (cuBLAS batched, equal groups)"
            else:
                run_lib = lambda: torch.bmm(a3, wt)
                baseline = "torch.bmm (cuBLAS batched, equal groups)"
            ours, cublas = median_ms(run_ours), median_ms(run_lib)
            c, ref = run_ours().float(), run_lib().reshape(per * G, -1).float()
            torch.cuda.synchronize()
            flops = 2.0 * per * G * n * k
            print(json.dumps({"shape": [per * G, n, k], "groups": G, "swiglu": args.swiglu, "baseline": baseline, "ours_us": ours * 1e3,
                              "cublas_us": cublas * 1e3, "ours_tflops": flops / ours / 1e9, "cublas_tflops": flops / cublas / 1e9,
                              "ratio": cublas / ours, "max_abs_diff": (c - ref).abs().max().item()}), flush=True)
            continue
        if block:
            qa, sa = txr.quant.fp8_quant_1x128((torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16))
            qb, sb = txr.gemm.quantize_weight_128x128(torch.randn(n, k, device="cuda") * 0.5)
            run_ours = lambda: txr.gemm.matmul_fp8_block(qa, sa, qb, sb)
            # cuBLASLt's block-wise modes want the activation scales K-major-outer ([M, K/128] stored column-major) and the
            # weight scales as [K/128, N/128]; whether they exist depends on the torch / cuBLASLt build
            sa_t = sa.t().contiguous().t()
            sb_t = sb.t().contiguous()
            run_lib = lambda: torch._scaled_mm(qa, qb.t(), scale_a=sa_t, scale_b=sb_t, out_dtype=torch.bfloat16)
            baseline = "torch._scaled_mm block-wise (cuBLASLt)"
            try:
                run_lib()
                torch.cuda.synchronize()
            except Exception:
                one = torch.tensor(1.0, device="cuda")
                run_lib = lambda: torch._scaled_mm(qa, qb.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
                baseline = "torch._scaled_mm per-tensor (cuBLASLt; block-wise scales are not accepted by this build)"
        elif dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            baseline = "torch._scaled_mm per-tensor (cuBLASLt)"
            one = torch.tensor(1.0, device="cuda")
            run_ours = lambda: txr.gemm.matmul_fp8(a, b, 1.0)
            run_lib = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        else:
            run_ours = lambda: txr.gemm.matmul(a, b)
            run_lib = lambda: torch.matmul(a, b.t())
        ours = median_ms(run_ours)
        cublas = median_ms(run_lib)
        c, ref = run_ours(), run_lib()
        torch.cuda.synchronize()
        flops = 2.0 * m * n * k
        identical = bool(torch.equal(c, ref)) if not block else None
        close = None
        if block:
            close = bool(torch.allclose(c.float(), ref.float(), rtol=2e-2, atol=2e-2 * ref.float().abs().max().item())) if "block-wise" in baseline and "not accepted" not in baseline else None
        print(json.dumps({"shape": [m, n, k], "baseline": baseline, "close_to_baseline": close, "ours_us": ours * 1e3, "cublas_us": cublas * 1e3, "ours_tflops": flops / ours / 1e9,
                          "cublas_tflops": flops / cublas / 1e9, "ratio": cublas / ours, "identical_bits": identical}),
              flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
