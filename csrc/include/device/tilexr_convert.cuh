// 16-byte vectors of 16-bit floats <-> fp32, shared by kernels that accumulate in fp32.
#ifndef TILEXR_CONVERT_CUH
#define TILEXR_CONVERT_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tilexr_platform.cuh"

namespace tilexr {

__device__ __forceinline__ void Unpack8(const Vec16 &v, bool bf16, float *f)
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (bf16) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = f2.x;
            f[2 * i + 1] = f2.y;
        }
    }
}

__device__ __forceinline__ Vec16 Pack8(const float *f, bool bf16)
{
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (bf16) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&b);
        } else {
            const __half2 h2 = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h2);
        }
    }
    return Vec16{w[0], w[1], w[2], w[3]};
}

// Sum over k (ascending, so the result does not depend on how the loop is cut) of the 16-byte column `col` of rows
// base + k * stride, k in [0, K) with bit k of `have` set; the rows are 16-bit floats (8 per column) or fp32 (4 per column).
// Up to eight rows' columns are fetched before the first is added: taken one at a time, every row costs the thread a
// memory round trip of its own, which made an 8-row reduction eight times slower than the memory allows.
__device__ __forceinline__ void SumRowsColumn(const uint8_t *base, uint64_t stride, int K, uint32_t have, uint64_t col, int elemKind,
                                              float *acc /* 8 (16-bit) or 4 (fp32) */)
{
    const int width = elemKind == 2 ? 4 : 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += 8) {
        Vec16 q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (k0 + u < K && ((have >> (k0 + u)) & 1u)) q[u] = ld_vec16_stream(base + static_cast<uint64_t>(k0 + u) * stride + col * 16);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (k0 + u < K && ((have >> (k0 + u)) & 1u)) {
                if (width == 4) {
                    acc[0] += __uint_as_float(q[u].x);
                    acc[1] += __uint_as_float(q[u].y);
                    acc[2] += __uint_as_float(q[u].z);
                    acc[3] += __uint_as_float(q[u].w);
                } else {
                    float f[8];
                    Unpack8(q[u], elemKind == 1, f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += f[j];
                }
            }
        }
    }
}

} // namespace tilexr

#endif
