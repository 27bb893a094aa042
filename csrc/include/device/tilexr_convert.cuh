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

} // namespace tilexr

#endif
