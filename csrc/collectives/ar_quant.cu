// All-reduce of int8 payloads with dequantisation:  out[i] = sum over ranks of (x_r[i] + offset) * scale[i % scaleCount]
// in fp16 or bf16.  The payload crosses NVLink as int8 (half the bytes of a 16-bit all-reduce in the first phase); the
// owner of a slice dequantises each rank's values in fp32, sums them in rank order and rounds once.
//
// One cooperative kernel, two hops:
//   1. every rank pushes slice p of its int8 input into rank p's window (region [source]) and raises one flag per
//      block portion;
//   2. the owner waits for the portion from every source, dequantises, sums, writes its own output slice and pushes the
//      16-bit result into every peer's window (region [owner]) with a second flag; peers copy it out.
// Block b of every rank works on portion b of every slice, so a flag is per (source, block).  All waits are bounded.
//
// Reference: AllReduceOneShot/TwoShot/BigData<half, int8_t> with a scalar or per-channel scale and an offset
// (src/collectives/kernels/allreduce_quant.h:15-216, selected by extraFlag QUANT_FP16 in kernels/lccl_op.h:168-181).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <numeric>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "tilexr_collectives.h"
#include "tilexr_launch.h"
#include "tilexr_log.h"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr unsigned ARQ_THREADS = 256;

struct ArQuantArgs {
    const uint8_t *x;        // int8 [count]
    uint8_t *out;            // 16-bit [count]
    const uint8_t *scale;    // 16-bit [scaleCount]
    CommArgs *comm;
    int64_t magic;
    uint64_t sliceVecs;      // 16-element vectors per rank slice (the last slice may be shorter)
    uint64_t totalVecs;
    uint64_t planeBOff;      // byte offset of the result regions inside a data half
    uint32_t scaleCount;
    uint32_t isBf16;
    float offset;
    uint32_t pad;
};

__device__ __forceinline__ float ToFloat16Bit(uint16_t v, bool bf16)
{
    return bf16 ? __uint_as_float(static_cast<uint32_t>(v) << 16) : __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ uint16_t From32(float f, bool bf16)
{
    return bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(f)) : __half_as_ushort(__float2half_rn(f));
}

__device__ __forceinline__ uint64_t *FlagOf(const ArQuantArgs &a, int plane, int owner, int src)
{
    return FlagSlot(a.comm, owner, plane + static_cast<int64_t>(src) * TILEXR_FLAGS_PER_PAIR + blockIdx.x);
}

__device__ void ArQuantBody(const ArQuantArgs &a)
{
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_ALL_REDUCE, static_cast<int64_t>(a.totalVecs) * 16, true);
    CommArgs *comm = a.comm;
    const int R = comm->rankSize, rank = comm->rank;
    const uint32_t epoch = w.epoch;
    const int tid = threadIdx.x;
    const bool bf16 = a.isBf16 != 0;
    const uint64_t per = (a.sliceVecs + gridDim.x - 1) / gridDim.x;     // vectors of a slice handled by one block
    const uint64_t p0 = per * blockIdx.x;
    const auto sliceLen = [&](int r) -> uint64_t {
        const uint64_t first = a.sliceVecs * r;
        return first >= a.totalVecs ? 0 : (a.totalVecs - first < a.sliceVecs ? a.totalVecs - first : a.sliceVecs);
    };
    const auto portion = [&](int r, uint64_t *first, uint64_t *n) {
        const uint64_t len = sliceLen(r);
        *first = p0 < len ? p0 : len;
        *n = len - *first < per ? len - *first : per;
    };
    if (ok) {
        // 1. my int8 values of slice p go to rank p
        for (int i = 1; i < R; ++i) {
            const int p = (rank + i) % R;
            uint64_t first, n;
            portion(p, &first, &n);
            const uint8_t *src = a.x + (a.sliceVecs * p + first) * 16;
            uint8_t *dst = DataHalf(comm, p, epoch) + (a.sliceVecs * rank + first) * 16;
            for (uint64_t v = tid; v < n; v += ARQ_THREADS) st_vec16(dst + v * 16, ld_vec16_stream(src + v * 16));
        }
        __syncthreads();
        if (tid < R && tid != rank) {
            fence_acq_rel_sys();
            SetFlag(FlagOf(a, TILEXR_FLAG_DATA_BASE, tid, rank), epoch, 1);
        }
        // 2. my slice: dequantise every rank's values, sum in rank order, fan out
        bool got = true;
        if (tid < R && tid != rank) got = WaitFlagGE(w, FlagOf(a, TILEXR_FLAG_DATA_BASE, rank, tid), 1, tid, blockIdx.x);
        ok = BlockBroadcastOk(got);
    }
    if (ok) {
        uint64_t first, n;
        portion(rank, &first, &n);
        const uint8_t *half = DataHalf(comm, rank, epoch);
        for (uint64_t v = tid; v < n; v += ARQ_THREADS) {
            const uint64_t vec = a.sliceVecs * rank + first + v;       // index of this 16-element vector in the message
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
            for (int s = 0; s < R; ++s) {
                const uint8_t *src = s == rank ? a.x + vec * 16 : half + (a.sliceVecs * s + first + v) * 16;
                const Vec16 q = ld_vec16_stream(src);
                const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int8_t b = static_cast<int8_t>((words[j >> 2] >> ((j & 3) * 8)) & 0xffu);
                    const uint64_t e = vec * 16 + j;
                    const float sc = ToFloat16Bit(reinterpret_cast<const uint16_t *>(a.scale)[a.scaleCount == 1 ? 0 : e % a.scaleCount], bf16);
                    // separate roundings (no fused multiply-add): the result equals a plain fp32 evaluation in rank order
                    acc[j] = __fadd_rn(acc[j], __fmul_rn(static_cast<float>(b) + a.offset, sc));
                }
            }
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o[j] = static_cast<uint32_t>(From32(acc[2 * j], bf16)) | (static_cast<uint32_t>(From32(acc[2 * j + 1], bf16)) << 16);
            }
            const Vec16 lo{o[0], o[1], o[2], o[3]}, hi{o[4], o[5], o[6], o[7]};
            st_vec16(a.out + vec * 32, lo);
            st_vec16(a.out + vec * 32 + 16, hi);
            for (int i = 1; i < R; ++i) {
                const int p = (rank + i) % R;
                uint8_t *dst = DataHalf(comm, p, epoch) + a.planeBOff + (a.sliceVecs * rank + first + v) * 32;
                st_vec16(dst, lo);
                st_vec16(dst + 16, hi);
            }
        }
        __syncthreads();
        if (tid < R && tid != rank) {
            fence_acq_rel_sys();
            SetFlag(FlagOf(a, TILEXR_FLAG_ACK_BASE, tid, rank), epoch, 1);
        }
        // 3. the other slices come back summed
        bool got = true;
        if (tid < R && tid != rank) got = WaitFlagGE(w, FlagOf(a, TILEXR_FLAG_ACK_BASE, rank, tid), 1, tid, blockIdx.x);
        ok = BlockBroadcastOk(got);
    }
    if (ok) {
        const uint8_t *half = DataHalf(comm, rank, epoch) + a.planeBOff;
        for (int i = 1; i < R; ++i) {
            const int owner = (rank + i) % R;
            uint64_t first, n;
            portion(owner, &first, &n);
            const uint64_t base = (a.sliceVecs * owner + first) * 32;
            for (uint64_t v = tid; v < n * 2; v += ARQ_THREADS) st_vec16(a.out + base + v * 16, ld_vec16_stream(half + base + v * 16));
        }
    }
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRAllReduceQuantKernel, ArQuantArgs, ArQuantBody, ARQ_THREADS)

long EnvLongQ(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

} // namespace
} // namespace TileXR

using namespace TileXR;

extern "C" {

int TileXRAllReduceQuant(const void *sendBuf, void *recvBuf, int64_t count, TileXRDataType outType, const void *scale,
                         int64_t scaleCount, float offset, TileXRCommPtr comm, TileXRStream stream)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_ERROR_NOT_SUPPORT;
    if (sendBuf == nullptr || recvBuf == nullptr || scale == nullptr || count <= 0 || count % 16 != 0 || scaleCount <= 0 ||
        (scaleCount > 1 && count % scaleCount != 0) || scaleCount > 0x7fffffff ||
        (outType != TILEXR_DATA_TYPE_FP16 && outType != TILEXR_DATA_TYPE_BFP16) || reinterpret_cast<uintptr_t>(sendBuf) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(recvBuf) % 16 != 0) {
        TILEXR_LOG(ERROR) << "quantised all-reduce: int8 input of a multiple of 16 elements (16-byte aligned), fp16 or bf16 output, "
                          << "scaleCount 1 or a divisor of count (count " << count << ", scaleCount " << scaleCount << ")";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const int R = hostArgs->rankSize;
    // a launch holds int8 slices (1 byte / element) and 16-bit results (2 bytes / element) in one data half
    if (hostArgs->dataHalfBytes < 256 + 48ull * R * 2) return TILEXR_ERROR_PARA_CHECK_FAIL;
    const uint64_t maxVecs = ((hostArgs->dataHalfBytes - 256) / 48 / static_cast<uint64_t>(R)) * static_cast<uint64_t>(R) - static_cast<uint64_t>(R);
    const int ranksPerDevice = (hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? R : 1;
    unsigned maxGrid = 0;
    ret = MaxCooperativeGrid(comm, TileXRAllReduceQuantKernelEntry, ARQ_THREADS, 0, ranksPerDevice, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t totalVecs = static_cast<uint64_t>(count) / 16;
    // scale indices restart with every launch: cut launches at multiples of scaleCount elements
    uint64_t stepVecs = maxVecs;
    if (scaleCount > 1) {
        const uint64_t lcmVecs = static_cast<uint64_t>(scaleCount) / std::gcd<uint64_t, uint64_t>(static_cast<uint64_t>(scaleCount), 16);
        if (lcmVecs > maxVecs) {
            TILEXR_LOG(ERROR) << "quantised all-reduce: one period of the scales does not fit a launch";
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
        stepVecs = maxVecs / lcmVecs * lcmVecs;
    }
    for (uint64_t done = 0; done < totalVecs; done += stepVecs) {
        const uint64_t n = std::min(stepVecs, totalVecs - done);
        ArQuantArgs a;
        std::memset(&a, 0, sizeof(a));
        a.x = static_cast<const uint8_t *>(sendBuf) + done * 16;
        a.out = static_cast<uint8_t *>(recvBuf) + done * 32;
        a.scale = static_cast<const uint8_t *>(scale);
        a.comm = reinterpret_cast<CommArgs *>(devArgs);
        a.totalVecs = n;
        a.sliceVecs = (n + R - 1) / R;
        a.planeBOff = (a.sliceVecs * R * 16 + 255) / 256 * 256;
        a.scaleCount = static_cast<uint32_t>(scaleCount);
        a.isBf16 = outType == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
        a.offset = offset;
        int64_t magic = 0;
        ret = TileXRCommNextMagic(comm, &magic);
        if (ret != TILEXR_SUCCESS) return ret;
        a.magic = magic;
        const uint64_t sliceBytes = a.sliceVecs * 16;
        long want = sliceBytes <= (64u << 10) ? 8 : sliceBytes <= (1u << 20) ? 32 : 96;
        want = EnvLongQ("TILEXR_AR_QUANT_BLOCKS", want);
        const unsigned grid = std::max(1u, std::min<unsigned>({static_cast<unsigned>(std::min<long>(want, TILEXR_FLAGS_PER_PAIR)), maxGrid,
                                                                static_cast<unsigned>(std::min<uint64_t>(a.sliceVecs, 1u << 20))}));
        LaunchConfig cfg{grid, ARQ_THREADS, 0, true};
        ret = LaunchKernel(comm, TileXRAllReduceQuantKernelEntry, &a, cfg, stream);
        if (ret != TILEXR_SUCCESS) return ret;
    }
    return TILEXR_SUCCESS;
}

} // extern "C"
