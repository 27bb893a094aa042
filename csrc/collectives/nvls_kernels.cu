// Collectives through the NVSwitch multicast object (NVLS): `multimem` loads reduce inside the switch and
// `multimem` stores land in every rank's copy of the buffer, so a rank moves its slice over NVLink once where a
// peer-to-peer kernel moves it R-1 times.
//
//   all-reduce      every rank reduces 1/R of the buffer with multimem.ld_reduce and writes the sum back with
//                   multimem.st: 2/R of the bytes leave each GPU (one-shot peer pushes: (R-1) x).
//   reduce-scatter  multimem.ld_reduce of the rank's own slice into a local output.
//   all-gather      multimem.st of the rank's shard to its place in every copy.
//   broadcast       the root's multimem.st of the whole message.
//
// The buffer is a symmetric allocation bound to a multicast object; the host passes its multicast address and
// the offset of the message in it.  Every rank calls with the same offset and count.  Blocks of the same index
// meet across ranks before the first access (the peers' inputs are in place, nobody still reads the last
// result) and after the last one (every store has landed) through flags in the communicator's windows; each
// wait is bounded and a give-up is reported through the communicator's device status.
//
// Sums accumulate in fp32 inside the switch (.acc::f32 for 16-bit types).  Each element is reduced exactly once,
// by its owner, and the owner's result is what every rank receives: all ranks hold bit-identical results.
//
// The reference reduces through its own memory route only (src/collectives/kernels/allreduce_*.h); there is
// no in-fabric reduction on its hardware.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "device/tilexr_convert.cuh"
#include "coll_kernels.cuh"
#include "tilexr_collectives.h"
#include "tilexr_launch.h"
#include "tilexr_log.h"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr unsigned NVLS_THREADS = 512;
constexpr int NVLS_UNROLL = 4;

enum NvlsMode : int32_t { NVLS_ALL_REDUCE = 0, NVLS_REDUCE_SCATTER = 1, NVLS_ALL_GATHER = 2, NVLS_BROADCAST = 3 };

struct NvlsArgs {
    uint8_t *mc;            // multicast address of the message
    const uint8_t *in;      // all-gather / broadcast: local input
    uint8_t *out;           // reduce-scatter: local output
    CommArgs *comm;
    int64_t magic;
    uint64_t vecs;          // 16-byte vectors: whole message (all-reduce, reduce-scatter, broadcast), one shard (all-gather)
    int32_t mode;
    int32_t kind;           // 0 bf16, 1 fp16, 2 fp32
    int32_t root;
    int32_t pad;
};

__device__ __forceinline__ Vec16 MultimemLdReduce(const uint8_t *p, int kind)
{
    Vec16 v;
    if (kind == 0) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    } else if (kind == 1) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    }
    return v;
}

__device__ __forceinline__ void MultimemSt(uint8_t *p, const Vec16 &v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Block b of every rank meets block b of every other rank: thread t talks to rank t.
__device__ __forceinline__ bool MeetPeers(Waiter &w, const NvlsArgs &a, uint32_t value)
{
    CommArgs *comm = a.comm;
    const int R = comm->rankSize;
    const int rank = comm->rank;
    __syncthreads();
    bool ok = true;
    const int t = threadIdx.x;
    if (t < R && t != rank) {
        fence_acq_rel_sys();
        const int64_t base = TILEXR_FLAG_OP_BASE + static_cast<int64_t>(blockIdx.x) * TILEXR_MAX_RANK_SIZE;
        SetFlag(FlagSlot(comm, t, base + rank), w.epoch, value);
        ok = WaitFlagGE(w, FlagSlot(comm, rank, base + t), value, t, base + t);
    }
    return BlockBroadcastOk(ok);
}

__device__ void NvlsBody(const NvlsArgs &a)
{
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_ALL_REDUCE, static_cast<int64_t>(a.vecs), false);
    const int R = a.comm->rankSize;
    const int rank = a.comm->rank;
    if (ok) ok = MeetPeers(w, a, 1);
    if (ok) {
        const uint64_t stride = static_cast<uint64_t>(gridDim.x) * NVLS_THREADS;
        const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * NVLS_THREADS + threadIdx.x;
        if (a.mode == NVLS_ALL_REDUCE || a.mode == NVLS_REDUCE_SCATTER) {
            const uint64_t per = (a.vecs + R - 1) / R;
            const uint64_t start = per * static_cast<uint64_t>(rank);
            const uint64_t first = start < a.vecs ? start : a.vecs;
            const uint64_t mine = (first + per < a.vecs ? first + per : a.vecs) - first;
            for (uint64_t i0 = tid; i0 < mine; i0 += stride * NVLS_UNROLL) {
                Vec16 v[NVLS_UNROLL];
#pragma unroll
                for (int q = 0; q < NVLS_UNROLL; ++q) {
                    const uint64_t i = i0 + q * stride;
                    if (i < mine) v[q] = MultimemLdReduce(a.mc + (first + i) * 16, a.kind);
                }
#pragma unroll
                for (int q = 0; q < NVLS_UNROLL; ++q) {
                    const uint64_t i = i0 + q * stride;
                    if (i < mine) {
                        if (a.mode == NVLS_ALL_REDUCE) {
                            MultimemSt(a.mc + (first + i) * 16, v[q]);
                        } else {
                            st_vec16(a.out + i * 16, v[q]);
                        }
                    }
                }
            }
        } else if (a.mode == NVLS_ALL_GATHER || rank == a.root) {
            uint8_t *dst = a.mc + (a.mode == NVLS_ALL_GATHER ? a.vecs * 16 * rank : 0);
            for (uint64_t i0 = tid; i0 < a.vecs; i0 += stride * NVLS_UNROLL) {
                Vec16 v[NVLS_UNROLL];
#pragma unroll
                for (int q = 0; q < NVLS_UNROLL; ++q) {
                    const uint64_t i = i0 + q * stride;
                    if (i < a.vecs) v[q] = ld_vec16_stream(a.in + i * 16);
                }
#pragma unroll
                for (int q = 0; q < NVLS_UNROLL; ++q) {
                    const uint64_t i = i0 + q * stride;
                    if (i < a.vecs) MultimemSt(dst + i * 16, v[q]);
                }
            }
        }
        // Every rank leaves only when all stores into its copy have been issued and fenced by their senders.
        // A reduce-scatter writes nothing remote, but its peers still read this rank's input until they arrive.
        ok = MeetPeers(w, a, 2);
    }
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRNvlsKernel, NvlsArgs, NvlsBody, NVLS_THREADS)

// ---- all-reduce + residual add + RMSNorm through the switch -----------------------------------------------------------
// y = RMSNorm(sum over ranks of x + residual) * gamma, residual <- sum + residual, for [rows, h] of 16-bit elements.
// Rows are dealt to the ranks in contiguous ranges.  The owner of a row reads it with multimem.ld_reduce (one pass
// through the switch sums all ranks' copies), adds its local residual row, normalises, and writes y and the new
// residual with multimem.st into every rank's copy: per rank rows/R x rowBytes in and 2 x that out, where the
// peer-to-peer two-shot kernel moves (R-1)/R x rows x rowBytes in and twice that out.  x, y and the residual are
// views of the symmetric buffer at the same offsets on every rank; y may be x (only a row's owner reads it).
// The sum of x leaves the switch rounded to the storage type, as NCCL's all-reduce result would be.
struct NvlsNormArgs {
    uint8_t *mcX;
    uint8_t *mcY;
    uint8_t *mcRes;            // null: no residual
    const uint8_t *resLocal;   // this rank's copy of the residual
    const uint8_t *gamma;
    CommArgs *comm;
    int64_t magic;
    float eps;
    int32_t rows;
    int32_t h;
    uint32_t rowBytes;
    uint32_t isBf16;
};

constexpr int NVLS_NORM_MAX_VECS = 4;   // 512 threads x 4 x 8 elements = 16384 columns

__device__ void NvlsNormBody(const NvlsNormArgs &a)
{
    __shared__ float sPartial[NVLS_THREADS / 32];
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_ALL_REDUCE_RMSNORM, a.rows, false);
    const int R = a.comm->rankSize;
    const int rank = a.comm->rank;
    NvlsArgs meet;
    meet.comm = a.comm;
    if (ok) ok = MeetPeers(w, meet, 1);
    if (ok) {
        const bool bf16 = a.isBf16 != 0;
        const int per = (a.rows + R - 1) / R;
        const int first = min(a.rows, per * rank);
        const int last = min(a.rows, first + per);
        const int vecs = a.rowBytes / 16;
        const int kind = bf16 ? 0 : 1;
        for (int row = first + blockIdx.x; row < last; row += gridDim.x) {
            const uint64_t off = static_cast<uint64_t>(row) * a.rowBytes;
            float vals[NVLS_NORM_MAX_VECS][8];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < NVLS_NORM_MAX_VECS; ++i) {
                const int v = i * NVLS_THREADS + threadIdx.x;
                if (v < vecs) {
                    float acc[8];
                    Unpack8(MultimemLdReduce(a.mcX + off + v * 16, kind), bf16, acc);
                    if (a.mcRes != nullptr) {
                        float r[8];
                        Unpack8(ld_vec16(a.resLocal + off + v * 16), bf16, r);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] += r[j];
                    }
                    // the sum rounded to the storage type is the new residual and the input of the norm
                    const Vec16 packed = Pack8(acc, bf16);
                    if (a.mcRes != nullptr) MultimemSt(a.mcRes + off + v * 16, packed);
                    Unpack8(packed, bf16, vals[i]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            __syncthreads();   // sPartial of the previous row is no longer read
            if ((threadIdx.x & 31) == 0) sPartial[threadIdx.x >> 5] = ss;
            __syncthreads();
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < static_cast<int>(NVLS_THREADS / 32); ++i) tot += sPartial[i];
            const float rstd = rsqrtf(tot / static_cast<float>(a.h) + a.eps);
#pragma unroll
            for (int i = 0; i < NVLS_NORM_MAX_VECS; ++i) {
                const int v = i * NVLS_THREADS + threadIdx.x;
                if (v < vecs) {
                    float g[8], o[8];
                    Unpack8(ld_vec16(a.gamma + v * 16), bf16, g);
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * g[j];
                    MultimemSt(a.mcY + off + v * 16, Pack8(o, bf16));
                }
            }
        }
        ok = MeetPeers(w, meet, 2);
    }
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRNvlsNormKernel, NvlsNormArgs, NvlsNormBody, NVLS_THREADS)

// ---- the same operations for ordinary buffers, staged through the window ---------------------------------------------
// TileXRAllReduce / ReduceScatter / AllGather / Broadcast take any device pointers.  When the communicator's
// window is bound to a multicast object they run here for large messages: the message is cut into one chunk per
// block; block c of every rank copies its chunk into the window's data half of this launch, meets block c of the
// other ranks, works on the chunk through the multicast alias of the window, and copies the result out.  Blocks
// never wait for other blocks of their own rank, so copy-in, switch traffic and copy-out of different chunks
// overlap.  The data halves alternate with the launch epoch and the prologue's guard keeps a rank from reusing a
// half that a peer may still read, so the kernels need no meeting for reuse:
//
//   all-reduce, small   copy in, ONE meeting, every rank load-reduces the whole chunk into its output;
//   all-reduce, large   copy in, meeting, rank r load-reduces part r of the chunk and multicasts the sum into the
//                       half, meeting, copy out: 2/R of the bytes leave each GPU;
//   reduce-scatter      copy in (all R slices), meeting, load-reduce the own slice's chunk into the output;
//   all-gather          multicast the shard's chunk into slot `rank` of the half, meeting, copy all slots out;
//   broadcast           the root multicasts its chunk, meeting, the others copy out.
enum NvlsWindowMode : int32_t {
    NVLS_WIN_ALL_REDUCE_ONE_SHOT = 0,
    NVLS_WIN_ALL_REDUCE_TWO_SHOT = 1,
    NVLS_WIN_REDUCE_SCATTER = 2,
    NVLS_WIN_ALL_GATHER = 3,
    NVLS_WIN_BROADCAST = 4,
};

struct NvlsWindowArgs {
    const uint8_t *in;
    uint8_t *out;
    CommArgs *comm;
    int64_t magic;
    uint64_t vecs;          // 16-byte vectors per rank's contribution: the message (all-reduce, broadcast), one slice
                            // (reduce-scatter: of R in the input), one shard (all-gather)
    int32_t mode;
    int32_t kind;           // 0 bf16, 1 fp16, 2 fp32 (reductions)
    int32_t root;
    int32_t opType;
};

__device__ __forceinline__ void CopyVecs(uint8_t *dst, const uint8_t *src, uint64_t vecs)
{
    uint64_t i = threadIdx.x;
    for (; i + 3ull * NVLS_THREADS < vecs; i += 4ull * NVLS_THREADS) {
        const Vec16 a = ld_vec16_stream(src + i * 16);
        const Vec16 b = ld_vec16_stream(src + (i + NVLS_THREADS) * 16);
        const Vec16 c = ld_vec16_stream(src + (i + 2ull * NVLS_THREADS) * 16);
        const Vec16 d = ld_vec16_stream(src + (i + 3ull * NVLS_THREADS) * 16);
        st_vec16(dst + i * 16, a);
        st_vec16(dst + (i + NVLS_THREADS) * 16, b);
        st_vec16(dst + (i + 2ull * NVLS_THREADS) * 16, c);
        st_vec16(dst + (i + 3ull * NVLS_THREADS) * 16, d);
    }
    for (; i < vecs; i += NVLS_THREADS) st_vec16(dst + i * 16, ld_vec16_stream(src + i * 16));
}

// dst (local memory or null) and mcDst (multicast address or null) receive the in-switch sum of `vecs` vectors at mcSrc.
__device__ __forceinline__ void ReduceVecs(uint8_t *dst, uint8_t *mcDst, const uint8_t *mcSrc, uint64_t vecs, int kind)
{
    for (uint64_t i0 = threadIdx.x; i0 < vecs; i0 += static_cast<uint64_t>(NVLS_THREADS) * NVLS_UNROLL) {
        Vec16 v[NVLS_UNROLL];
#pragma unroll
        for (int q = 0; q < NVLS_UNROLL; ++q) {
            const uint64_t i = i0 + static_cast<uint64_t>(q) * NVLS_THREADS;
            if (i < vecs) v[q] = MultimemLdReduce(mcSrc + i * 16, kind);
        }
#pragma unroll
        for (int q = 0; q < NVLS_UNROLL; ++q) {
            const uint64_t i = i0 + static_cast<uint64_t>(q) * NVLS_THREADS;
            if (i < vecs) {
                if (mcDst != nullptr) MultimemSt(mcDst + i * 16, v[q]);
                if (dst != nullptr) st_vec16(dst + i * 16, v[q]);
            }
        }
    }
}

__device__ __forceinline__ void MulticastVecs(uint8_t *mcDst, const uint8_t *src, uint64_t vecs)
{
    for (uint64_t i0 = threadIdx.x; i0 < vecs; i0 += static_cast<uint64_t>(NVLS_THREADS) * NVLS_UNROLL) {
        Vec16 v[NVLS_UNROLL];
#pragma unroll
        for (int q = 0; q < NVLS_UNROLL; ++q) {
            const uint64_t i = i0 + static_cast<uint64_t>(q) * NVLS_THREADS;
            if (i < vecs) v[q] = ld_vec16_stream(src + i * 16);
        }
#pragma unroll
        for (int q = 0; q < NVLS_UNROLL; ++q) {
            const uint64_t i = i0 + static_cast<uint64_t>(q) * NVLS_THREADS;
            if (i < vecs) MultimemSt(mcDst + i * 16, v[q]);
        }
    }
}

__device__ void NvlsWindowBody(const NvlsWindowArgs &a)
{
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, a.opType, static_cast<int64_t>(a.vecs), true);
    CommArgs *comm = a.comm;
    const int R = comm->rankSize;
    const int rank = comm->rank;
    const uint64_t halfOff = TILEXR_WIN_DATA_OFFSET + static_cast<uint64_t>(w.epoch & 1u) * comm->dataHalfBytes;
    uint8_t *stage = comm->peerMems[rank] + halfOff;          // this rank's copy
    uint8_t *mcStage = comm->multicastMem + halfOff;          // all ranks' copies at once
    NvlsArgs meet;
    meet.comm = comm;
    // chunk of this block: vectors [c0, c0 + n) of every rank's contribution
    const uint64_t per = (a.vecs + gridDim.x - 1) / gridDim.x;
    const uint64_t c0 = min(a.vecs, per * blockIdx.x);
    const uint64_t n = min(a.vecs - c0, per);
    if (ok) {
        switch (a.mode) {
            case NVLS_WIN_ALL_REDUCE_ONE_SHOT: {
                CopyVecs(stage + c0 * 16, a.in + c0 * 16, n);
                ok = MeetPeers(w, meet, 1);
                if (ok) ReduceVecs(a.out + c0 * 16, nullptr, mcStage + c0 * 16, n, a.kind);
                break;
            }
            case NVLS_WIN_ALL_REDUCE_TWO_SHOT: {
                CopyVecs(stage + c0 * 16, a.in + c0 * 16, n);
                ok = MeetPeers(w, meet, 1);
                if (ok) {
                    const uint64_t part = (n + R - 1) / R;
                    const uint64_t p0 = min(n, part * rank);
                    const uint64_t pn = min(n - p0, part);
                    // the rank's own output gets its part straight from the registers
                    ReduceVecs(a.out + (c0 + p0) * 16, mcStage + (c0 + p0) * 16, mcStage + (c0 + p0) * 16, pn, a.kind);
                    ok = MeetPeers(w, meet, 2);
                    if (ok) {
                        if (p0 > 0) CopyVecs(a.out + c0 * 16, stage + c0 * 16, p0);
                        if (p0 + pn < n) CopyVecs(a.out + (c0 + p0 + pn) * 16, stage + (c0 + p0 + pn) * 16, n - p0 - pn);
                    }
                }
                break;
            }
            case NVLS_WIN_REDUCE_SCATTER: {
                for (int s = 0; s < R; ++s) CopyVecs(stage + (static_cast<uint64_t>(s) * a.vecs + c0) * 16, a.in + (static_cast<uint64_t>(s) * a.vecs + c0) * 16, n);
                ok = MeetPeers(w, meet, 1);
                if (ok) ReduceVecs(a.out + c0 * 16, nullptr, mcStage + (static_cast<uint64_t>(rank) * a.vecs + c0) * 16, n, a.kind);
                break;
            }
            case NVLS_WIN_ALL_GATHER: {
                MulticastVecs(mcStage + (static_cast<uint64_t>(rank) * a.vecs + c0) * 16, a.in + c0 * 16, n);
                ok = MeetPeers(w, meet, 1);
                if (ok) {
                    for (int s = 0; s < R; ++s) {
                        const uint64_t off = (static_cast<uint64_t>(s) * a.vecs + c0) * 16;
                        if (s == rank) {
                            if (a.out + off != a.in + c0 * 16) CopyVecs(a.out + off, a.in + c0 * 16, n);
                        } else {
                            CopyVecs(a.out + off, stage + off, n);
                        }
                    }
                }
                break;
            }
            default: {   // broadcast: in == out == the caller's buffer
                if (rank == a.root) MulticastVecs(mcStage + c0 * 16, a.in + c0 * 16, n);
                ok = MeetPeers(w, meet, 1);
                if (ok && rank != a.root) CopyVecs(a.out + c0 * 16, stage + c0 * 16, n);
                break;
            }
        }
    }
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRNvlsWindowKernel, NvlsWindowArgs, NvlsWindowBody, NVLS_THREADS)

long EnvLongNvls(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

int Launch(int mode, void *mc, const void *in, void *out, uint64_t bytes, TileXRDataType dtype, int root, TileXRCommPtr comm,
           TileXRStream stream)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    // Ranks of an emulated world share one GPU and a host-memory communicator has none: neither has a switch between them.
    if (hostArgs->extraFlag & (TILEXR_FLAG_HOST_MEMORY | TILEXR_FLAG_EMULATED)) return TILEXR_ERROR_NOT_SUPPORT;
    int kind;
    switch (dtype) {
        case TILEXR_DATA_TYPE_BFP16: kind = 0; break;
        case TILEXR_DATA_TYPE_FP16: kind = 1; break;
        case TILEXR_DATA_TYPE_FP32: kind = 2; break;
        default:
            if (mode == NVLS_ALL_GATHER || mode == NVLS_BROADCAST) { kind = 2; break; }   // plain bytes
            TILEXR_LOG(ERROR) << "nvls: reductions take bf16, fp16 or fp32 (dtype " << dtype << ")";
            return TILEXR_ERROR_NOT_SUPPORT;
    }
    const int R = hostArgs->rankSize;
    if (mc == nullptr || bytes == 0 || bytes % 16 != 0 || reinterpret_cast<uintptr_t>(mc) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(in) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0 || root < 0 || root >= R ||
        (mode == NVLS_ALL_GATHER && in == nullptr) || (mode == NVLS_BROADCAST && hostArgs->rank == root && in == nullptr) || (mode == NVLS_REDUCE_SCATTER && out == nullptr)) {
        TILEXR_LOG(ERROR) << "nvls: bad arguments (mode " << mode << ", bytes " << bytes << "); addresses and sizes are multiples of 16";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    NvlsArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mc = static_cast<uint8_t *>(mc);
    a.in = static_cast<const uint8_t *>(in);
    a.out = static_cast<uint8_t *>(out);
    a.comm = reinterpret_cast<CommArgs *>(devArgs);
    a.vecs = bytes / 16;
    a.mode = mode;
    a.kind = kind;
    a.root = root;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    unsigned maxGrid = 0;
    ret = MaxCooperativeGrid(comm, TileXRNvlsKernelEntry, NVLS_THREADS, 0, 1, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    // Work of one rank: its slice for the reducing modes, its whole input for the storing ones.
    const uint64_t mine = (mode == NVLS_ALL_REDUCE || mode == NVLS_REDUCE_SCATTER) ? bytes / R : bytes;
    long want = mine <= (128u << 10) ? 8 : mine <= (2u << 20) ? 32 : 96;
    want = EnvLongNvls("TILEXR_NVLS_BLOCKS", want);
    const unsigned grid = std::max(1u, std::min<unsigned>(static_cast<unsigned>(std::min<long>(want, TILEXR_FLAGS_PER_PAIR)), maxGrid));
    LaunchConfig cfg{grid, NVLS_THREADS, 0, true};
    return LaunchKernel(comm, TileXRNvlsKernelEntry, &a, cfg, stream);
}

} // namespace

// Runs `op` of the plain collective API through the window's multicast alias, or says NOT_SUPPORT so that the
// caller takes the peer-to-peer kernels (no multicast object, message too small or too large for a data half,
// dtype or reduce op the switch cannot do, misaligned buffers).  `count` as in the API: elements of the whole
// vector (all-reduce, broadcast), of one output slice (reduce-scatter), of one shard (all-gather).
int NvlsWindowCollective(int kind, const void *in, void *out, int64_t count, TileXRDataType dtype, int reduceOp, int root,
                         TileXRCommPtr comm, TileXRStream stream)
{
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    if (comm == nullptr || TileXRGetCommArgsHost(comm, &hostArgs) != TILEXR_SUCCESS || TileXRGetCommArgsDev(comm, &devArgs) != TILEXR_SUCCESS) {
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    if ((hostArgs->extraFlag & TILEXR_FLAG_NVLS) == 0 || hostArgs->multicastMem == nullptr || hostArgs->rankSize < 2) return TILEXR_ERROR_NOT_SUPPORT;
    if (EnvLongNvls("TILEXR_NVLS_AUTO", 1) == 0) return TILEXR_ERROR_NOT_SUPPORT;
    const int R = hostArgs->rankSize;
    const uint64_t bytes = static_cast<uint64_t>(count) * TileXRDataTypeSize(dtype);
    const bool reduces = kind == COLL_KIND_ALL_REDUCE || kind == COLL_KIND_REDUCE_SCATTER;
    int ek = 2;
    if (reduces) {
        if (reduceOp != TILEXR_REDUCE_SUM) return TILEXR_ERROR_NOT_SUPPORT;
        // the order in which the switch adds the ranks' values is not ours to fix
        if (hostArgs->extraFlag & TILEXR_FLAG_DETERMINISTIC) return TILEXR_ERROR_NOT_SUPPORT;
        if (dtype == TILEXR_DATA_TYPE_BFP16) ek = 0;
        else if (dtype == TILEXR_DATA_TYPE_FP16) ek = 1;
        else if (dtype == TILEXR_DATA_TYPE_FP32) ek = 2;
        else return TILEXR_ERROR_NOT_SUPPORT;
    }
    if (bytes == 0 || bytes % 16 != 0 || reinterpret_cast<uintptr_t>(in) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0) return TILEXR_ERROR_NOT_SUPPORT;
    const uint64_t staged = (kind == COLL_KIND_REDUCE_SCATTER || kind == COLL_KIND_ALL_GATHER) ? bytes * R : bytes;
    if (staged > hostArgs->dataHalfBytes) return TILEXR_ERROR_NOT_SUPPORT;
    // Below these sizes the peer-to-peer kernels (one launch, direct pushes) are as fast or faster.
    const uint64_t floorBytes = static_cast<uint64_t>(EnvLongNvls("TILEXR_NVLS_MIN_BYTES", kind == COLL_KIND_ALL_REDUCE ? (32 << 10) : (1 << 20)));
    if (staged < floorBytes) return TILEXR_ERROR_NOT_SUPPORT;
    // With two or three ranks the switch saves little traffic and the staging copies cost more than they save on
    // large messages; the latency advantage of the single meeting remains below a few megabytes.
    if (R < 4 && staged > static_cast<uint64_t>(EnvLongNvls("TILEXR_NVLS_SMALL_WORLD_MAX_BYTES", 8 << 20))) return TILEXR_ERROR_NOT_SUPPORT;
    NvlsWindowArgs a;
    std::memset(&a, 0, sizeof(a));
    a.in = static_cast<const uint8_t *>(in);
    a.out = static_cast<uint8_t *>(out);
    a.comm = reinterpret_cast<CommArgs *>(devArgs);
    a.vecs = bytes / 16;
    a.kind = ek;
    a.root = root;
    switch (kind) {
        case COLL_KIND_ALL_REDUCE:
            a.mode = bytes <= static_cast<uint64_t>(EnvLongNvls("TILEXR_NVLS_ONE_SHOT_BYTES", 512 << 10)) ? NVLS_WIN_ALL_REDUCE_ONE_SHOT : NVLS_WIN_ALL_REDUCE_TWO_SHOT;
            a.opType = TILEXR_OP_ALL_REDUCE;
            break;
        case COLL_KIND_REDUCE_SCATTER: a.mode = NVLS_WIN_REDUCE_SCATTER; a.opType = TILEXR_OP_REDUCE_SCATTER; break;
        case COLL_KIND_ALL_GATHER: a.mode = NVLS_WIN_ALL_GATHER; a.opType = TILEXR_OP_ALL_GATHER; break;
        case COLL_KIND_BROADCAST: a.mode = NVLS_WIN_BROADCAST; a.opType = TILEXR_OP_BROADCAST; break;
        default: return TILEXR_ERROR_NOT_SUPPORT;
    }
    int64_t magic = 0;
    int ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    unsigned maxGrid = 0;
    ret = MaxCooperativeGrid(comm, TileXRNvlsWindowKernelEntry, NVLS_THREADS, 0, 1, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    // one chunk per block: enough blocks to keep the switch busy, few enough that a chunk is worth a meeting
    const uint64_t perBlockFloor = 64u << 10;
    long want = static_cast<long>(std::max<uint64_t>(1, std::min<uint64_t>(128, bytes / perBlockFloor)));
    want = EnvLongNvls("TILEXR_NVLS_BLOCKS", want);
    const unsigned grid = std::max(1u, std::min<unsigned>(static_cast<unsigned>(std::min<long>(want, TILEXR_FLAGS_PER_PAIR)), maxGrid));
    LaunchConfig cfg{grid, NVLS_THREADS, 0, true};
    return LaunchKernel(comm, TileXRNvlsWindowKernelEntry, &a, cfg, stream);
}

} // namespace TileXR

using namespace TileXR;

extern "C" {

int TileXRNvlsAllReduce(void *mcAddr, uint64_t bytes, TileXRDataType dtype, TileXRCommPtr comm, TileXRStream stream)
{
    return Launch(NVLS_ALL_REDUCE, mcAddr, nullptr, nullptr, bytes, dtype, 0, comm, stream);
}

int TileXRNvlsReduceScatter(void *mcAddr, void *out, uint64_t bytes, TileXRDataType dtype, TileXRCommPtr comm, TileXRStream stream)
{
    return Launch(NVLS_REDUCE_SCATTER, mcAddr, nullptr, out, bytes, dtype, 0, comm, stream);
}

int TileXRNvlsAllGather(const void *shard, void *mcAddr, uint64_t shardBytes, TileXRCommPtr comm, TileXRStream stream)
{
    return Launch(NVLS_ALL_GATHER, mcAddr, shard, nullptr, shardBytes, TILEXR_DATA_TYPE_FP32, 0, comm, stream);
}

int TileXRNvlsBroadcast(const void *in, void *mcAddr, uint64_t bytes, int root, TileXRCommPtr comm, TileXRStream stream)
{
    return Launch(NVLS_BROADCAST, mcAddr, in, nullptr, bytes, TILEXR_DATA_TYPE_FP32, root, comm, stream);
}

int TileXRNvlsAllReduceRmsNorm(void *mcX, void *mcResidual, const void *residualLocal, const void *gamma, float eps, int64_t rows,
                               int64_t h, TileXRDataType dtype, void *mcY, TileXRCommPtr comm, TileXRStream stream)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (hostArgs->extraFlag & (TILEXR_FLAG_HOST_MEMORY | TILEXR_FLAG_EMULATED)) return TILEXR_ERROR_NOT_SUPPORT;
    const auto misaligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 != 0; };
    if (mcX == nullptr || mcY == nullptr || gamma == nullptr || rows <= 0 || rows > 0x7fffffff || h <= 0 || h % 8 != 0 ||
        h > static_cast<int64_t>(NVLS_THREADS) * NVLS_NORM_MAX_VECS * 8 || (dtype != TILEXR_DATA_TYPE_FP16 && dtype != TILEXR_DATA_TYPE_BFP16) ||
        ((mcResidual == nullptr) != (residualLocal == nullptr)) || misaligned(mcX) || misaligned(mcY) || misaligned(mcResidual) ||
        misaligned(residualLocal) || misaligned(gamma)) {
        TILEXR_LOG(ERROR) << "nvls all-reduce+rmsnorm: bad arguments (rows " << rows << ", h " << h << ", dtype " << dtype << ")";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    NvlsNormArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mcX = static_cast<uint8_t *>(mcX);
    a.mcY = static_cast<uint8_t *>(mcY);
    a.mcRes = static_cast<uint8_t *>(mcResidual);
    a.resLocal = static_cast<const uint8_t *>(residualLocal);
    a.gamma = static_cast<const uint8_t *>(gamma);
    a.comm = reinterpret_cast<CommArgs *>(devArgs);
    a.eps = eps;
    a.rows = static_cast<int32_t>(rows);
    a.h = static_cast<int32_t>(h);
    a.rowBytes = static_cast<uint32_t>(h * 2);
    a.isBf16 = dtype == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    unsigned maxGrid = 0;
    ret = MaxCooperativeGrid(comm, TileXRNvlsNormKernelEntry, NVLS_THREADS, 0, 1, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    const int64_t mine = (rows + hostArgs->rankSize - 1) / hostArgs->rankSize;
    const long want = EnvLongNvls("TILEXR_NVLS_NORM_BLOCKS", 128);
    const unsigned grid = std::max(1u, std::min<unsigned>(static_cast<unsigned>(std::min<int64_t>(std::min<long>(want, TILEXR_FLAGS_PER_PAIR), mine)), maxGrid));
    LaunchConfig cfg{grid, NVLS_THREADS, 0, true};
    return LaunchKernel(comm, TileXRNvlsNormKernelEntry, &a, cfg, stream);
}

} // extern "C"
