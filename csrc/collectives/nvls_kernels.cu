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

#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
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

} // extern "C"
