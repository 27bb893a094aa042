#include <cstring>

#include "device/tilexr_data_as_flag.cuh"
#include "device/tilexr_local_copy.cuh"
#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "device/tilexr_udma.cuh"
#include "tilexr_launch.h"
#include "tilexr_log.h"
#include "tilexr_probes.h"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr unsigned PROBE_THREADS = 512;

struct ProbeArgs {
    CommArgs *comm;
    int64_t magic;
    uint8_t *local;
    const uint8_t *localSrc;
    int32_t *result;
    uint64_t offset;
    uint64_t bytes;
    uint64_t signalValue;
    uint32_t handle;
    uint32_t signalIndex;
    int32_t mode;     // 0 put+signal, 1 get, 2 local copy, 3 signal wait, 4 range check, 5 data-as-flag round trip, 6 reference-named verbs
};

__device__ void ProbeBody(const ProbeArgs &a)
{
    extern __shared__ __align__(128) uint8_t smemRaw[];
    Waiter w;
    // the data-as-flag probe writes into its peer's low-latency plane, whose halves alternate with the launch epoch: the
    // reuse guard (the peer has finished the launch before last) applies to it as to every operator
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_BANDWIDTH, static_cast<int64_t>(a.bytes), a.mode == 5);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int R = comm->rankSize;
    const int peer = (rank + 1) % R;
    const uint64_t per = ((a.bytes + gridDim.x - 1) / gridDim.x + 15) & ~15ull;
    const uint64_t begin = min(a.bytes, per * blockIdx.x);
    const uint64_t n = min(a.bytes - begin, per);
    if (a.mode == 0) {
        const int st = PutNbi(comm->registryPtr, a.handle, peer, a.offset + begin, a.localSrc + begin, n, threadIdx.x, blockDim.x);
        fence_acq_rel_sys();
        __syncthreads();
        if (threadIdx.x == 0) {
            if (st != RMA_OK) RaiseFailure(w, TILEXR_DEV_BAD_RANGE, peer, a.handle, a.offset + begin, n);
            else SignalAdd(comm, peer, a.signalIndex, 1);
            // every block signalled once: the word reaches blocks * calls
            if (WaitSignalGE(w, a.signalIndex, a.signalValue) != RMA_OK) ok = false;
        }
        ok = BlockBroadcastOk(ok && w.ok());
    } else if (a.mode == 1) {
        const int st = GetNbi(comm->registryPtr, a.handle, peer, a.offset + begin, a.local + begin, n, threadIdx.x, blockDim.x);
        if (st != RMA_OK && threadIdx.x == 0) RaiseFailure(w, TILEXR_DEV_BAD_RANGE, peer, a.handle, a.offset + begin, n);
        Quiet();
    } else if (a.mode == 2) {
        LocalCopyLane *lane = reinterpret_cast<LocalCopyLane *>(smemRaw);
        if (threadIdx.x == 0) {
            LocalCopyLaneInit(lane);
            const LocalCopyEvent ev = LocalCopyNbi(comm, lane, a.local + begin, a.localSrc + begin, n);
            if (ev.status == RMA_MISALIGNED) {
                lane->ready = 2;       // fall back to the cooperative copy below
            } else if (!LocalCopyWait(ev)) {
                RaiseFailure(w, TILEXR_DEV_MBARRIER_TIMEOUT, rank, blockIdx.x, 0, 0);
            }
        }
        __syncthreads();
        if (lane->ready == 2) CopyLanes(a.local + begin, a.localSrc + begin, n, threadIdx.x, blockDim.x);
    } else if (a.mode == 3) {
        if (blockIdx.x == 0 && threadIdx.x == 0) WaitSignalGE(w, a.signalIndex, a.signalValue);
        ok = BlockBroadcastOk(w.ok());
    } else if (a.mode == 5) {
        // Every block sends its share of the payload to the next rank as 16-byte units that carry the launch epoch in
        // their last word (payload and flag in ONE transaction), and receives the previous rank's share the same way.
        // Block `signalIndex` sends nothing: its counterpart's wait runs out of budget and the kernel reports it.
        const int from = (rank - 1 + R) % R;
        const uint64_t words = a.bytes / 4;
        const uint64_t wordsPerBlock = ((words + gridDim.x - 1) / gridDim.x + 2) / 3 * 3;      // whole units per block
        const uint64_t w0 = min(words, wordsPerBlock * blockIdx.x);
        const uint64_t nw = min(words - w0, wordsPerBlock);
        const uint64_t unit0 = w0 / 3;
        if (ok && blockIdx.x != a.signalIndex) {
            Ll16Send(LlHalf(comm, peer, w.epoch) + unit0 * LL16_UNIT_BYTES, a.localSrc + w0 * 4, nw * 4, w.epoch, threadIdx.x, blockDim.x);
        }
        const bool got = ok && Ll16Recv(w, a.local + w0 * 4, LlHalf(comm, rank, w.epoch) + unit0 * LL16_UNIT_BYTES, nw * 4, from, threadIdx.x, blockDim.x);
        ok = BlockBroadcastOk(got);
    } else if (a.mode == 6) {
        // The reference's verb names (device/tilexr_udma.cuh).  Warp g of the launch puts its share of the payload into the
        // next rank's region 0 and raises signal word g of that region behind it (put with signal), waits for its own
        // word g, which the previous rank's warp g raises, and reads its share back from the next rank (get).  The signal
        // words follow the payload at a.offset.  A put that leaves the region must be refused.
        const uint64_t warps = blockDim.x / 32;
        const uint64_t g = blockIdx.x * warps + threadIdx.x / 32;
        const uint64_t G = gridDim.x * warps;
        const uint64_t share = ((a.bytes + G - 1) / G + 15) & ~15ull;
        const uint64_t b0 = min(a.bytes, share * g);
        const uint32_t nb = static_cast<uint32_t>(min(a.bytes - b0, share));
        const int from = (rank - 1 + R) % R;
        bool good = ok;
        if (good) {
            const uint32_t lanes = UDMAQpCount(comm);      // 0 on a communicator without registered memory: the verbs then refuse
            const uint32_t qp = lanes != 0 ? static_cast<uint32_t>(g % lanes) : 0u;
            good = UDMAPutSignalNbiOnQp<uint8_t>(comm, peer, qp, a.localSrc + b0, b0, nb, a.offset + g * 8, MakeFlag(w.epoch, 1)) ==
                   TILEXR_UDMA_STATUS_SUCCESS;
            good = good && UDMAPutNbiOnQp<uint8_t>(comm, peer, 0, a.localSrc, a.offset + G * 8, 16) == TILEXR_UDMA_STATUS_INVALID;
            if (!good && (threadIdx.x & 31u) == 0) RaiseFailure(w, TILEXR_DEV_BAD_RANGE, peer, static_cast<int64_t>(g), a.offset, nb);
        }
        if (good && (threadIdx.x & 31u) == 0) {
            const uint64_t *word = reinterpret_cast<const uint64_t *>(UDMARegisteredRemoteAddr(comm, rank, a.offset + g * 8, 8));
            good = word != nullptr && WaitFlagGE(w, word, 1, from, static_cast<int64_t>(g));
        }
        good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;
        if (good) {
            good = UDMAGetNbiOnQp<uint8_t>(comm, peer, 0, a.local + b0, b0, nb) == TILEXR_UDMA_STATUS_SUCCESS;
            UDMAQuiet(comm, peer);
        }
        ok = BlockBroadcastOk(good);
    } else if (a.mode == 4) {
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            int st = RMA_OK;
            RmaTranslate(comm->registryPtr, a.handle, peer, a.offset, a.bytes, &st);
            *a.result = st;
        }
    }
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRProbeKernel, ProbeArgs, ProbeBody, PROBE_THREADS)

int Launch(TileXRCommPtr comm, ProbeArgs &a, unsigned blocks, size_t smem, TileXRStream stream)
{
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_ERROR_NOT_SUPPORT;
    a.comm = reinterpret_cast<CommArgs *>(devArgs);
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    const int ranksPerDevice = (hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? hostArgs->rankSize : 1;
    unsigned maxGrid = 0;
    ret = MaxCooperativeGrid(comm, TileXRProbeKernelEntry, PROBE_THREADS, smem, ranksPerDevice, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    const unsigned grid = blocks == 0 ? 1 : (blocks > maxGrid ? maxGrid : blocks);
    LaunchConfig cfg{grid, PROBE_THREADS, smem, true};
    return LaunchKernel(comm, TileXRProbeKernelEntry, &a, cfg, stream);
}

} // namespace
} // namespace TileXR

using namespace TileXR;

extern "C" {

int TileXRPutSignalProbe(TileXRCommPtr comm, TileXRUDMAMemHandle handle, uint64_t dstOffset, const void *localSrc, uint64_t bytes,
                         uint32_t signalIndex, uint64_t expectedSignal, uint32_t blocks, TileXRStream stream)
{
    if (localSrc == nullptr || bytes == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    ProbeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mode = 0;
    a.handle = handle;
    a.offset = dstOffset;
    a.localSrc = static_cast<const uint8_t *>(localSrc);
    a.bytes = bytes;
    a.signalIndex = signalIndex;
    a.signalValue = expectedSignal;
    return Launch(comm, a, blocks, 0, stream);
}

int TileXRGetProbe(TileXRCommPtr comm, TileXRUDMAMemHandle handle, uint64_t srcOffset, void *localDst, uint64_t bytes,
                   uint32_t blocks, TileXRStream stream)
{
    if (localDst == nullptr || bytes == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    ProbeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mode = 1;
    a.handle = handle;
    a.offset = srcOffset;
    a.local = static_cast<uint8_t *>(localDst);
    a.bytes = bytes;
    return Launch(comm, a, blocks, 0, stream);
}

int TileXRLocalCopyProbe(TileXRCommPtr comm, void *dst, const void *src, uint64_t bytes, uint32_t blocks, TileXRStream stream)
{
    if (dst == nullptr || src == nullptr || bytes == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    ProbeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mode = 2;
    a.local = static_cast<uint8_t *>(dst);
    a.localSrc = static_cast<const uint8_t *>(src);
    a.bytes = bytes;
    return Launch(comm, a, blocks, sizeof(LocalCopyLane) + 128, stream);
}

int TileXRDataAsFlagProbe(TileXRCommPtr comm, void *dst, const void *src, uint64_t bytes, uint32_t withheldBlock, uint32_t blocks,
                          TileXRStream stream)
{
    if (dst == nullptr || src == nullptr || bytes == 0 || bytes % 4 != 0 || blocks == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    // every block's share is rounded up to whole units
    if (tilexr::Ll16PackedBytes(bytes) + static_cast<uint64_t>(blocks) * tilexr::LL16_UNIT_BYTES > TILEXR_WIN_LL_HALF_BYTES) {
        TILEXR_LOG(ERROR) << "data-as-flag probe: " << bytes << " payload bytes do not fit one half of the low-latency plane";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    ProbeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mode = 5;
    a.local = static_cast<uint8_t *>(dst);
    a.localSrc = static_cast<const uint8_t *>(src);
    a.bytes = bytes;
    a.signalIndex = withheldBlock;
    return Launch(comm, a, blocks, 0, stream);
}

int TileXRNamedVerbsProbe(TileXRCommPtr comm, void *dst, const void *src, uint64_t bytes, uint64_t signalOffset, uint32_t blocks,
                          TileXRStream stream)
{
    if (dst == nullptr || src == nullptr || bytes == 0 || bytes % 16 != 0 || signalOffset % 8 != 0 || signalOffset < bytes || blocks == 0) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    ProbeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mode = 6;
    a.local = static_cast<uint8_t *>(dst);
    a.localSrc = static_cast<const uint8_t *>(src);
    a.bytes = bytes;
    a.offset = signalOffset;
    return Launch(comm, a, blocks, 0, stream);
}

int TileXRSignalWaitProbe(TileXRCommPtr comm, uint32_t signalIndex, uint64_t value, TileXRStream stream)
{
    ProbeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mode = 3;
    a.signalIndex = signalIndex;
    a.signalValue = value;
    return Launch(comm, a, 1, 0, stream);
}

int TileXRRangeCheckProbe(TileXRCommPtr comm, TileXRUDMAMemHandle handle, uint64_t offset, uint64_t bytes, int32_t *deviceResult,
                          TileXRStream stream)
{
    if (deviceResult == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    ProbeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.mode = 4;
    a.handle = handle;
    a.offset = offset;
    a.bytes = bytes;
    a.result = deviceResult;
    return Launch(comm, a, 1, 0, stream);
}

} // extern "C"
