// The reference's device verb names over this runtime's registered-memory verbs, for kernels that were written against
// its UDMA / SDMA device API (src/include/tilexr_udma.h:58-90, 748-1046; src/include/tilexr_sdma.h:30-100).
//
// The verbs keep their names, their order of arguments and their status values.  What differs, because two GPUs behind
// an NVSwitch have no work queue between them:
//   * there is no work-queue scratch argument: a put is the stores, a get the loads, of the calling WARP (all 32 lanes
//     call with the same arguments and the bytes are spread over them; on the host there is one caller);
//   * a queue-pair index names an ordering lane and is only validated (UDMAQpCount() lanes exist): operations of one warp
//     are ordered by that warp's fences, independent lanes are different warps;
//   * `byteOffset` addresses registered region 0 (the reference's single registered window); the `Region` forms of
//     tilexr_rma.cuh (PutNbi / GetNbi with a handle) reach the other regions;
//   * the signal of a put-with-signal is the 64-bit word at `signalByteOffset` of the target's region 0, stored with
//     release order after the payload, so that a reader who acquires it sees the payload;
//   * quiet is a system-scope fence: when it returns, every put and get of the calling thread has been performed.
// A bad rank, lane or range yields TILEXR_UDMA_STATUS_INVALID before a byte moves, as in the reference.
#ifndef TILEXR_UDMA_CUH
#define TILEXR_UDMA_CUH

#include "tilexr_local_copy.cuh"
#include "tilexr_rma.cuh"

namespace tilexr {

constexpr uint32_t TILEXR_UDMA_STATUS_SUCCESS = 0u;
constexpr uint32_t TILEXR_UDMA_STATUS_CQ_TIMEOUT = 0xFFu;
constexpr uint32_t TILEXR_UDMA_STATUS_SQ_FULL = 0xFFFFFFFEu;      // never returned: there is no queue to fill
constexpr uint32_t TILEXR_UDMA_STATUS_INVALID = 0xFFFFFFFFu;
constexpr uint32_t TILEXR_UDMA_DEVICE_MAX_QP_COUNT = 32u;
constexpr uint32_t TILEXR_UDMA_REGION = 0u;                       // the region that the offset forms address
constexpr uint32_t TILEXR_SDMA_AUTO_CHANNEL_GROUP = 0xFFFFFFFFu;

TXR_D bool UDMAEnabled(const CommArgs *args)
{
    return args != nullptr && (args->extraFlag & TileXR::TILEXR_FLAG_RMA) != 0 && args->registryPtr != nullptr;
}

TXR_D bool UDMARegistryEnabled(const CommArgs *args)
{
    return UDMAEnabled(args) && args->registryPtr->magic == TILEXR_REGISTRY_MAGIC && args->registryPtr->regionCount > 0;
}

// Ordering lanes a kernel may name.  Every warp is its own lane here, so the number only bounds the index.
TXR_D uint32_t UDMAQpCount(const CommArgs *args) { return UDMAEnabled(args) ? TILEXR_UDMA_DEVICE_MAX_QP_COUNT : 0u; }
TXR_D bool UDMAQpValid(const CommArgs *args, uint32_t qpIdx) { return qpIdx < UDMAQpCount(args); }

TXR_D bool UDMARankValid(const CommArgs *args, int peer)
{
    return args != nullptr && args->rankSize > 0 && args->rankSize <= TILEXR_MAX_RANK_SIZE && peer >= 0 && peer < args->rankSize &&
           peer != args->rank;
}

TXR_D bool UDMAQueueOperationValid(const CommArgs *args, int peer, uint32_t qpIdx)
{
    return UDMARegistryEnabled(args) && UDMARankValid(args, peer) && UDMAQpValid(args, qpIdx);
}

// Address of [byteOffset, byteOffset + byteCount) of region 0 in `peer`'s copy, or null when the range is not inside it.
TXR_D uint8_t *UDMARegisteredRemoteAddr(const CommArgs *args, int peer, uint64_t byteOffset, uint64_t byteCount)
{
    if (!UDMARegistryEnabled(args)) return nullptr;
    int st;
    return RmaTranslate(args->registryPtr, TILEXR_UDMA_REGION, peer, byteOffset, byteCount, &st);
}

TXR_D bool UDMARegisteredRangeValid(const CommArgs *args, int peer, uint64_t byteOffset, uint64_t byteCount)
{
    return UDMARegisteredRemoteAddr(args, peer, byteOffset, byteCount) != nullptr;
}

namespace detail {
TXR_D int UdmaLane()
{
#if defined(__CUDA_ARCH__)
    return static_cast<int>(threadIdx.x & 31u);
#else
    return 0;
#endif
}
TXR_D int UdmaLanes()
{
#if defined(__CUDA_ARCH__)
    return 32;
#else
    return 1;
#endif
}
TXR_D void UdmaJoin()
{
#if defined(__CUDA_ARCH__)
    __syncwarp();
#endif
}
} // namespace detail

template <typename T>
TXR_D uint32_t UDMAPutNbiOnQp(const CommArgs *args, int targetRank, uint32_t qpIdx, const T *localSrc, uint64_t byteOffset, uint32_t byteCount)
{
    if (!UDMAQueueOperationValid(args, targetRank, qpIdx) || (localSrc == nullptr && byteCount != 0u)) return TILEXR_UDMA_STATUS_INVALID;
    const int st = PutNbi(args->registryPtr, TILEXR_UDMA_REGION, targetRank, byteOffset, localSrc, byteCount, detail::UdmaLane(), detail::UdmaLanes());
    return st == RMA_OK ? TILEXR_UDMA_STATUS_SUCCESS : TILEXR_UDMA_STATUS_INVALID;
}

template <typename T>
TXR_D void UDMAPutNbi(const CommArgs *args, int targetRank, const T *localSrc, uint64_t byteOffset, uint32_t byteCount)
{
    (void)UDMAPutNbiOnQp<T>(args, targetRank, 0u, localSrc, byteOffset, byteCount);
}

template <typename T>
TXR_D void UDMAPutRegisteredNbi(const CommArgs *args, int targetRank, const T *localSrc, uint64_t byteOffset, uint32_t byteCount)
{
    UDMAPutNbi<T>(args, targetRank, localSrc, byteOffset, byteCount);
}

template <typename T>
TXR_D uint32_t UDMAGetNbiOnQp(const CommArgs *args, int sourceRank, uint32_t qpIdx, T *localDst, uint64_t byteOffset, uint32_t byteCount)
{
    if (!UDMAQueueOperationValid(args, sourceRank, qpIdx) || (localDst == nullptr && byteCount != 0u)) return TILEXR_UDMA_STATUS_INVALID;
    const int st = GetNbi(args->registryPtr, TILEXR_UDMA_REGION, sourceRank, byteOffset, localDst, byteCount, detail::UdmaLane(), detail::UdmaLanes());
    return st == RMA_OK ? TILEXR_UDMA_STATUS_SUCCESS : TILEXR_UDMA_STATUS_INVALID;
}

template <typename T>
TXR_D void UDMAGetNbi(const CommArgs *args, int sourceRank, T *localDst, uint64_t byteOffset, uint32_t byteCount)
{
    (void)UDMAGetNbiOnQp<T>(args, sourceRank, 0u, localDst, byteOffset, byteCount);
}

template <typename T>
TXR_D void UDMAGetRegisteredNbi(const CommArgs *args, int sourceRank, T *localDst, uint64_t byteOffset, uint32_t byteCount)
{
    UDMAGetNbi<T>(args, sourceRank, localDst, byteOffset, byteCount);
}

// The payload, then `signal` into the 64-bit word at signalByteOffset of the target's region (8-byte aligned).
template <typename T>
TXR_D uint32_t UDMAPutSignalNbiOnQp(const CommArgs *args, int targetRank, uint32_t qpIdx, const T *localSrc, uint64_t byteOffset,
                                    uint32_t byteCount, uint64_t signalByteOffset, uint64_t signal)
{
    if (!UDMAQueueOperationValid(args, targetRank, qpIdx) || (localSrc == nullptr && byteCount != 0u) || (signalByteOffset & 7u) != 0 ||
        !UDMARegisteredRangeValid(args, targetRank, byteOffset, byteCount)) {
        return TILEXR_UDMA_STATUS_INVALID;
    }
    uint8_t *word = UDMARegisteredRemoteAddr(args, targetRank, signalByteOffset, sizeof(uint64_t));
    if (word == nullptr) return TILEXR_UDMA_STATUS_INVALID;
    (void)PutNbi(args->registryPtr, TILEXR_UDMA_REGION, targetRank, byteOffset, localSrc, byteCount, detail::UdmaLane(), detail::UdmaLanes());
    fence_acq_rel_sys();
    detail::UdmaJoin();
    if (detail::UdmaLane() == 0) st_release_sys_u64(reinterpret_cast<uint64_t *>(word), signal);
    return TILEXR_UDMA_STATUS_SUCCESS;
}

template <typename T>
TXR_D void UDMAPutSignalNbi(const CommArgs *args, int targetRank, const T *localSrc, uint64_t byteOffset, uint32_t byteCount,
                            uint64_t signalByteOffset, uint64_t signal)
{
    (void)UDMAPutSignalNbiOnQp<T>(args, targetRank, 0u, localSrc, byteOffset, byteCount, signalByteOffset, signal);
}

template <typename T>
TXR_D uint32_t UDMAPutRegisteredSignalNbiOnQp(const CommArgs *args, int targetRank, uint32_t qpIdx, const T *localSrc, uint64_t byteOffset,
                                              uint32_t byteCount, uint64_t signalByteOffset, uint64_t signal)
{
    return UDMAPutSignalNbiOnQp<T>(args, targetRank, qpIdx, localSrc, byteOffset, byteCount, signalByteOffset, signal);
}

template <typename T>
TXR_D void UDMAPutRegisteredSignalNbi(const CommArgs *args, int targetRank, const T *localSrc, uint64_t byteOffset, uint32_t byteCount,
                                      uint64_t signalByteOffset, uint64_t signal)
{
    (void)UDMAPutRegisteredSignalNbiOnQp<T>(args, targetRank, 0u, localSrc, byteOffset, byteCount, signalByteOffset, signal);
}

// Completion of everything the calling thread has issued towards `targetRank` (towards anybody, in fact).
TXR_D uint32_t UDMAQuietStatusOnQp(const CommArgs *args, int targetRank, uint32_t qpIdx)
{
    if (!UDMAQueueOperationValid(args, targetRank, qpIdx)) return TILEXR_UDMA_STATUS_INVALID;
    (void)Quiet();
    return TILEXR_UDMA_STATUS_SUCCESS;
}
TXR_D uint32_t UDMAQuietStatusOnQpUntil(const CommArgs *args, int targetRank, uint32_t qpIdx, uint32_t completionTarget)
{
    (void)completionTarget;      // stores complete in order behind the fence: there is no partial completion to ask for
    return UDMAQuietStatusOnQp(args, targetRank, qpIdx);
}
TXR_D uint32_t UDMAQuietStatus(const CommArgs *args, int targetRank) { return UDMAQuietStatusOnQp(args, targetRank, 0u); }
TXR_D void UDMAQuiet(const CommArgs *args, int targetRank) { (void)UDMAQuietStatus(args, targetRank); }

// ---- SDMA names over the device-initiated local copy ------------------------------------------------------------------
TXR_D bool SDMAEnabled(const CommArgs *args) { return args != nullptr && (args->extraFlag & TileXR::TILEXR_FLAG_LOCAL_COPY) != 0; }

#if defined(__CUDACC__)
__device__ __forceinline__ uint32_t SDMAResolveChannelGroup(uint32_t channelGroupIdx)
{
    return channelGroupIdx == TILEXR_SDMA_AUTO_CHANNEL_GROUP ? blockIdx.x : channelGroupIdx;
}

// One thread of the block calls; `lane` is the block's copy lane in shared memory (LocalCopyLaneInit).  The handle is 0
// when nothing was started (engine off, misaligned, empty): the caller then copies with its threads, as with the reference.
__device__ __forceinline__ uint64_t SDMACopyNbi(const CommArgs *args, LocalCopyLane *lane, uint8_t *dst, const uint8_t *src, uint64_t bytes,
                                                uint32_t channelGroupIdx = TILEXR_SDMA_AUTO_CHANNEL_GROUP)
{
    if (!SDMAEnabled(args) || lane == nullptr || dst == nullptr || src == nullptr || bytes == 0) return 0;
    const LocalCopyEvent ev = LocalCopyNbi(args, lane, dst, src, bytes, SDMAResolveChannelGroup(channelGroupIdx));
    if (ev.status != RMA_OK) return 0;
    return (static_cast<uint64_t>(ev.groups) << 32) | 1u;
}

__device__ __forceinline__ bool SDMAWait(const CommArgs *args, uint64_t eventHandle, uint32_t channelGroupIdx = TILEXR_SDMA_AUTO_CHANNEL_GROUP)
{
    (void)channelGroupIdx;
    if (eventHandle == 0) return true;
    if (!SDMAEnabled(args)) return false;
    const LocalCopyEvent ev{RMA_OK, static_cast<uint32_t>(eventHandle >> 32)};
    return LocalCopyWait(ev);
}
#endif

} // namespace tilexr

#endif // TILEXR_UDMA_CUH
