// Device-initiated local copy (global -> global on the same GPU) that does not occupy the
// calling block's threads: one thread drives a TMA pipeline global -> shared -> global and
// the rest of the block keeps computing.  Counterpart of the reference's SDMA device API
// (src/include/tilexr_sdma.h:43-100: SDMACopyNbi returns an event handle, SDMAWait joins it,
// and both degrade to a synchronous path when the engine is not available).
//
// The host-initiated form of the same transport is a copy-engine `cudaMemcpyAsync` on a side
// stream (TileXRLocalCopyAsync in tilexr_api.h).
#ifndef TILEXR_LOCAL_COPY_CUH
#define TILEXR_LOCAL_COPY_CUH

#include "tilexr_rma.cuh"

namespace tilexr {

constexpr uint32_t LOCAL_COPY_STAGE_BYTES = 32 * 1024;
constexpr uint32_t LOCAL_COPY_STAGES = 2;

#if defined(__CUDACC__)

// Shared-memory footprint of one copy lane; place it in dynamic shared memory, 128-byte aligned.
struct alignas(128) LocalCopyLane {
    uint8_t stage[LOCAL_COPY_STAGES][LOCAL_COPY_STAGE_BYTES];
    uint64_t full[LOCAL_COPY_STAGES];
    uint32_t phase[LOCAL_COPY_STAGES];
    uint32_t ready;
};

struct LocalCopyEvent {
    int status;          // RMA_OK, RMA_MISALIGNED (nothing copied) or RMA_TIMEOUT
    uint32_t groups;     // bulk groups committed by the issuing thread
};

// One thread of the block calls this once before the first copy on `lane`.
__device__ __forceinline__ void LocalCopyLaneInit(LocalCopyLane *lane)
{
    for (uint32_t s = 0; s < LOCAL_COPY_STAGES; ++s) {
        MbarInit(&lane->full[s], 1);
        lane->phase[s] = 0;
    }
    lane->ready = 1;
    MbarInitFence();
}

// Issued by ONE thread.  Addresses 16-byte aligned, bytes a multiple of 16; otherwise nothing
// is copied and the event says RMA_MISALIGNED so the caller can use CopyLanes instead.
// `channelGroup` is accepted for parity with the reference API; lanes are chosen by the caller.
__device__ __forceinline__ LocalCopyEvent LocalCopyNbi(const CommArgs *args, LocalCopyLane *lane, void *dst,
                                                       const void *src, uint64_t bytes, uint32_t channelGroup = 0)
{
    (void)channelGroup;
    LocalCopyEvent ev{RMA_OK, 0};
    if ((args->extraFlag & TileXR::TILEXR_FLAG_LOCAL_COPY) == 0 ||
        ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | bytes) & 15u) != 0) {
        ev.status = RMA_MISALIGNED;
        return ev;
    }
    // Loads run LOCAL_COPY_STAGES - 1 chunks ahead of the stores: the load of chunk c + A is issued before the wait for
    // chunk c, so several loads are in flight at once and they overlap the stores (waiting for every load right after
    // issuing it left one transfer in flight per direction).
    const uint64_t chunks = (bytes + LOCAL_COPY_STAGE_BYTES - 1) / LOCAL_COPY_STAGE_BYTES;
    constexpr uint64_t AHEAD = LOCAL_COPY_STAGES - 1;
    auto issueLoad = [&](uint64_t c) {
        const uint32_t st = static_cast<uint32_t>(c % LOCAL_COPY_STAGES);
        const uint64_t off = c * LOCAL_COPY_STAGE_BYTES;
        const uint32_t n = static_cast<uint32_t>(bytes - off < LOCAL_COPY_STAGE_BYTES ? bytes - off : LOCAL_COPY_STAGE_BYTES);
        MbarExpectTx(&lane->full[st], n);
        BulkLoadToSmem(lane->stage[st], reinterpret_cast<const uint8_t *>(src) + off, n, &lane->full[st]);
    };
    BulkWaitRead<0>();                         // the stores of an earlier copy on this lane have finished reading the stages
    for (uint64_t c = 0; c < chunks && c < AHEAD; ++c) issueLoad(c);
    for (uint64_t c = 0; c < chunks; ++c) {
        if (c + AHEAD < chunks) {
            // its stage was last read by the store of chunk c - 1, the most recent bulk group
            if (c > 0) BulkWaitRead<0>();
            issueLoad(c + AHEAD);
        }
        const uint32_t st = static_cast<uint32_t>(c % LOCAL_COPY_STAGES);
        const uint64_t off = c * LOCAL_COPY_STAGE_BYTES;
        const uint32_t n = static_cast<uint32_t>(bytes - off < LOCAL_COPY_STAGE_BYTES ? bytes - off : LOCAL_COPY_STAGE_BYTES);
        if (!MbarWait(&lane->full[st], lane->phase[st], args->waitTimeoutNs)) {
            // the loads issued ahead are given the same (bounded) time to land before the caller may leave the kernel
            for (uint64_t k = c + 1; k < chunks && k <= c + AHEAD; ++k) {
                const uint32_t sk = static_cast<uint32_t>(k % LOCAL_COPY_STAGES);
                if (MbarWait(&lane->full[sk], lane->phase[sk], args->waitTimeoutNs)) lane->phase[sk] ^= 1u;
            }
            ev.status = RMA_TIMEOUT;
            break;
        }
        lane->phase[st] ^= 1u;
        BulkStoreFromSmem(reinterpret_cast<uint8_t *>(dst) + off, lane->stage[st], n);
        BulkCommit();
        ev.groups++;
    }
    return ev;
}

// Joins the copy: all bytes are written and visible to the calling thread afterwards.
__device__ __forceinline__ bool LocalCopyWait(const LocalCopyEvent &ev)
{
    BulkWait<0>();
    return ev.status == RMA_OK;
}

#endif // __CUDACC__

} // namespace tilexr

#endif // TILEXR_LOCAL_COPY_CUH
