// Kernel-side half of the stage profiler.  A kernel gets `perfTrace` (null when no session is
// active) and brackets its stages with PerfStageBegin/End; thread 0 of each block owns the
// block's records, so there is no contention.  With a null buffer every call is a no-op
// (reference: perf_trace_kernel.h:35-139 and its disabled stubs :141-205).
#ifndef TILEXR_PERF_TRACE_CUH
#define TILEXR_PERF_TRACE_CUH

#include "tilexr_platform.cuh"
#include "../tilexr_perf_trace.h"

namespace tilexr {

struct PerfScope {
    TileXR::TileXRPerfCoreStageStats *stats;   // this block's record array, or null
    uint64_t begin[TILEXR_PERF_STAGE_COUNT];
};

TXR_D PerfScope PerfInit(void *perfTrace, uint32_t rank, uint32_t block)
{
    PerfScope p;
    p.stats = nullptr;
    if (perfTrace != nullptr) {
        const TileXR::TileXRPerfTraceHeader *h = reinterpret_cast<const TileXR::TileXRPerfTraceHeader *>(perfTrace);
        if (h->magic == TILEXR_PERF_TRACE_MAGIC && block < h->maxCoreCount) {
            p.stats = reinterpret_cast<TileXR::TileXRPerfCoreStageStats *>(reinterpret_cast<uint8_t *>(perfTrace) +
                                                                          h->statsOffset) +
                      static_cast<size_t>(block) * TILEXR_PERF_STAGE_COUNT;
            for (uint32_t s = 0; s < TILEXR_PERF_STAGE_COUNT; ++s) {
                p.stats[s].rank = rank;
                p.stats[s].core = block;
                p.stats[s].stageId = s;
            }
        }
    }
    return p;
}

TXR_D void PerfStageBegin(PerfScope &p, uint32_t stage)
{
    if (p.stats != nullptr) p.begin[stage] = now_ns();
}

TXR_D void PerfStageEnd(PerfScope &p, uint32_t stage, uint64_t bytes = 0)
{
    if (p.stats == nullptr) return;
    const uint64_t end = now_ns();
    const uint64_t d = end - p.begin[stage];
    TileXR::TileXRPerfCoreStageStats &s = p.stats[stage];
    if (s.count == 0) {
        s.firstStartCycle = p.begin[stage];
        s.minCycles = d;
        s.maxCycles = d;
    } else {
        if (d < s.minCycles) s.minCycles = d;
        if (d > s.maxCycles) s.maxCycles = d;
    }
    s.count += 1;
    s.sumCycles += d;
    s.lastEndCycle = end;
    s.aux0 += bytes;
}

} // namespace tilexr

#endif // TILEXR_PERF_TRACE_CUH
