// Host side of the stage profiler: owns one device trace buffer per profiled launch and turns
// them into reports.  The CUDA calls go through a hook table so that unit tests can run the
// session logic without a GPU (reference: SetPerfTraceRuntimeHooksForTest,
// src/collectives/host/perf_trace_session.h:41).
#ifndef TILEXR_PERF_TRACE_SESSION_H
#define TILEXR_PERF_TRACE_SESSION_H

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "tilexr_collectives_perf.h"
#include "tilexr_perf_trace.h"

namespace TileXR {

struct PerfLaunchInfo {
    uint32_t opType;
    uint32_t dataType;
    uint32_t rank;
    uint32_t rankSize;
    uint32_t blocks;
    uint64_t messageBytes;
};

struct PerfTraceRuntimeHooks {
    int (*alloc)(void **ptr, size_t bytes);
    int (*release)(void *ptr);
    int (*uploadAsync)(void *dst, const void *src, size_t bytes, void *stream);
    int (*clearAsync)(void *dst, size_t bytes, void *stream);
    int (*download)(void *dst, const void *src, size_t bytes);   // synchronises first
};
void SetPerfTraceRuntimeHooksForTest(const PerfTraceRuntimeHooks *hooks);   // null restores CUDA

// Called by the launcher: a device trace buffer for this launch, or null when no session is
// active, profiling is disabled by TILEXR_COLLECTIVES_DISABLE_KERNEL_PROFILING, or the launch
// is not sampled.
void *PerfTracePrepareLaunch(const PerfLaunchInfo &info, void *stream);

struct PerfLaunchRecord {
    uint64_t launchId;
    PerfLaunchInfo info;
    TileXRPerfTraceHeader header;
    std::vector<TileXRPerfCoreStageStats> stats;   // [blocks][stageCount]
};

struct PerfStageSummary {
    uint32_t stageId;
    std::string name;
    uint64_t count;
    double sumUs;
    double maxUs;
    uint32_t maxCore;
    double spanUs;        // lastEnd - firstStart over all blocks
    uint64_t bytes;
};

std::vector<PerfStageSummary> SummarizeLaunch(const PerfLaunchRecord &rec);
std::string AnalyzeLaunch(const PerfLaunchRecord &rec, const std::vector<PerfStageSummary> &summary);
int WriteLaunchReport(const std::string &dir, const PerfLaunchRecord &rec, bool emitAiPrompt, const std::string &aiCommand,
                      const std::string &incompleteReason);

} // namespace TileXR

#endif
