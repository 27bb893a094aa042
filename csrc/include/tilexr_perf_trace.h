// Device stage profiler ABI shared by kernels, the host session and the report tools.
// A trace buffer is a 128-byte header followed by one statistics record per
// (rank, block, stage).  Same record shape and the same seven stage ids as the reference
// (src/include/tilexr_perf_trace.h:15-121) so its report tooling concepts carry over; the
// time base is the GPU's nanosecond `globaltimer`, i.e. 1000 ticks per microsecond.
#ifndef TILEXR_PERF_TRACE_H
#define TILEXR_PERF_TRACE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
namespace TileXR {
#endif

#define TILEXR_PERF_TRACE_MAGIC 0x54585054u   /* "TXPT" */
#define TILEXR_PERF_TRACE_VERSION 1u
#define TILEXR_PERF_MAX_STAGE_NAME 32u
#define TILEXR_PERF_STAGE_COUNT 7u
#define TILEXR_PERF_TRACE_STATS_OFFSET 128u
#define TILEXR_PERF_TICKS_PER_US 1000u

enum TileXRPerfStageCategory { TILEXR_PERF_CAT_TOTAL = 0, TILEXR_PERF_CAT_COPY = 1, TILEXR_PERF_CAT_WAIT = 2,
                               TILEXR_PERF_CAT_SYNC = 3, TILEXR_PERF_CAT_BARRIER = 4 };
enum TileXRPerfBarrierPolicy { TILEXR_PERF_NO_BARRIER = 0, TILEXR_PERF_END_BARRIER_ONLY = 1, TILEXR_PERF_BARRIERED = 2 };

enum TileXRPerfStageId {
    TILEXR_PERF_KERNEL_TOTAL = 0,
    TILEXR_PERF_CHUNK_TOTAL = 1,
    TILEXR_PERF_POST_SYNC = 2,
    TILEXR_PERF_LOCAL_INPUT_TO_IPC = 3,
    TILEXR_PERF_FLAG_POLL_WAIT = 4,
    TILEXR_PERF_PEER_IPC_TO_OUTPUT = 5,
    TILEXR_PERF_CHUNK_BARRIER = 6,
};

struct TileXRPerfTraceHeader {
    uint32_t magic;
    uint32_t version;
    uint32_t headerSize;
    uint32_t stageDescSize;
    uint32_t coreStageStatsSize;
    uint32_t flags;
    uint32_t rank;
    uint32_t rankSize;
    uint32_t blockDim;        // blocks launched
    uint32_t maxCoreCount;    // blocks the buffer has room for
    uint32_t stageCount;
    uint32_t cycleToUsDivisor;
    uint64_t launchId;
    uint64_t messageBytes;
    uint32_t opType;
    uint32_t dataType;
    uint64_t statsOffset;
    uint64_t statsBytes;
};

struct TileXRPerfStageDesc {
    uint32_t stageId;
    uint32_t category;
    uint32_t barrierPolicy;
    uint32_t displayOrder;
    char name[TILEXR_PERF_MAX_STAGE_NAME];
};

struct TileXRPerfCoreStageStats {
    uint32_t rank;
    uint32_t core;
    uint32_t stageId;
    uint32_t reserved;
    uint64_t count;
    uint64_t sumCycles;
    uint64_t minCycles;
    uint64_t maxCycles;
    uint64_t firstStartCycle;
    uint64_t lastEndCycle;
    uint64_t aux0;   // bytes moved in this stage
    uint64_t aux1;
    uint64_t aux2;
    uint64_t aux3;
};

static inline size_t TileXRPerfStatsIndex(uint32_t core, uint32_t stage, uint32_t stageCount)
{
    return (size_t)core * stageCount + stage;
}

static inline size_t TileXRPerfTraceBytes(uint32_t maxCoreCount)
{
    return TILEXR_PERF_TRACE_STATS_OFFSET +
           (size_t)maxCoreCount * TILEXR_PERF_STAGE_COUNT * sizeof(struct TileXRPerfCoreStageStats);
}

static inline double TileXRPerfTicksToUs(uint64_t ticks, uint32_t divisor)
{
    return divisor == 0 ? 0.0 : (double)ticks / (double)divisor;
}

static const struct TileXRPerfStageDesc TILEXR_PERF_STAGE_TABLE[TILEXR_PERF_STAGE_COUNT] = {
    {TILEXR_PERF_KERNEL_TOTAL, TILEXR_PERF_CAT_TOTAL, TILEXR_PERF_NO_BARRIER, 0, "kernel_total"},
    {TILEXR_PERF_CHUNK_TOTAL, TILEXR_PERF_CAT_TOTAL, TILEXR_PERF_NO_BARRIER, 1, "chunk_total"},
    {TILEXR_PERF_POST_SYNC, TILEXR_PERF_CAT_SYNC, TILEXR_PERF_END_BARRIER_ONLY, 2, "post_sync"},
    {TILEXR_PERF_LOCAL_INPUT_TO_IPC, TILEXR_PERF_CAT_COPY, TILEXR_PERF_NO_BARRIER, 3, "local_input_to_ipc"},
    {TILEXR_PERF_FLAG_POLL_WAIT, TILEXR_PERF_CAT_WAIT, TILEXR_PERF_NO_BARRIER, 4, "flag_poll_wait"},
    {TILEXR_PERF_PEER_IPC_TO_OUTPUT, TILEXR_PERF_CAT_COPY, TILEXR_PERF_NO_BARRIER, 5, "peer_ipc_to_output"},
    {TILEXR_PERF_CHUNK_BARRIER, TILEXR_PERF_CAT_BARRIER, TILEXR_PERF_BARRIERED, 6, "chunk_barrier"},
};

#ifdef __cplusplus
} // namespace TileXR
#endif

#endif // TILEXR_PERF_TRACE_H
