// What the MoonEP stage kernels can write about themselves, and where.
//
// Two records, both filled by one thread per block and read on the host after the stream has drained:
//
//  * an EVENT TRACE of the dispatch stage (TileXRMoonEpDispatchArgsV1::trace): a header, one record per (iteration,
//    block) and up to `eventCapacity` events per block, each a phase with begin / end times, the peer it concerned
//    and the bytes and rows it moved.  tools/moonep/dispatch_trace.py turns a dump of the buffer into a Chrome /
//    Perfetto trace and a per-phase table.  Counterpart of the reference's dispatch trace
//    (src/moonep/dispatch/urma/common/dispatch_trace.h:16-80: 4 KiB header, per-core records, 15 phases); the phases
//    here are the ones this implementation has (there are no work-queue entries, doorbells or completion queues on
//    NVLink).
//
//  * a PROFILE RECORD per block of the combine stage, second generation (TileXRMoonEpCombineStageV2): cumulative
//    time points, counters, and the description of the first wait that gave up in that block.  Counterpart of
//    src/moonep/combine_v2/common/combine_v2_profile.h:16-141 (448-byte record, 22 time points, 10 metrics, failure
//    diagnostics); tools/moonep/combine_v2_trace.py decodes it.
//
// Times are nanoseconds of the GPU's global timer.
#ifndef TILEXR_MOONEP_TRACE_H
#define TILEXR_MOONEP_TRACE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TILEXR_MOONEP_TRACE_MARKER UINT32_C(0x544D5854)          /* "TXMT" */
#define TILEXR_MOONEP_TRACE_VERSION 1
#define TILEXR_MOONEP_TRACE_HEADER_BYTES 256
#define TILEXR_MOONEP_TRACE_MAX_ITERATIONS 100
#define TILEXR_MOONEP_TRACE_MAX_EVENTS_PER_BLOCK 4096
#define TILEXR_MOONEP_TRACE_NO_PEER (-1)

enum TileXRMoonEpTracePhase {
    TILEXR_MOONEP_TRACE_PLAN_CHECK = 0,     /* prologue: reuse guard and plan status */
    TILEXR_MOONEP_TRACE_ZERO_FILL = 1,      /* padding rows cleared */
    TILEXR_MOONEP_TRACE_ROUTE_SEND = 2,     /* rows stored to their destination slots (one event per block and peer) */
    TILEXR_MOONEP_TRACE_FLAG_RAISE = 3,     /* "this block has sent" published to every peer */
    TILEXR_MOONEP_TRACE_FLAG_WAIT = 4,      /* waiting for every sender block of every peer */
    TILEXR_MOONEP_TRACE_OUTPUT_COPY = 5,    /* window to output tensor (absent when peers wrote the tensor directly) */
    TILEXR_MOONEP_TRACE_PHASE_COUNT = 6
};

typedef struct TileXRMoonEpTraceHeader {
    uint32_t marker;
    uint16_t version;
    uint16_t headerBytes;
    uint32_t rank;
    uint32_t rankSize;
    uint32_t iterationCount;
    uint32_t blockCount;          /* blocks per iteration (the grid of the traced kernel) */
    uint32_t eventCapacity;       /* events per block record */
    uint32_t phaseCount;
    uint32_t blockRecordBytes;
    uint32_t eventBytes;
    uint64_t ticksPerUs;          /* 1000: times are nanoseconds */
    uint64_t traceBytes;
    uint64_t blockRecordOffset;
    uint64_t eventOffset;
    uint64_t reserved[23];
} TileXRMoonEpTraceHeader;

typedef struct TileXRMoonEpTraceBlockRecord {
    uint64_t beginNs;
    uint64_t endNs;
    uint64_t epoch;
    uint32_t iteration;
    uint32_t block;
    uint32_t rank;
    uint32_t eventCount;
    uint32_t droppedCount;        /* events that did not fit eventCapacity */
    uint32_t status;              /* TileXRDeviceStatus of the block's waits */
    uint64_t reserved[3];
} TileXRMoonEpTraceBlockRecord;

typedef struct TileXRMoonEpTraceEvent {
    uint64_t beginNs;
    uint64_t endNs;
    uint64_t bytes;
    uint64_t sequence;
    uint32_t phase;
    int32_t peer;
    uint32_t rows;
    uint32_t reserved;
} TileXRMoonEpTraceEvent;

/* Offsets and size of a trace buffer for `iterationCount` traced launches of `blockCount` blocks.  Returns 0, or -1
 * when a count is outside its range. */
#if defined(__CUDACC__)
#define TILEXR_TRACE_HD __host__ __device__
#else
#define TILEXR_TRACE_HD
#endif
TILEXR_TRACE_HD static inline int TileXRMoonEpTraceLayout(uint32_t iterationCount, uint32_t blockCount, uint32_t eventCapacity,
                                          uint64_t *blockRecordOffset, uint64_t *eventOffset, uint64_t *traceBytes)
{
    if (iterationCount == 0 || iterationCount > TILEXR_MOONEP_TRACE_MAX_ITERATIONS || blockCount == 0 || eventCapacity == 0 ||
        eventCapacity > TILEXR_MOONEP_TRACE_MAX_EVENTS_PER_BLOCK) {
        return -1;
    }
    const uint64_t records = (uint64_t)iterationCount * blockCount;
    *blockRecordOffset = TILEXR_MOONEP_TRACE_HEADER_BYTES;
    *eventOffset = *blockRecordOffset + records * sizeof(TileXRMoonEpTraceBlockRecord);
    *traceBytes = *eventOffset + records * eventCapacity * sizeof(TileXRMoonEpTraceEvent);
    return 0;
}

/* ---- combine, second generation: profile record ------------------------------------------------------------------ */

#define TILEXR_MOONEP_COMBINE_PROFILE_MARKER UINT32_C(0x50475854)  /* "TXGP" */
#define TILEXR_MOONEP_COMBINE_PROFILE_VERSION 1
#define TILEXR_MOONEP_COMBINE_PROFILE_MAX_BLOCKS 512

enum TileXRMoonEpCombineTimePoint {
    TILEXR_MOONEP_COMBINE_TIME_BEGIN = 0,          /* after the prologue (reuse guard, plan status) */
    TILEXR_MOONEP_COMBINE_TIME_INDEX_CLEARED = 1,  /* group index reset, all blocks met */
    TILEXR_MOONEP_COMBINE_TIME_INDEX_BUILT = 2,    /* every row entered into its (source, token) group, all blocks met */
    TILEXR_MOONEP_COMBINE_TIME_SEND_END = 3,       /* this block has no more groups to send */
    TILEXR_MOONEP_COMBINE_TIME_REDUCE_END = 4,     /* this block has no more tokens to reduce */
    TILEXR_MOONEP_COMBINE_TIME_END = 5,
    TILEXR_MOONEP_COMBINE_TIME_COUNT = 6
};

enum TileXRMoonEpCombineMetric {
    TILEXR_MOONEP_COMBINE_METRIC_ROWS_INDEXED = 0,   /* rows this block entered into the index */
    TILEXR_MOONEP_COMBINE_METRIC_GROUPS_SENT = 1,    /* rows that travelled (one per group) */
    TILEXR_MOONEP_COMBINE_METRIC_ROWS_FOLDED = 2,    /* rows summed into another row instead of travelling */
    TILEXR_MOONEP_COMBINE_METRIC_BYTES_SENT = 3,
    TILEXR_MOONEP_COMBINE_METRIC_REMOTE_GROUPS = 4,  /* of the groups sent, those that went to another rank */
    TILEXR_MOONEP_COMBINE_METRIC_TOKENS_REDUCED = 5,
    TILEXR_MOONEP_COMBINE_METRIC_SLOT_WAITS = 6,     /* flags waited for */
    TILEXR_MOONEP_COMBINE_METRIC_SLOT_WAIT_NS = 7,
    TILEXR_MOONEP_COMBINE_METRIC_PROBES = 8,         /* hash-table probes beyond the first */
    TILEXR_MOONEP_COMBINE_METRIC_COUNT = 9
};

typedef struct TileXRMoonEpCombineProfileRecord {
    uint32_t marker;
    uint16_t version;
    uint16_t recordBytes;
    uint32_t rank;
    uint32_t block;
    uint32_t blockDim;
    uint32_t gridDim;
    uint32_t timePointCount;
    uint32_t metricCount;
    uint64_t epoch;
    uint64_t timePoint[8];        /* ns; zero when the block never got there */
    uint64_t metric[12];
    /* the first wait of this block that gave up (all zero when none did) */
    uint32_t failureStatus;       /* TileXRDeviceStatus */
    uint32_t failureStep;         /* TileXRMoonEpCombineTimePoint reached before it */
    int32_t failurePeer;
    uint32_t failureReserved;
    int64_t failureSlot;
    uint64_t failureExpected;
    uint64_t failureObserved;
    uint64_t reserved[2];
} TileXRMoonEpCombineProfileRecord;

#ifdef __cplusplus
}
#endif

#endif /* TILEXR_MOONEP_TRACE_H */
