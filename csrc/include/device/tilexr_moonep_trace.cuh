// Device side of the MoonEP event trace (tilexr_moonep_trace.h): one thread of a block opens and closes phases;
// a null buffer makes every call a no-op, so kernels carry the calls unconditionally.
#ifndef TILEXR_MOONEP_TRACE_CUH
#define TILEXR_MOONEP_TRACE_CUH

#include "../tilexr_moonep_trace.h"
#include "tilexr_platform.cuh"

namespace tilexr {

struct MoonTrace {
    TileXRMoonEpTraceBlockRecord *record;   // null: tracing is off (or this is not the recording thread)
    TileXRMoonEpTraceEvent *events;
    uint32_t capacity;
    uint32_t count;
    uint32_t dropped;
    uint64_t openedNs;
};

// `buffer` holds header + block records + events for `iterationCount` launches; this launch is `iteration`.
// Call from the one thread that records (thread 0).  The header is written by block 0.
TXR_D MoonTrace MoonTraceOpen(void *buffer, uint32_t iteration, uint32_t iterationCount, uint32_t eventCapacity, uint32_t rank,
                              uint32_t rankSize, uint32_t block, uint32_t blocks, uint64_t epoch)
{
    MoonTrace t{nullptr, nullptr, 0, 0, 0, 0};
    uint64_t recOff = 0, evOff = 0, total = 0;
    if (buffer == nullptr || iteration >= iterationCount ||
        TileXRMoonEpTraceLayout(iterationCount, blocks, eventCapacity, &recOff, &evOff, &total) != 0) {
        return t;
    }
    uint8_t *base = reinterpret_cast<uint8_t *>(buffer);
    if (block == 0) {
        TileXRMoonEpTraceHeader *h = reinterpret_cast<TileXRMoonEpTraceHeader *>(base);
        h->marker = TILEXR_MOONEP_TRACE_MARKER;
        h->version = TILEXR_MOONEP_TRACE_VERSION;
        h->headerBytes = TILEXR_MOONEP_TRACE_HEADER_BYTES;
        h->rank = rank;
        h->rankSize = rankSize;
        h->iterationCount = iterationCount;
        h->blockCount = blocks;
        h->eventCapacity = eventCapacity;
        h->phaseCount = TILEXR_MOONEP_TRACE_PHASE_COUNT;
        h->blockRecordBytes = sizeof(TileXRMoonEpTraceBlockRecord);
        h->eventBytes = sizeof(TileXRMoonEpTraceEvent);
        h->ticksPerUs = 1000;
        h->traceBytes = total;
        h->blockRecordOffset = recOff;
        h->eventOffset = evOff;
    }
    const uint64_t index = static_cast<uint64_t>(iteration) * blocks + block;
    t.record = reinterpret_cast<TileXRMoonEpTraceBlockRecord *>(base + recOff) + index;
    t.events = reinterpret_cast<TileXRMoonEpTraceEvent *>(base + evOff) + index * eventCapacity;
    t.capacity = eventCapacity;
    t.record->beginNs = now_ns();
    t.record->endNs = 0;
    t.record->epoch = epoch;
    t.record->iteration = iteration;
    t.record->block = block;
    t.record->rank = rank;
    t.record->eventCount = 0;
    t.record->droppedCount = 0;
    t.record->status = 0;
    return t;
}

TXR_D void MoonTraceBegin(MoonTrace &t)
{
    if (t.record != nullptr) t.openedNs = now_ns();
}

// Closes the phase opened last.
TXR_D void MoonTraceEnd(MoonTrace &t, uint32_t phase, int32_t peer, uint64_t bytes, uint32_t rows)
{
    if (t.record == nullptr) return;
    if (t.count >= t.capacity) {
        t.dropped += 1;
        return;
    }
    TileXRMoonEpTraceEvent &e = t.events[t.count];
    e.beginNs = t.openedNs;
    e.endNs = now_ns();
    e.bytes = bytes;
    e.sequence = t.count;
    e.phase = phase;
    e.peer = peer;
    e.rows = rows;
    e.reserved = 0;
    t.count += 1;
}

TXR_D void MoonTraceClose(MoonTrace &t, uint32_t status)
{
    if (t.record == nullptr) return;
    t.record->endNs = now_ns();
    t.record->eventCount = t.count;
    t.record->droppedCount = t.dropped;
    t.record->status = status;
}

} // namespace tilexr

#endif // TILEXR_MOONEP_TRACE_CUH
