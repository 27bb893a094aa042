// Recorder behind the observation points of tilexr_platform.cuh: while it is switched on for a host-memory
// communicator, every flag store, finished wait, window copy and window read that the PRODUCTION primitives
// (tilexr_sync.cuh compiled for the host, driven by the CPU kernels of hostsim.cpp) perform on this rank becomes
// one line of the protocol checker's event format.  Event ids come from one counter in rank 0's window, so the
// files of all ranks merge into one global order; stores and copies take their id BEFORE they are performed and
// waits AFTER they end, so an event that depends on another always has the larger id.  The checker then judges
// what the production code did (csrc/checker: CheckOrdering) -- a wrong flag slot or a missing wait in
// tilexr_sync.cuh or hostsim.cpp shows up as a finding, which a hand-written model of the protocol could not see.
//
// Reference: tools/checker/shim/tilexr/checker/collective_trace_shim.h and tools/checker/src/trace_runtime.cpp
// (kernel headers replayed through recording shims).
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "device/tilexr_sync.cuh"
#include "tilexr_hostsim.h"
#include "tilexr_log.h"
#include "tilexr_types.h"

using namespace TileXR;
using namespace tilexr;

namespace {

constexpr int64_t CHECKER_SLOT_DONE_BASE = 1 << 20;     // the checker's numbering of the done-epoch words
constexpr int TRACE_COUNTER_WORD = TILEXR_CTRL_SCRATCH_WORD + 4000;

struct Recorder {
    HostTraceHooks hooks{};
    CommArgs *args = nullptr;
    std::FILE *file = nullptr;
    uint64_t events = 0;
};

std::mutex g_mutex;
std::map<TileXRCommPtr, Recorder *> g_recorders;

uint64_t NextId(Recorder *r)
{
    uint64_t *counter = CtrlWord(r->args, 0, TRACE_COUNTER_WORD);
    return __atomic_fetch_add(counter, 1, __ATOMIC_ACQ_REL);
}

// Which rank's window holds `addr`, and where inside it.
bool Locate(const Recorder *r, const void *addr, int *owner, uint64_t *offset)
{
    const uint8_t *p = static_cast<const uint8_t *>(addr);
    for (int i = 0; i < r->args->rankSize; ++i) {
        const uint8_t *base = r->args->peerMems[i];
        if (p >= base && p < base + r->args->peerMemBytes) {
            *owner = i;
            *offset = static_cast<uint64_t>(p - base);
            return true;
        }
    }
    return false;
}

// Flag slot in the checker's numbering, or -1 for a word that is not part of a protocol (abort word, barriers, scratch).
int64_t FlagSlotOf(uint64_t offset)
{
    if (offset >= TILEXR_WIN_FLAG_OFFSET && offset < TILEXR_WIN_FLAG_OFFSET + TILEXR_WIN_FLAG_BYTES) {
        return static_cast<int64_t>((offset - TILEXR_WIN_FLAG_OFFSET) / 8);
    }
    const uint64_t word = offset / 8;
    if (offset < TILEXR_WIN_CTRL_BYTES && word >= TILEXR_CTRL_DONE_WORD && word < TILEXR_CTRL_DONE_WORD + TILEXR_MAX_RANK_SIZE) {
        return CHECKER_SLOT_DONE_BASE + static_cast<int64_t>(word - TILEXR_CTRL_DONE_WORD);
    }
    return -1;
}

void Emit(Recorder *r, uint64_t id, const char *kind, int peer, const char *role, int64_t slot, int64_t magic, uint64_t offset, uint64_t bytes,
          int satisfied, const char *source)
{
    std::fprintf(r->file,
                 "{\"id\": %llu, \"kind\": \"%s\", \"rank\": %d, \"peer\": %d, \"block\": 0, \"role\": \"%s\", \"slot\": %lld, \"pipe\": -1, "
                 "\"magic\": %lld, \"offset\": %llu, \"bytes\": %llu, \"satisfied\": %d, \"source\": \"%s\"}\n",
                 static_cast<unsigned long long>(id), kind, r->args->rank, peer, role, static_cast<long long>(slot), static_cast<long long>(magic),
                 static_cast<unsigned long long>(offset), static_cast<unsigned long long>(bytes), satisfied, source);
    r->events += 1;
}

void OnFlagStore(void *ctx, const void *addr, uint64_t value)
{
    Recorder *r = static_cast<Recorder *>(ctx);
    int owner = 0;
    uint64_t off = 0;
    if (!Locate(r, addr, &owner, &off)) return;
    const int64_t slot = FlagSlotOf(off);
    if (slot < 0) return;
    Emit(r, NextId(r), "FlagStore", owner, "comm_flag", slot, static_cast<int64_t>(value), 0, 8, 1, "tilexr_sync.cuh:SetFlag/PublishDone");
}

void OnFlagWait(void *ctx, const void *addr, uint64_t want, uint64_t seen, int peer, int satisfied)
{
    (void)seen;
    Recorder *r = static_cast<Recorder *>(ctx);
    int owner = 0;
    uint64_t off = 0;
    if (!Locate(r, addr, &owner, &off)) return;
    const int64_t slot = FlagSlotOf(off);
    if (slot < 0) return;
    Emit(r, NextId(r), "FlagWait", peer, "comm_flag", slot, static_cast<int64_t>(want), 0, 8, satisfied, "tilexr_sync.cuh:WaitFlagGE/WaitPeerFinished");
}

// Data events are keyed (owner, region 0, epoch) with the byte offset inside the data half of that epoch.
void DataEvent(Recorder *r, const char *kind, const void *addr, uint64_t bytes, const char *source)
{
    int owner = 0;
    uint64_t off = 0;
    if (!Locate(r, addr, &owner, &off) || off < TILEXR_WIN_DATA_OFFSET) return;
    const uint64_t inner = (off - TILEXR_WIN_DATA_OFFSET) % r->args->dataHalfBytes;
    Emit(r, NextId(r), kind, owner, "comm_data", 0, static_cast<int64_t>(r->hooks.epoch), inner, bytes, 1, source);
}

void OnCopy(void *ctx, const void *dst, const void *src, uint64_t bytes)
{
    (void)src;
    DataEvent(static_cast<Recorder *>(ctx), "Copy", dst, bytes, "hostsim.cpp:window store");
}

void OnRead(void *ctx, const void *src, uint64_t bytes) { DataEvent(static_cast<Recorder *>(ctx), "Read", src, bytes, "hostsim.cpp:window load"); }

} // namespace

extern "C" {

int TileXRHostTraceStart(TileXRCommPtr comm, const char *path)
{
    TileXRCommArgs *args = nullptr;
    if (path == nullptr || TileXRGetCommArgsHost(comm, &args) != TILEXR_SUCCESS) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if ((args->extraFlag & TILEXR_FLAG_HOST_MEMORY) == 0) return TILEXR_ERROR_NOT_SUPPORT;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_recorders.count(comm) != 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    Recorder *r = new Recorder();
    r->file = std::fopen(path, "w");
    if (r->file == nullptr) {
        delete r;
        return TILEXR_ERROR_INTERNAL;
    }
    r->args = args;
    r->hooks.onFlagStore = OnFlagStore;
    r->hooks.onFlagWait = OnFlagWait;
    r->hooks.onCopy = OnCopy;
    r->hooks.onRead = OnRead;
    r->hooks.ctx = r;
    r->hooks.epoch = 0;
    g_recorders[comm] = r;
    Emit(r, NextId(r), "RankStart", -1, "none", -1, 0, 0, 0, 1, "TileXRHostTraceStart");
    HostTraceSlot() = &r->hooks;          // the kernels of this communicator run on the calling thread
    return TILEXR_SUCCESS;
}

int TileXRHostTraceStop(TileXRCommPtr comm, uint64_t *eventCount)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_recorders.find(comm);
    if (it == g_recorders.end()) return TILEXR_ERROR_NOT_FOUND;
    Recorder *r = it->second;
    if (HostTraceSlot() == &r->hooks) HostTraceSlot() = nullptr;
    Emit(r, NextId(r), "RankEnd", -1, "none", -1, 0, 0, 0, 1, "TileXRHostTraceStop");
    if (eventCount != nullptr) *eventCount = r->events;
    std::fclose(r->file);
    delete r;
    g_recorders.erase(it);
    return TILEXR_SUCCESS;
}

} // extern "C"
