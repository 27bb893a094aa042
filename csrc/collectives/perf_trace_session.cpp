#include "perf_trace_session.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <sys/stat.h>

#include <cuda_runtime_api.h>

#include "tilexr_log.h"
#include "tilexr_types.h"

namespace TileXR {

namespace {

int CudaAlloc(void **p, size_t n) { return cudaMalloc(p, n) == cudaSuccess ? 0 : -1; }
int CudaRelease(void *p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
int CudaUpload(void *d, const void *s, size_t n, void *st)
{
    return cudaMemcpyAsync(d, s, n, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(st)) == cudaSuccess ? 0 : -1;
}
int CudaClear(void *d, size_t n, void *st) { return cudaMemsetAsync(d, 0, n, static_cast<cudaStream_t>(st)) == cudaSuccess ? 0 : -1; }
int CudaDownload(void *d, const void *s, size_t n)
{
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    return cudaMemcpy(d, s, n, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}

const PerfTraceRuntimeHooks kCudaHooks = {CudaAlloc, CudaRelease, CudaUpload, CudaClear, CudaDownload};
const PerfTraceRuntimeHooks *g_hooks = &kCudaHooks;

struct Session {
    bool enabled = false;
    std::string outputDir;
    unsigned sampleEveryN = 1;
    bool emitAiPrompt = false;
    std::string aiCommand;
    uint64_t launchesSeen = 0;
    struct Pending {
        uint64_t launchId;
        PerfLaunchInfo info;
        void *device;
        size_t bytes;
        // Header staged here until the asynchronous upload has certainly been consumed.
        TileXRPerfTraceHeader header;
    };
    std::vector<Pending *> pending;
};

std::mutex g_mutex;
Session *g_active = nullptr;

bool ProfilingDisabledByEnv()
{
    const char *v = std::getenv("TILEXR_COLLECTIVES_DISABLE_KERNEL_PROFILING");
    return v != nullptr && *v != '\0' && std::strcmp(v, "0") != 0;
}

void MakeDirs(const std::string &path)
{
    std::string cur;
    for (size_t i = 0; i <= path.size(); ++i) {
        if (i == path.size() || path[i] == '/') {
            if (!cur.empty()) mkdir(cur.c_str(), 0755);
        }
        if (i < path.size()) cur.push_back(path[i]);
    }
}

int Flush(Session *s, const char *incompleteReason)
{
    int result = TILEXR_SUCCESS;
    for (Session::Pending *p : s->pending) {
        PerfLaunchRecord rec;
        rec.launchId = p->launchId;
        rec.info = p->info;
        std::vector<uint8_t> raw(p->bytes);
        if (g_hooks->download(raw.data(), p->device, p->bytes) != 0) {
            result = TILEXR_ERROR_RUNTIME;
        } else {
            std::memcpy(&rec.header, raw.data(), sizeof(rec.header));
            const size_t n = static_cast<size_t>(rec.header.maxCoreCount) * rec.header.stageCount;
            rec.stats.resize(n);
            std::memcpy(rec.stats.data(), raw.data() + rec.header.statsOffset, n * sizeof(TileXRPerfCoreStageStats));
            std::ostringstream dir;
            dir << s->outputDir << "/rank" << p->info.rank << "/launch" << p->launchId;
            MakeDirs(dir.str());
            int ret = WriteLaunchReport(dir.str(), rec, s->emitAiPrompt, s->aiCommand,
                                        incompleteReason != nullptr ? incompleteReason : "");
            if (ret != TILEXR_SUCCESS) result = ret;
        }
        g_hooks->release(p->device);
        delete p;
    }
    s->pending.clear();
    return result;
}

} // namespace

void SetPerfTraceRuntimeHooksForTest(const PerfTraceRuntimeHooks *hooks)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    g_hooks = hooks != nullptr ? hooks : &kCudaHooks;
}

void *PerfTracePrepareLaunch(const PerfLaunchInfo &info, void *stream)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    Session *s = g_active;
    if (s == nullptr || !s->enabled || ProfilingDisabledByEnv()) return nullptr;
    const uint64_t id = s->launchesSeen++;
    if (s->sampleEveryN > 1 && (id % s->sampleEveryN) != 0) return nullptr;
    Session::Pending *p = new Session::Pending();
    p->launchId = id;
    p->info = info;
    p->bytes = TileXRPerfTraceBytes(info.blocks);
    p->device = nullptr;
    if (g_hooks->alloc(&p->device, p->bytes) != 0) {
        delete p;
        return nullptr;
    }
    TileXRPerfTraceHeader &h = p->header;
    std::memset(&h, 0, sizeof(h));
    h.magic = TILEXR_PERF_TRACE_MAGIC;
    h.version = TILEXR_PERF_TRACE_VERSION;
    h.headerSize = sizeof(TileXRPerfTraceHeader);
    h.stageDescSize = sizeof(TileXRPerfStageDesc);
    h.coreStageStatsSize = sizeof(TileXRPerfCoreStageStats);
    h.rank = info.rank;
    h.rankSize = info.rankSize;
    h.blockDim = info.blocks;
    h.maxCoreCount = info.blocks;
    h.stageCount = TILEXR_PERF_STAGE_COUNT;
    h.cycleToUsDivisor = TILEXR_PERF_TICKS_PER_US;
    h.launchId = id;
    h.messageBytes = info.messageBytes;
    h.opType = info.opType;
    h.dataType = info.dataType;
    h.statsOffset = TILEXR_PERF_TRACE_STATS_OFFSET;
    h.statsBytes = p->bytes - TILEXR_PERF_TRACE_STATS_OFFSET;
    if (g_hooks->clearAsync(p->device, p->bytes, stream) != 0 ||
        g_hooks->uploadAsync(p->device, &h, sizeof(h), stream) != 0) {
        g_hooks->release(p->device);
        delete p;
        return nullptr;
    }
    s->pending.push_back(p);
    return p->device;
}

} // namespace TileXR

using namespace TileXR;

extern "C" {

int TileXRCollectivePerfSessionCreate(const TileXRCollectivePerfConfig *config, TileXRCollectivePerfSession *session)
{
    if (config == nullptr || session == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (config->enabled && (config->outputDir == nullptr || *config->outputDir == '\0')) return TILEXR_ERROR_PARA_CHECK_FAIL;
    Session *s = new Session();
    s->enabled = config->enabled != 0;
    s->outputDir = config->outputDir != nullptr ? config->outputDir : "";
    s->sampleEveryN = config->sampleEveryN == 0 ? 1 : config->sampleEveryN;
    s->emitAiPrompt = config->emitAiPrompt != 0;
    s->aiCommand = config->aiCommand != nullptr ? config->aiCommand : "";
    *session = s;
    return TILEXR_SUCCESS;
}

int TileXRCollectivePerfSessionDestroy(TileXRCollectivePerfSession session)
{
    if (session == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    std::lock_guard<std::mutex> lock(g_mutex);
    Session *s = static_cast<Session *>(session);
    if (g_active == s) g_active = nullptr;
    for (Session::Pending *p : s->pending) {
        g_hooks->release(p->device);
        delete p;
    }
    delete s;
    return TILEXR_SUCCESS;
}

int TileXRCollectivePerfSetActiveSession(TileXRCollectivePerfSession session)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    g_active = static_cast<Session *>(session);   // null deactivates
    return TILEXR_SUCCESS;
}

int TileXRCollectivePerfWriteReport(TileXRCollectivePerfSession session)
{
    if (session == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    std::lock_guard<std::mutex> lock(g_mutex);
    return Flush(static_cast<Session *>(session), nullptr);
}

int TileXRCollectivePerfWriteIncompleteReport(TileXRCollectivePerfSession session, const char *reason)
{
    if (session == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    std::lock_guard<std::mutex> lock(g_mutex);
    return Flush(static_cast<Session *>(session), reason != nullptr ? reason : "incomplete");
}

} // extern "C"
