#include "tilexr_launch.h"

#include <atomic>
#include <cstring>
#include <functional>
#include <map>
#include <vector>

#include <cuda_runtime_api.h>

#include "comm.h"
#include "tilexr_log.h"

namespace TileXR {

namespace {

struct PendingLaunch {
    TileXRComm *comm;
    const KernelEntry *kernel;
    std::vector<uint8_t> args;
    LaunchConfig cfg;
    cudaStream_t stream;
    std::vector<std::function<int()>> after;     // host work to run once the launch has been issued (RunAfterLaunch)
};

struct GroupState {
    int depth = 0;
    std::vector<PendingLaunch> pending;
};

thread_local GroupState g_group;
std::atomic<uint64_t> g_launches{0};

int SetSmemLimit(const void *fn, size_t smemBytes)
{
    if (smemBytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytes));
        if (e != cudaSuccess) {
            TILEXR_LOG(ERROR) << "cudaFuncSetAttribute(smem=" << smemBytes << "): " << cudaGetErrorString(e);
            return TILEXR_ERROR_RUNTIME;
        }
    }
    return TILEXR_SUCCESS;
}

int IssueWorldLaunch(EmulatedWorld *world, std::vector<PendingLaunch *> &perRank)
{
    const PendingLaunch &first = *perRank[0];
    const int ranks = world->rankSize;
    for (int r = 0; r < ranks; ++r) {
        const PendingLaunch &p = *perRank[r];
        if (p.kernel != first.kernel || p.cfg.grid != first.cfg.grid || p.cfg.block != first.cfg.block ||
            p.cfg.smemBytes != first.cfg.smemBytes) {
            TILEXR_LOG(ERROR) << "emulated world: rank " << r << " queued " << p.kernel->name << " grid " << p.cfg.grid
                              << " but rank 0 queued " << first.kernel->name << " grid " << first.cfg.grid;
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
    }
    if (cudaSetDevice(world->device) != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    const size_t argBytes = first.kernel->argBytes;
    std::vector<uint8_t> packed(argBytes * ranks);
    for (int r = 0; r < ranks; ++r) std::memcpy(packed.data() + r * argBytes, perRank[r]->args.data(), argBytes);
    void *devArgs = nullptr;
    // stream-ordered scratch: freed after the kernel on the same stream
    if (cudaMallocAsync(&devArgs, packed.size(), first.stream) != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    if (cudaMemcpyAsync(devArgs, packed.data(), packed.size(), cudaMemcpyHostToDevice, first.stream) != cudaSuccess) {
        return TILEXR_ERROR_RUNTIME;
    }
    // pageable source: the copy is staged before the call returns, `packed` may go away
    int ret = SetSmemLimit(first.kernel->emulated, first.cfg.smemBytes);
    if (ret != TILEXR_SUCCESS) return ret;
    void *params[] = {&devArgs};
    const dim3 grid(first.cfg.grid, ranks, 1);
    const dim3 block(first.cfg.block, 1, 1);
    cudaError_t e = cudaLaunchCooperativeKernel(first.kernel->emulated, grid, block, params, first.cfg.smemBytes,
                                                first.stream);
    cudaFreeAsync(devArgs, first.stream);
    if (e != cudaSuccess) {
        TILEXR_LOG(ERROR) << "cooperative launch of " << first.kernel->name << " for " << ranks << " emulated ranks x "
                          << first.cfg.grid << " blocks failed: " << cudaGetErrorString(e);
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    g_launches.fetch_add(1);
    return TILEXR_SUCCESS;
}

} // namespace

uint64_t LaunchCount() { return g_launches.load(); }
void NoteLaunch() { g_launches.fetch_add(1); }

int LaunchKernel(TileXRCommPtr commPtr, const KernelEntry &kernel, const void *args, const LaunchConfig &cfg,
                 TileXRStream streamPtr)
{
    TileXRComm *comm = static_cast<TileXRComm *>(commPtr);
    cudaStream_t stream = static_cast<cudaStream_t>(streamPtr);
    if (comm == nullptr || !comm->initialized()) return TILEXR_ERROR_NOT_INITIALIZED;
    if (comm->isHostMemory()) return TILEXR_ERROR_NOT_SUPPORT;
    if (comm->isEmulated()) {
        if (g_group.depth == 0) {
            TILEXR_LOG(ERROR) << kernel.name << ": a communicator of an emulated world launches only inside "
                              << "TileXRGroupStart/TileXRGroupEnd";
            return TILEXR_ERROR_NOT_SUPPORT;
        }
        PendingLaunch p;
        p.comm = comm;
        p.kernel = &kernel;
        p.args.assign(static_cast<const uint8_t *>(args), static_cast<const uint8_t *>(args) + kernel.argBytes);
        p.cfg = cfg;
        p.stream = stream;
        g_group.pending.push_back(std::move(p));
        return TILEXR_SUCCESS;
    }
    int ret = SetSmemLimit(kernel.single, cfg.smemBytes);
    if (ret != TILEXR_SUCCESS) return ret;
    void *params[] = {const_cast<void *>(args)};
    cudaError_t e;
    if (cfg.cooperative) {
        e = cudaLaunchCooperativeKernel(kernel.single, dim3(cfg.grid), dim3(cfg.block), params, cfg.smemBytes, stream);
    } else {
        e = cudaLaunchKernel(kernel.single, dim3(cfg.grid), dim3(cfg.block), params, cfg.smemBytes, stream);
    }
    if (e != cudaSuccess) {
        TILEXR_LOG(ERROR) << "launch of " << kernel.name << " grid " << cfg.grid << " block " << cfg.block << " smem "
                          << cfg.smemBytes << " failed: " << cudaGetErrorString(e);
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    g_launches.fetch_add(1);
    return TILEXR_SUCCESS;
}

int RunAfterLaunch(TileXRCommPtr commPtr, std::function<int()> fn)
{
    TileXRComm *comm = static_cast<TileXRComm *>(commPtr);
    if (comm != nullptr && comm->isEmulated() && g_group.depth > 0) {
        for (auto it = g_group.pending.rbegin(); it != g_group.pending.rend(); ++it) {
            if (it->comm == comm) {
                it->after.push_back(std::move(fn));
                return TILEXR_SUCCESS;
            }
        }
    }
    return fn();
}

int MaxCooperativeGrid(TileXRCommPtr commPtr, const KernelEntry &kernel, unsigned block, size_t smemBytes,
                       int ranksPerDevice, unsigned *maxGrid)
{
    TileXRComm *comm = static_cast<TileXRComm *>(commPtr);
    if (comm == nullptr || !comm->initialized() || comm->isHostMemory()) return TILEXR_ERROR_NOT_INITIALIZED;
    const void *fn = comm->isEmulated() ? kernel.emulated : kernel.single;
    int ret = SetSmemLimit(fn, smemBytes);
    if (ret != TILEXR_SUCCESS) return ret;
    int perSm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, fn, static_cast<int>(block), smemBytes) != cudaSuccess) {
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, comm->device()) != cudaSuccess) {
        return TILEXR_ERROR_RUNTIME;
    }
    const int total = perSm * sms;
    *maxGrid = static_cast<unsigned>(total / (ranksPerDevice > 0 ? ranksPerDevice : 1));
    return TILEXR_SUCCESS;
}

extern "C" int TileXRGroupStart(void)
{
    g_group.depth += 1;
    return TILEXR_SUCCESS;
}

extern "C" int TileXRGroupEnd(void)
{
    if (g_group.depth == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    g_group.depth -= 1;
    if (g_group.depth > 0) return TILEXR_SUCCESS;
    std::vector<PendingLaunch> pending;
    pending.swap(g_group.pending);
    // The k-th call of every rank of a world forms the k-th launch of that world.
    std::map<EmulatedWorld *, std::vector<std::vector<PendingLaunch *>>> byWorld;
    for (PendingLaunch &p : pending) {
        EmulatedWorld *w = p.comm->world();
        std::vector<std::vector<PendingLaunch *>> &perRank = byWorld[w];
        if (perRank.empty()) perRank.resize(w->rankSize);
        perRank[p.comm->rank()].push_back(&p);
    }
    int result = TILEXR_SUCCESS;
    for (auto &kv : byWorld) {
        EmulatedWorld *w = kv.first;
        const size_t calls = kv.second[0].size();
        for (int r = 0; r < w->rankSize; ++r) {
            if (kv.second[r].size() != calls) {
                TILEXR_LOG(ERROR) << "emulated world: rank " << r << " queued " << kv.second[r].size()
                                  << " launches, rank 0 queued " << calls;
                return TILEXR_ERROR_PARA_CHECK_FAIL;
            }
        }
        for (size_t k = 0; k < calls; ++k) {
            std::vector<PendingLaunch *> row(w->rankSize);
            for (int r = 0; r < w->rankSize; ++r) row[r] = kv.second[r][k];
            int ret = IssueWorldLaunch(w, row);
            if (ret != TILEXR_SUCCESS) result = ret;
            for (PendingLaunch *p : row) {
                for (auto &fn : p->after) {
                    ret = fn();
                    if (ret != TILEXR_SUCCESS) result = ret;
                }
            }
        }
    }
    return result;
}

} // namespace TileXR
