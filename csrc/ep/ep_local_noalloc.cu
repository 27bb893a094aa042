// Single-GPU MoE dispatch whose scratch memory is a fixed array inside the library image
// (see tilexr_noalloc.h for why).  One cooperative kernel:
//   1. each block ranks the routes of its token range per expert and stores its per-expert
//      counts into the scratch table;
//   2. after a barrier among the blocks, each block derives the first output row of every
//      expert and its own offset inside it, then copies its rows and writes the assist tuples.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <mutex>
#include <cuda_runtime_api.h>

#include "device/tilexr_rma.cuh"
#include "device/tilexr_route_rank.cuh"
#include "tilexr_noalloc.h"
#include "tilexr_types.h"

namespace {

using namespace tilexr;

constexpr unsigned THREADS = 512;
constexpr unsigned WARPS = THREADS / 32;
constexpr int MAX_ROUTES_PER_BLOCK = 4096;
constexpr int MAX_DEVICES = 64;

// `barrier` holds (call number << 32) | blocks that arrived.  Its first arriver of a call finds another call's number
// (or a count that is already complete or poisoned) and restarts the word, so nothing has to be put back at the end
// of a call and a call whose barrier gave up leaves nothing that the next call could trip over.
struct Scratch {
    unsigned long long barrier;
    int32_t status;
    int32_t pad[61];
    int32_t blockCounts[TILEXR_NOALLOC_MAX_BLOCKS][TILEXR_NOALLOC_MAX_EXPERTS];
};

// The scratch memory.  In host code this name is only a stand-in for the symbol: the device
// address comes from cudaGetSymbolAddress at set-up.
static __device__ __align__(256) unsigned char g_scratchBytes[sizeof(Scratch)];

struct Args {
    const uint8_t *x;
    const int32_t *ids;
    uint8_t *expandX;
    int32_t *assist;
    int64_t *tokenNums;
    int32_t *sendCounts;
    Scratch *scratch;
    int32_t bs, topK, experts;
    uint32_t rowBytes;
    uint32_t tokensPerBlock;
    uint32_t call;            // number of this call on its device, from 1
};

constexpr uint32_t BARRIER_POISON = 0xffffffffu;

__global__ void __launch_bounds__(THREADS) LocalDispatchKernel(const Args a)
{
    extern __shared__ __align__(16) uint8_t smemRaw[];
    const int E = a.experts, K = a.topK;
    const int routesPerBlock = static_cast<int>(a.tokensPerBlock) * K;
    int32_t *sExpert = reinterpret_cast<int32_t *>(smemRaw);
    int32_t *sRank = sExpert + routesPerBlock;
    int32_t *sHist = sRank + routesPerBlock;
    int32_t *sRow = sHist + E;        // first output row of this block's routes to expert e
    int32_t *sTotal = sRow + E;
    Scratch *sc = a.scratch;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x;
    const int t0 = min(a.bs, static_cast<int>(blockIdx.x * a.tokensPerBlock));
    const int t1 = min(a.bs, t0 + static_cast<int>(a.tokensPerBlock));
    const int nRoutes = (t1 - t0) * K;

    if (blockIdx.x == 0 && tid == 0) sc->status = 0;
    for (int e = tid; e < E; e += blockDim.x) sHist[e] = 0;
    for (int i = tid; i < nRoutes; i += blockDim.x) {
        int e = a.ids[static_cast<int64_t>(t0) * K + i];
        if (e < 0 || e >= E) e = -1;
        sExpert[i] = e;
    }
    __syncthreads();
    // rank of each route among the block's routes to its expert, and the per-expert counts: one warp, linear time
    if (warp == 0) RankRoutesByWarp(sExpert, sRank, sHist, nRoutes, lane);
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) sc->blockCounts[blockIdx.x][e] = sHist[e];

    // barrier among the blocks (all resident: cooperative launch); bounded
    __syncthreads();
    __shared__ int sOk;
    if (tid == 0) {
        sOk = 1;
        __threadfence();              // this block's counts before its arrival
        // arrive: continue this call's count, or restart a word that another call (or a poisoned one) left
        unsigned long long seen = *reinterpret_cast<volatile unsigned long long *>(&sc->barrier);
        for (;;) {
            const bool mine = static_cast<uint32_t>(seen >> 32) == a.call && static_cast<uint32_t>(seen) < static_cast<uint32_t>(G);
            const unsigned long long next = mine ? seen + 1ull : ((static_cast<unsigned long long>(a.call) << 32) | 1ull);
            const unsigned long long old = atomicCAS(&sc->barrier, seen, next);
            if (old == seen) break;
            seen = old;
        }
        __threadfence();
        const unsigned long long full = (static_cast<unsigned long long>(a.call) << 32) | static_cast<uint32_t>(G);
        const uint64_t deadline = now_ns() + 2000000000ull;
        uint32_t polls = 0;
        for (;;) {
            const unsigned long long v = *reinterpret_cast<volatile unsigned long long *>(&sc->barrier);
            if (v == full) break;
            const bool poisoned = static_cast<uint32_t>(v >> 32) == a.call && static_cast<uint32_t>(v) == BARRIER_POISON;
            if (poisoned || ((++polls & 255u) == 0 && now_ns() > deadline)) {
                // give up, and make every other block of this call give up at once instead of after its own two seconds
                atomicExch(&sc->barrier, (static_cast<unsigned long long>(a.call) << 32) | BARRIER_POISON);
                sOk = 0;
                atomicExch(&sc->status, 5);
                break;
            }
        }
        __threadfence();
    }
    __syncthreads();
    if (sOk == 0) return;

    for (int e = tid; e < E; e += blockDim.x) {
        int total = 0, before = 0;
        for (int b = 0; b < G; ++b) {
            const int c = sc->blockCounts[b][e];
            total += c;
            if (b < static_cast<int>(blockIdx.x)) before += c;
        }
        sTotal[e] = total;
        sRow[e] = before;
    }
    __syncthreads();
    if (tid == 0) {
        int running = 0;
        for (int e = 0; e < E; ++e) {
            const int start = running;
            running += sTotal[e];
            sRow[e] += start;
            if (blockIdx.x == 0) {
                a.tokenNums[e] = sTotal[e];
                a.sendCounts[e] = running;
            }
        }
    }
    __syncthreads();
    for (int i = warp; i < nRoutes; i += WARPS) {
        const int e = sExpert[i];
        if (e < 0) continue;
        const int token = t0 + i / K;
        const int k = i % K;
        const int64_t row = sRow[e] + sRank[i];
        CopyLanes(a.expandX + row * a.rowBytes, a.x + static_cast<int64_t>(token) * a.rowBytes, a.rowBytes, lane, 32);
        if (lane == 0) {
            st_vec16(a.assist + row * 4, Vec16{0u, static_cast<uint32_t>(token), static_cast<uint32_t>(k), static_cast<uint32_t>(e)});
        }
    }
}

// Per device: the scratch array's address (looked up once, under the flag) and the number of calls made.
Scratch *g_devicePtr[MAX_DEVICES] = {};
std::once_flag g_deviceOnce[MAX_DEVICES];
std::atomic<uint32_t> g_deviceCalls[MAX_DEVICES];

void LookUpScratch(int dev)
{
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_scratchBytes);
    if (e != cudaSuccess || p == nullptr) {
        std::fprintf(stderr, "[TileXR] cudaGetSymbolAddress(scratch) failed: %s\n", cudaGetErrorString(e));
        return;
    }
    if (cudaMemset(p, 0, 256) != cudaSuccess) return;     // barrier word and status
    g_devicePtr[dev] = static_cast<Scratch *>(p);
}

} // namespace

extern "C" {

int TileXRMoeLocalDispatchNoAlloc(const void *x, const int32_t *expertIds, int64_t bs, int64_t h, int64_t topK,
                                  int64_t moeExpertNum, void *expandXOut, int32_t *assistOut, int64_t *expertTokenNumsOut,
                                  int32_t *sendCountsOut, int dtype, TileXRStream stream)
{
    using namespace TileXR;
    if (x == nullptr || expertIds == nullptr || expandXOut == nullptr || assistOut == nullptr || expertTokenNumsOut == nullptr ||
        sendCountsOut == nullptr || bs <= 0 || h <= 0 || topK <= 0 || moeExpertNum <= 0 ||
        (dtype != TILEXR_DATA_TYPE_FP16 && dtype != TILEXR_DATA_TYPE_BFP16) || (h * 2) % 16 != 0) {
        std::fprintf(stderr, "[TileXR] TileXRMoeLocalDispatchNoAlloc: bad arguments\n");
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (moeExpertNum > TILEXR_NOALLOC_MAX_EXPERTS || bs * topK > TILEXR_NOALLOC_MAX_ROUTES) {
        std::fprintf(stderr,
                     "[TileXR] TileXRMoeLocalDispatchNoAlloc: %lld experts / %lld routes exceed the built-in scratch "
                     "(at most %d experts, %d routes); use TileXRMoeEpDispatchFused with a communicator instead\n",
                     static_cast<long long>(moeExpertNum), static_cast<long long>(bs * topK), TILEXR_NOALLOC_MAX_EXPERTS,
                     TILEXR_NOALLOC_MAX_ROUTES);
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return TILEXR_ERROR_RUNTIME;
    // once per device, with that device current; host threads that make their first calls together wait for the one
    // that does the lookup
    std::call_once(g_deviceOnce[dev], LookUpScratch, dev);
    if (g_devicePtr[dev] == nullptr) return TILEXR_ERROR_RUNTIME;
    // grid: blocks must be co-resident (they meet at a barrier)
    unsigned grid = static_cast<unsigned>(std::min<int64_t>(TILEXR_NOALLOC_MAX_BLOCKS, (bs + 15) / 16));
    if (grid == 0) grid = 1;
    uint32_t tokensPerBlock = 0;
    size_t smem = 0;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    for (;;) {
        tokensPerBlock = static_cast<uint32_t>((bs + grid - 1) / grid);
        if (static_cast<int64_t>(tokensPerBlock) * topK > MAX_ROUTES_PER_BLOCK) {
            std::fprintf(stderr, "[TileXR] TileXRMoeLocalDispatchNoAlloc: %u tokens x %lld routes per block exceed %d\n",
                         tokensPerBlock, static_cast<long long>(topK), MAX_ROUTES_PER_BLOCK);
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
        smem = static_cast<size_t>(tokensPerBlock) * topK * 8 + static_cast<size_t>(moeExpertNum) * 12;
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(LocalDispatchKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
            return TILEXR_ERROR_RUNTIME;
        }
        int perSm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, LocalDispatchKernel, THREADS, smem) != cudaSuccess || perSm <= 0) {
            return TILEXR_ERROR_RUNTIME;
        }
        const unsigned maxGrid = static_cast<unsigned>(perSm * sms);
        if (grid <= maxGrid) break;
        grid = maxGrid;
    }
    grid = static_cast<unsigned>((bs + tokensPerBlock - 1) / tokensPerBlock);
    Args a;
    a.x = static_cast<const uint8_t *>(x);
    a.ids = expertIds;
    a.expandX = static_cast<uint8_t *>(expandXOut);
    a.assist = assistOut;
    a.tokenNums = expertTokenNumsOut;
    a.sendCounts = sendCountsOut;
    a.scratch = g_devicePtr[dev];
    a.bs = static_cast<int32_t>(bs);
    a.topK = static_cast<int32_t>(topK);
    a.experts = static_cast<int32_t>(moeExpertNum);
    a.rowBytes = static_cast<uint32_t>(h * 2);
    a.tokensPerBlock = tokensPerBlock;
    a.call = g_deviceCalls[dev].fetch_add(1, std::memory_order_relaxed) + 1u;
    void *params[] = {&a};
    const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&LocalDispatchKernel), dim3(grid), dim3(THREADS),
                                                      params, smem, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        std::fprintf(stderr, "[TileXR] TileXRMoeLocalDispatchNoAlloc launch failed: %s\n", cudaGetErrorString(e));
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    return TILEXR_SUCCESS;
}

int TileXRMoeLocalDispatchNoAllocStatus(int *status)
{
    using namespace TileXR;
    if (status == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return TILEXR_ERROR_RUNTIME;
    *status = 0;
    if (g_devicePtr[dev] == nullptr) return TILEXR_SUCCESS;
    if (cudaDeviceSynchronize() != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    int32_t v = 0;
    if (cudaMemcpy(&v, &g_devicePtr[dev]->status, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    *status = v;
    return TILEXR_SUCCESS;
}

} // extern "C"
