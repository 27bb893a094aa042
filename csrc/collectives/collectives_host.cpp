// Host side of the collectives library: argument validation, splitting a call into
// launches that fit the window, choosing tile size and block roles, launching.
// (Reference: src/collectives/host/tilexr_collectives.cpp:20-134, collective_utils.cpp:20-234.)
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <limits>

#include <cuda_runtime_api.h>

#include "coll_kernels.cuh"
#include "perf_trace_session.h"
#include "tilexr_collectives.h"
#include "tilexr_log.h"

using namespace TileXR;

namespace {

long EnvLong(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

bool IsReduceType(int dtype)
{
    switch (dtype) {
        case TILEXR_DATA_TYPE_INT8: case TILEXR_DATA_TYPE_INT16: case TILEXR_DATA_TYPE_INT32: case TILEXR_DATA_TYPE_INT64:
        case TILEXR_DATA_TYPE_FP16: case TILEXR_DATA_TYPE_FP32: case TILEXR_DATA_TYPE_BFP16:
            return true;
        default:
            return false;
    }
}

bool MulOverflows(uint64_t a, uint64_t b, uint64_t *out)
{
    if (a != 0 && b > std::numeric_limits<uint64_t>::max() / a) return true;
    *out = a * b;
    return false;
}

uint64_t RoundUp(uint64_t v, uint64_t m) { return (v + m - 1) / m * m; }

uint64_t OneShotMaxBytes() { return static_cast<uint64_t>(EnvLong("TILEXR_AR_ONESHOT_MAX_BYTES", 256 * 1024)); }

struct Geometry {
    int32_t kind;
    uint32_t tileBytes;
    uint64_t bytesPerLaunch;   // slice bytes per launch (two-shot: vector bytes per launch)
    uint32_t launches;
    uint32_t producers, reducers, consumers;
    uint32_t pairStride;
};

// Pure arithmetic: how `sliceBytes` per pair (or `sliceBytes` total for the all-reduce kinds)
// is cut into launches and tiles, and how many blocks take which role.
int Plan(int kind, uint64_t sliceBytes, int rankSize, uint64_t dataHalfBytes, unsigned maxGrid, Geometry *g)
{
    if (rankSize < 2 || dataHalfBytes < (1u << 20)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    std::memset(g, 0, sizeof(*g));
    g->kind = kind;
    const uint64_t pairStride = (dataHalfBytes / rankSize) & ~static_cast<uint64_t>(255);
    if (pairStride > 0xffffff00ull) return TILEXR_ERROR_PARA_CHECK_FAIL;
    g->pairStride = static_cast<uint32_t>(pairStride);
    const bool twoShot = kind == COLL_ALL_REDUCE_TWO_SHOT;
    const uint32_t planes = twoShot ? 2 : 1;

    // bytes that one pair moves per launch, before cutting into tiles
    uint64_t perPair = twoShot ? RoundUp((sliceBytes + rankSize - 1) / rankSize, 512) : sliceBytes;
    if (perPair == 0) perPair = 16;

    uint32_t tile = static_cast<uint32_t>(EnvLong("TILEXR_COLL_TILE_BYTES", 0));
    if (tile == 0) {
        if (perPair <= 32 * 1024) {
            tile = static_cast<uint32_t>(RoundUp(perPair, 16));
        } else {
            const uint64_t want = RoundUp(perPair / 32, 16 * 1024);
            tile = static_cast<uint32_t>(std::min<uint64_t>(std::max<uint64_t>(want, 16 * 1024), TILEXR_TILE_BYTES));
        }
    }
    tile = static_cast<uint32_t>(RoundUp(tile, 16));
    const uint64_t capacity = std::min<uint64_t>(pairStride / planes / tile, TILEXR_FLAGS_PER_PAIR) * tile;
    if (capacity == 0) {
        TILEXR_LOG(ERROR) << "window too small: " << pairStride << " bytes per pair cannot hold a " << tile << " byte tile";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    g->tileBytes = tile;
    const uint64_t launchPair = std::min<uint64_t>(perPair, capacity);
    g->launches = static_cast<uint32_t>((perPair + launchPair - 1) / launchPair);
    g->bytesPerLaunch = twoShot ? launchPair * rankSize : launchPair;
    const uint32_t tiles = static_cast<uint32_t>((launchPair + tile - 1) / tile);

    // block roles
    // blocks per role: measured on NVLink 5, 16 blocks carry messages up to a few hundred KB at the lowest
    // latency, and 64 are needed from about 1 MB per pair to keep the links busy
    const uint32_t autoCap = launchPair >= (512u << 10) ? 64 : launchPair >= (128u << 10) ? 32 : 16;
    uint32_t cap = static_cast<uint32_t>(EnvLong("TILEXR_COLL_BLOCKS", autoCap));
    if (EnvLong("LCCL_PARALLEL", 0) == 1) cap = static_cast<uint32_t>(rankSize);
    const uint64_t fanItems = (kind == COLL_ALL_TO_ALL || kind == COLL_SCATTER) ? static_cast<uint64_t>(tiles) * rankSize
                              : (kind == COLL_REDUCE_SCATTER || twoShot) ? static_cast<uint64_t>(tiles) * (rankSize - 1)
                                                                        : tiles;
    uint32_t producers = static_cast<uint32_t>(std::min<uint64_t>(fanItems, cap));
    uint32_t reducers = 0;
    uint32_t consumers;
    if (kind == COLL_REDUCE_SCATTER || kind == COLL_ALL_REDUCE_ONE_SHOT) {
        consumers = std::min<uint32_t>(tiles, cap);
    } else if (twoShot) {
        reducers = std::min<uint32_t>(tiles, cap);
        consumers = static_cast<uint32_t>(std::min<uint64_t>(static_cast<uint64_t>(tiles) * (rankSize - 1), cap));
    } else {
        consumers = static_cast<uint32_t>(std::min<uint64_t>(static_cast<uint64_t>(tiles) * (rankSize - 1), cap));
    }
    producers = std::max(producers, 1u);
    consumers = std::max(consumers, 1u);
    // the grid must be co-resident
    while (maxGrid > 0 && producers + reducers + consumers > maxGrid) {
        if (producers >= consumers && producers >= reducers && producers > 1) --producers;
        else if (consumers >= reducers && consumers > 1) --consumers;
        else if (reducers > 1) --reducers;
        else break;
    }
    if (maxGrid > 0 && producers + reducers + consumers > maxGrid) return TILEXR_ERROR_NOT_SUPPORT;
    g->producers = producers;
    g->reducers = reducers;
    g->consumers = consumers;
    return TILEXR_SUCCESS;
}

struct CallContext {
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int rank = 0;
    int rankSize = 0;
    int device = 0;
};

int Prepare(TileXRCommPtr comm, CallContext *ctx)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    int ret = TileXRGetCommArgsHost(comm, &ctx->hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &ctx->devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (ctx->hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) {
        TILEXR_LOG(ERROR) << "host-memory communicators run the CPU collectives (tilexr_hostsim.h), not CUDA kernels";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    ctx->rank = ctx->hostArgs->rank;
    ctx->rankSize = ctx->hostArgs->rankSize;
    return TileXRCommGetInfo(comm, nullptr, nullptr, &ctx->device, nullptr);
}

int ValidateCommon(const void *send, const void *recv, int64_t count, int dtype, bool reduce, int op)
{
    if (send == nullptr || recv == nullptr) {
        TILEXR_LOG(ERROR) << "null buffer";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (count <= 0) {
        TILEXR_LOG(ERROR) << "count must be positive, got " << count;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (TileXRDataTypeSize(dtype) == 0 || (reduce && !IsReduceType(dtype))) {
        TILEXR_LOG(ERROR) << "unsupported data type " << dtype;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (reduce && (op < TILEXR_REDUCE_SUM || op > TILEXR_REDUCE_MIN)) {
        TILEXR_LOG(ERROR) << "unsupported reduce op " << op;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return TILEXR_SUCCESS;
}

const KernelEntry &KernelFor(int kind)
{
    switch (kind) {
        case COLL_REDUCE_SCATTER:
        case COLL_ALL_REDUCE_ONE_SHOT: return ReduceKernelEntry();
        case COLL_ALL_REDUCE_TWO_SHOT: return TwoShotKernelEntry();
        case COLL_PROFILE_PROBE: return ProbeKernelEntry();
        default: return PushKernelEntry();
    }
}

// Issues the launches of one collective call.  `sliceBytes`: bytes per pair (all-reduce
// kinds: bytes of the whole vector); `sliceStride`: distance of slices in the user buffers.
int Run(TileXRCommPtr comm, const CallContext &ctx, int kind, int opType, const uint8_t *in, uint8_t *out,
        uint64_t sliceBytes, uint64_t sliceStride, uint64_t outBytes, int dtype, int op, int root, TileXRStream stream,
        uint32_t burstBytes = 0, uint32_t pitchBytes = 0)
{
    const KernelEntry &kernel = KernelFor(kind);
    const int ranksPerDevice = (ctx.hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? ctx.rankSize : 1;
    unsigned maxGrid = 0;
    int ret = MaxCooperativeGrid(comm, kernel, COLL_BLOCK_THREADS, 0, ranksPerDevice, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    Geometry g;
    ret = Plan(kind, sliceBytes, ctx.rankSize, ctx.hostArgs->dataHalfBytes, maxGrid, &g);
    if (ret != TILEXR_SUCCESS) return ret;

    // zero-copy only makes sense where peers write final data: push kinds and two-shot
    TileXRUDMAMemHandle handle = 0;
    uint64_t regionOffset = 0;
    bool zeroCopy = false;
    if (kind == COLL_ALL_GATHER || kind == COLL_ALL_TO_ALL || kind == COLL_BROADCAST || kind == COLL_SCATTER ||
        kind == COLL_ALL_REDUCE_TWO_SHOT) {
        zeroCopy = EnvLong("TILEXR_COLL_ZERO_COPY", 1) != 0 &&
                   TileXRFindRegistration(comm, out, outBytes, &handle, &regionOffset) == TILEXR_SUCCESS;
    }

    const bool twoShot = kind == COLL_ALL_REDUCE_TWO_SHOT;
    uint64_t done = 0;
    const uint64_t total = sliceBytes;
    for (uint32_t l = 0; l < g.launches; ++l) {
        const uint64_t n = std::min<uint64_t>(g.bytesPerLaunch, total - done);
        CollArgs a;
        std::memset(&a, 0, sizeof(a));
        a.in = burstBytes != 0 ? in : in + done;   // a transposed all-to-all addresses its input by (row, column block)
        a.out = out + done;
        a.burstBytes = burstBytes;
        a.pitchBytes = pitchBytes;
        a.sliceBase = done;
        a.comm = reinterpret_cast<CommArgs *>(ctx.devArgs);
        a.kind = kind;
        a.opType = static_cast<uint32_t>(opType);
        a.root = root;
        a.dtype = dtype;
        a.reduceOp = op;
        a.elemSize = static_cast<uint32_t>(TileXRDataTypeSize(dtype));
        a.tileBytes = g.tileBytes;
        a.pairStride = g.pairStride;
        a.sliceStride = sliceStride;
        if (twoShot) {
            a.totalBytes = n;
            a.sliceBytes = RoundUp((n + ctx.rankSize - 1) / ctx.rankSize, 512);
        } else {
            a.totalBytes = n;
            a.sliceBytes = n;
        }
        a.tiles = static_cast<uint32_t>((a.sliceBytes + g.tileBytes - 1) / g.tileBytes);
        a.ringTiles = a.tiles;
        a.producers = g.producers;
        a.reducers = g.reducers;
        uint32_t grid = g.producers + g.reducers + g.consumers;
        if (kind == COLL_BROADCAST || kind == COLL_SCATTER) {
            // the root only pushes, the others only consume; keep the grid equal on all ranks
            a.producers = (ctx.rank == root) ? grid : 0;
        }
        a.zeroCopy = zeroCopy ? 1u : 0u;
        a.outHandle = handle;
        a.outOffset = regionOffset + done;
        int64_t magic = 0;
        ret = TileXRCommNextMagic(comm, &magic);
        if (ret != TILEXR_SUCCESS) return ret;
        a.magic = magic;
        PerfLaunchInfo info{static_cast<uint32_t>(opType), static_cast<uint32_t>(dtype), static_cast<uint32_t>(ctx.rank),
                            static_cast<uint32_t>(ctx.rankSize), grid, n};
        a.perfTrace = PerfTracePrepareLaunch(info, stream);
        LaunchConfig cfg{grid, COLL_BLOCK_THREADS, 0, true};
        ret = LaunchKernel(comm, kernel, &a, cfg, stream);
        if (ret != TILEXR_SUCCESS) return ret;
        done += n;
    }
    return TILEXR_SUCCESS;
}

int Loopback(void *dst, const void *src, uint64_t bytes, TileXRStream stream)
{
    if (dst == src) return TILEXR_SUCCESS;
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        TILEXR_LOG(ERROR) << "loopback copy failed: " << cudaGetErrorString(e);
        return TILEXR_ERROR_RUNTIME;
    }
    return TILEXR_SUCCESS;
}

} // namespace

extern "C" {

int TileXRCollectivePlan(int opType, int64_t count, int dataType, int rankSize, uint64_t dataHalfBytes, unsigned maxGrid,
                         TileXRCollPlanInfo *info)
{
    if (info == nullptr || count <= 0 || TileXRDataTypeSize(dataType) == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    uint64_t bytes = 0;
    if (MulOverflows(static_cast<uint64_t>(count), TileXRDataTypeSize(dataType), &bytes)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    int kind;
    switch (opType) {
        case TILEXR_OP_ALL_GATHER: kind = COLL_ALL_GATHER; break;
        case TILEXR_OP_ALL2ALL: kind = COLL_ALL_TO_ALL; break;
        case TILEXR_OP_BROADCAST: kind = COLL_BROADCAST; break;
        case TILEXR_OP_REDUCE_SCATTER: kind = COLL_REDUCE_SCATTER; break;
        case TILEXR_OP_ALL_REDUCE:
            kind = bytes <= OneShotMaxBytes() ? COLL_ALL_REDUCE_ONE_SHOT : COLL_ALL_REDUCE_TWO_SHOT;
            break;
        default: return TILEXR_ERROR_NOT_SUPPORT;
    }
    Geometry g;
    int ret = Plan(kind, bytes, rankSize, dataHalfBytes, maxGrid, &g);
    if (ret != TILEXR_SUCCESS) return ret;
    info->kind = g.kind;
    info->launches = g.launches;
    info->tileBytes = g.tileBytes;
    const uint64_t pair = kind == COLL_ALL_REDUCE_TWO_SHOT ? g.bytesPerLaunch / rankSize : g.bytesPerLaunch;
    info->tilesPerLaunch = static_cast<uint32_t>((pair + g.tileBytes - 1) / g.tileBytes);
    info->producers = g.producers;
    info->reducers = g.reducers;
    info->consumers = g.consumers;
    info->grid = g.producers + g.reducers + g.consumers;
    info->bytesPerLaunch = g.bytesPerLaunch;
    return TILEXR_SUCCESS;
}

int TileXRAllGather(void *sendBuf, void *recvBuf, int64_t sendCount, TileXRDataType dataType, TileXRCommPtr comm,
                    TileXRStream stream)
{
    CallContext ctx;
    int ret = Prepare(comm, &ctx);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = ValidateCommon(sendBuf, recvBuf, sendCount, dataType, false, 0);
    if (ret != TILEXR_SUCCESS) return ret;
    uint64_t bytes = 0, outBytes = 0;
    if (MulOverflows(static_cast<uint64_t>(sendCount), TileXRDataTypeSize(dataType), &bytes) ||
        MulOverflows(bytes, static_cast<uint64_t>(ctx.rankSize), &outBytes)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (ctx.rankSize == 1) return Loopback(recvBuf, sendBuf, bytes, stream);
    // A registered output takes the peers' stores directly; otherwise large shards go through the switch once
    // instead of R - 1 times.
    if (TileXRFindRegistration(comm, recvBuf, outBytes, nullptr, nullptr) != TILEXR_SUCCESS) {
        ret = NvlsWindowCollective(COLL_KIND_ALL_GATHER, sendBuf, recvBuf, sendCount, dataType, 0, 0, comm, stream);
        if (ret != TILEXR_ERROR_NOT_SUPPORT) return ret;
    }
    return Run(comm, ctx, COLL_ALL_GATHER, TILEXR_OP_ALL_GATHER, static_cast<const uint8_t *>(sendBuf),
               static_cast<uint8_t *>(recvBuf), bytes, bytes, outBytes, dataType, 0, 0, stream);
}

int TileXRAllToAll(void *sendBuf, void *recvBuf, int64_t sendCount, TileXRDataType dataType, TileXRCommPtr comm,
                   TileXRStream stream)
{
    CallContext ctx;
    int ret = Prepare(comm, &ctx);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = ValidateCommon(sendBuf, recvBuf, sendCount, dataType, false, 0);
    if (ret != TILEXR_SUCCESS) return ret;
    if (sendBuf == recvBuf) {
        TILEXR_LOG(ERROR) << "all-to-all cannot run in place";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    uint64_t bytes = 0, outBytes = 0;
    if (MulOverflows(static_cast<uint64_t>(sendCount), TileXRDataTypeSize(dataType), &bytes) ||
        MulOverflows(bytes, static_cast<uint64_t>(ctx.rankSize), &outBytes)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (ctx.rankSize == 1) return Loopback(recvBuf, sendBuf, bytes, stream);
    return Run(comm, ctx, COLL_ALL_TO_ALL, TILEXR_OP_ALL2ALL, static_cast<const uint8_t *>(sendBuf),
               static_cast<uint8_t *>(recvBuf), bytes, bytes, outBytes, dataType, 0, 0, stream);
}

// recvBuf[s][row][0:burst] = sendBuf of rank s [row][rank * burst : (rank + 1) * burst], burst = width / rankSize.
int TileXRAllToAllTranspose(void *sendBuf, void *recvBuf, int64_t count, int64_t width, TileXRDataType dataType, TileXRCommPtr comm,
                            TileXRStream stream)
{
    CallContext ctx;
    int ret = Prepare(comm, &ctx);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = ValidateCommon(sendBuf, recvBuf, count, dataType, false, 0);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t es = TileXRDataTypeSize(dataType);
    uint64_t bytes = 0;
    if (sendBuf == recvBuf || width <= 0 || count % width != 0 || width % ctx.rankSize != 0 ||
        MulOverflows(static_cast<uint64_t>(count), es, &bytes) || static_cast<uint64_t>(width) * es > 0xffffffffull) {
        TILEXR_LOG(ERROR) << "all-to-all transpose: count " << count << " must be rows x width, width " << width << " a multiple of the rank count";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const uint64_t burst = static_cast<uint64_t>(width) / ctx.rankSize * es;
    if (burst % 16 != 0 || reinterpret_cast<uintptr_t>(sendBuf) % 16 != 0) {
        TILEXR_LOG(ERROR) << "all-to-all transpose: a column block of " << burst << " bytes per row must be a multiple of 16";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (ctx.rankSize == 1) return Loopback(recvBuf, sendBuf, bytes, stream);
    const uint64_t slice = bytes / ctx.rankSize;
    return Run(comm, ctx, COLL_ALL_TO_ALL, TILEXR_OP_ALL2ALL, static_cast<const uint8_t *>(sendBuf), static_cast<uint8_t *>(recvBuf), slice,
               slice, bytes, dataType, 0, 0, stream, static_cast<uint32_t>(burst), static_cast<uint32_t>(static_cast<uint64_t>(width) * es));
}

int TileXRAllReduce(void *sendBuf, void *recvBuf, int64_t count, TileXRDataType dataType, TileXRReduceOp op,
                    TileXRCommPtr comm, TileXRStream stream)
{
    CallContext ctx;
    int ret = Prepare(comm, &ctx);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = ValidateCommon(sendBuf, recvBuf, count, dataType, true, op);
    if (ret != TILEXR_SUCCESS) return ret;
    uint64_t bytes = 0;
    if (MulOverflows(static_cast<uint64_t>(count), TileXRDataTypeSize(dataType), &bytes)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (ctx.rankSize == 1) return Loopback(recvBuf, sendBuf, bytes, stream);
    // the switch reduces each element once, at its owner, and all ranks receive the owner's bits
    ret = NvlsWindowCollective(COLL_KIND_ALL_REDUCE, sendBuf, recvBuf, count, dataType, op, 0, comm, stream);
    if (ret != TILEXR_ERROR_NOT_SUPPORT) return ret;
    const int kind = bytes <= OneShotMaxBytes() ? COLL_ALL_REDUCE_ONE_SHOT : COLL_ALL_REDUCE_TWO_SHOT;
    return Run(comm, ctx, kind, TILEXR_OP_ALL_REDUCE, static_cast<const uint8_t *>(sendBuf), static_cast<uint8_t *>(recvBuf),
               bytes, bytes, bytes, dataType, op, 0, stream);
}

int TileXRReduceScatter(void *sendBuf, void *recvBuf, int64_t recvCount, TileXRDataType dataType, TileXRReduceOp op,
                        TileXRCommPtr comm, TileXRStream stream)
{
    CallContext ctx;
    int ret = Prepare(comm, &ctx);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = ValidateCommon(sendBuf, recvBuf, recvCount, dataType, true, op);
    if (ret != TILEXR_SUCCESS) return ret;
    uint64_t bytes = 0;
    if (MulOverflows(static_cast<uint64_t>(recvCount), TileXRDataTypeSize(dataType), &bytes)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (ctx.rankSize == 1) return Loopback(recvBuf, sendBuf, bytes, stream);
    ret = NvlsWindowCollective(COLL_KIND_REDUCE_SCATTER, sendBuf, recvBuf, recvCount, dataType, op, 0, comm, stream);
    if (ret != TILEXR_ERROR_NOT_SUPPORT) return ret;
    return Run(comm, ctx, COLL_REDUCE_SCATTER, TILEXR_OP_REDUCE_SCATTER, static_cast<const uint8_t *>(sendBuf),
               static_cast<uint8_t *>(recvBuf), bytes, bytes, bytes, dataType, op, 0, stream);
}

int TileXRBroadcast(void *buf, int64_t count, TileXRDataType dataType, int root, TileXRCommPtr comm, TileXRStream stream)
{
    CallContext ctx;
    int ret = Prepare(comm, &ctx);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = ValidateCommon(buf, buf, count, dataType, false, 0);
    if (ret != TILEXR_SUCCESS) return ret;
    if (root < 0 || root >= ctx.rankSize) {
        TILEXR_LOG(ERROR) << "broadcast root " << root << " outside [0," << ctx.rankSize << ")";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    uint64_t bytes = 0;
    if (MulOverflows(static_cast<uint64_t>(count), TileXRDataTypeSize(dataType), &bytes)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (ctx.rankSize == 1) return TILEXR_SUCCESS;
    // one multicast store stream of the root reaches every rank
    ret = NvlsWindowCollective(COLL_KIND_BROADCAST, buf, buf, count, dataType, 0, root, comm, stream);
    if (ret != TILEXR_ERROR_NOT_SUPPORT) return ret;
    // Large messages on more than two ranks: the root scatters 1/R of the buffer to every rank and an in-place
    // all-gather completes it, so the root sends the buffer about twice instead of R-1 times.
    const uint64_t R = static_cast<uint64_t>(ctx.rankSize);
    if (ctx.rankSize > 2 && bytes >= static_cast<uint64_t>(EnvLong("TILEXR_BCAST_SCATTER_MIN_BYTES", 2 << 20)) && bytes % (R * 16) == 0) {
        const uint64_t slice = bytes / R;
        uint8_t *base = static_cast<uint8_t *>(buf);
        ret = Run(comm, ctx, COLL_SCATTER, TILEXR_OP_BROADCAST, base, base, slice, slice, bytes, dataType, 0, root, stream);
        if (ret != TILEXR_SUCCESS) return ret;
        return Run(comm, ctx, COLL_ALL_GATHER, TILEXR_OP_BROADCAST, base + static_cast<uint64_t>(ctx.rank) * slice, base, slice, slice,
                   bytes, dataType, 0, 0, stream);
    }
    return Run(comm, ctx, COLL_BROADCAST, TILEXR_OP_BROADCAST, static_cast<const uint8_t *>(buf), static_cast<uint8_t *>(buf),
               bytes, bytes, bytes, dataType, 0, root, stream);
}

int TileXRProfileProbe(void *sendBuf, void *recvBuf, int64_t count, TileXRDataType dataType, TileXRCommPtr comm,
                       TileXRStream stream)
{
    CallContext ctx;
    int ret = Prepare(comm, &ctx);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = ValidateCommon(sendBuf, recvBuf, count, dataType, false, 0);
    if (ret != TILEXR_SUCCESS) return ret;
    uint64_t bytes = 0;
    if (MulOverflows(static_cast<uint64_t>(count), TileXRDataTypeSize(dataType), &bytes)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    CollArgs a;
    std::memset(&a, 0, sizeof(a));
    a.in = static_cast<const uint8_t *>(sendBuf);
    a.out = static_cast<uint8_t *>(recvBuf);
    a.comm = reinterpret_cast<CommArgs *>(ctx.devArgs);
    a.kind = COLL_PROFILE_PROBE;
    a.opType = TILEXR_OP_PROFILE_PROBE;
    a.sliceBytes = bytes;
    a.dtype = dataType;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    const unsigned grid = 4;   // the reference's probe also runs on four cores
    PerfLaunchInfo info{TILEXR_OP_PROFILE_PROBE, static_cast<uint32_t>(dataType), static_cast<uint32_t>(ctx.rank),
                        static_cast<uint32_t>(ctx.rankSize), grid, bytes};
    a.perfTrace = PerfTracePrepareLaunch(info, stream);
    LaunchConfig cfg{grid, COLL_BLOCK_THREADS, 0, false};
    return LaunchKernel(comm, ProbeKernelEntry(), &a, cfg, stream);
}

} // extern "C"
