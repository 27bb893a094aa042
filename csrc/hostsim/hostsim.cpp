#include "tilexr_hostsim.h"

#include <algorithm>
#include <cstring>
#include <vector>

#include "device/tilexr_sync.cuh"
#include "tilexr_log.h"
#include "tilexr_types.h"

using namespace TileXR;
using namespace tilexr;

namespace {

bool g_skipFlags = false;

// Every copy into a window and every load out of one passes here, so that a protocol recorder (host_trace.cpp) sees
// them; the flag stores and waits report themselves from tilexr_sync.cuh.
void WindowStore(void *dst, const void *src, uint64_t bytes)
{
    if (HostTraceHooks *h = HostTraceSlot()) h->onCopy(h->ctx, dst, src, bytes);
    std::memcpy(dst, src, bytes);
}
void WindowLoad(void *dst, const void *src, uint64_t bytes)
{
    if (HostTraceHooks *h = HostTraceSlot()) h->onRead(h->ctx, src, bytes);
    std::memcpy(dst, src, bytes);
}
void WindowRead(const void *src, uint64_t bytes)
{
    if (HostTraceHooks *h = HostTraceSlot()) h->onRead(h->ctx, src, bytes);
}

struct HostCtx {
    CommArgs *args = nullptr;
    Waiter w;
    int rank = 0, R = 0;
    uint32_t epoch = 0;
};

int Begin(TileXRCommPtr comm, int op, int64_t count, HostCtx *c)
{
    TileXRCommArgs *args = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &args);
    if (ret != TILEXR_SUCCESS) return ret;
    if ((args->extraFlag & TILEXR_FLAG_HOST_MEMORY) == 0) {
        TILEXR_LOG(ERROR) << "host kernels need a host-memory communicator";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    c->args = args;
    c->rank = args->rank;
    c->R = args->rankSize;
    c->w = MakeWaiter(args, magic, 0);
    c->epoch = c->w.epoch;
    if (HostTraceHooks *h = HostTraceSlot()) h->epoch = c->epoch;
    args->dfx[TILEXR_DFX_MAGIC] = magic;
    args->dfx[TILEXR_DFX_OP] = op;
    args->dfx[TILEXR_DFX_COUNT_ARG] = count;
    args->dfx[TILEXR_DFX_RUN_STATUS] = TILEXR_RUN_STARTED;
    if (c->epoch >= 3) {
        for (int p = 0; p < c->R; ++p) {
            if (p != c->rank && !WaitPeerFinished(c->w, p, c->epoch - 2)) return TILEXR_ERROR_TIMEOUT;
        }
    }
    return TILEXR_SUCCESS;
}

int End(HostCtx &c)
{
    if (!g_skipFlags) PublishDone(c.w);
    g_skipFlags = false;
    if (c.w.ok()) {
        c.args->dfx[TILEXR_DFX_RUN_STATUS] = TILEXR_RUN_FINISHED;
        c.args->dfx[TILEXR_DFX_LAUNCHES] += 1;
        return TILEXR_SUCCESS;
    }
    return TILEXR_ERROR_TIMEOUT;
}

} // namespace

extern "C" {

int TileXRHostInjectSkipFlags(int enable)
{
    g_skipFlags = enable != 0;
    return TILEXR_SUCCESS;
}

int TileXRHostAllGather(const void *send, void *recv, uint64_t bytes, uint32_t tileBytes, TileXRCommPtr comm)
{
    if (send == nullptr || recv == nullptr || bytes == 0 || tileBytes == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_ALL_GATHER, static_cast<int64_t>(bytes), &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t pairStride = (c.args->dataHalfBytes / c.R) & ~255ull;
    const uint64_t tiles = (bytes + tileBytes - 1) / tileBytes;
    if (bytes > pairStride || tiles > TILEXR_FLAGS_PER_PAIR) {
        TILEXR_LOG(ERROR) << "host all-gather: " << bytes << " bytes per rank do not fit the window (" << pairStride
                          << " per pair, " << TILEXR_FLAGS_PER_PAIR << " tiles)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const uint8_t *in = static_cast<const uint8_t *>(send);
    uint8_t *out = static_cast<uint8_t *>(recv);
    // produce: tile by tile into every peer's window, flag after each tile
    for (uint64_t t = 0; t < tiles; ++t) {
        const uint64_t off = t * tileBytes;
        const uint64_t n = std::min<uint64_t>(tileBytes, bytes - off);
        for (int i = 1; i < c.R; ++i) {
            const int peer = (c.rank + i) % c.R;
            WindowStore(DataHalf(c.args, peer, c.epoch) + c.rank * pairStride + off, in + off, n);
            if (!g_skipFlags) {
                SetFlag(FlagSlot(c.args, peer, TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(c.rank) * TILEXR_FLAGS_PER_PAIR + t),
                        c.epoch, static_cast<uint32_t>(t + 1));
            }
        }
        std::memcpy(out + c.rank * bytes + off, in + off, n);
    }
    // consume
    for (uint64_t t = 0; t < tiles && c.w.ok(); ++t) {
        const uint64_t off = t * tileBytes;
        const uint64_t n = std::min<uint64_t>(tileBytes, bytes - off);
        for (int i = 1; i < c.R; ++i) {
            const int src = (c.rank + i) % c.R;
            const int64_t slot = TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(src) * TILEXR_FLAGS_PER_PAIR + t;
            if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), static_cast<uint32_t>(t + 1), src, slot)) break;
            WindowLoad(out + src * bytes + off, DataHalf(c.args, c.rank, c.epoch) + src * pairStride + off, n);
        }
    }
    return End(c);
}

int TileXRHostAllReduceSumF32(const float *send, float *recv, uint64_t count, TileXRCommPtr comm)
{
    if (send == nullptr || recv == nullptr || count == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_ALL_REDUCE, static_cast<int64_t>(count), &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t pairStride = (c.args->dataHalfBytes / c.R) & ~255ull;
    const uint64_t bytes = count * sizeof(float);
    if (bytes > pairStride) return TILEXR_ERROR_PARA_CHECK_FAIL;
    for (int i = 1; i < c.R; ++i) {
        const int peer = (c.rank + i) % c.R;
        WindowStore(DataHalf(c.args, peer, c.epoch) + c.rank * pairStride, send, bytes);
        if (!g_skipFlags) {
            SetFlag(FlagSlot(c.args, peer, TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(c.rank) * TILEXR_FLAGS_PER_PAIR), c.epoch, 1);
        }
    }
    for (int s = 0; s < c.R && c.w.ok(); ++s) {
        if (s == c.rank) continue;
        const int64_t slot = TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(s) * TILEXR_FLAGS_PER_PAIR;
        WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), 1, s, slot);
    }
    if (c.w.ok()) {
        for (int s = 0; s < c.R; ++s) {
            if (s != c.rank) WindowRead(DataHalf(c.args, c.rank, c.epoch) + s * pairStride, bytes);
        }
        // rank order 0..R-1, like the CUDA kernels
        for (uint64_t i = 0; i < count; ++i) {
            float acc = 0.f;
            for (int s = 0; s < c.R; ++s) {
                const float v = s == c.rank
                                    ? send[i]
                                    : reinterpret_cast<const float *>(DataHalf(c.args, c.rank, c.epoch) + s * pairStride)[i];
                acc = s == 0 ? v : acc + v;
            }
            recv[i] = acc;
        }
    }
    return End(c);
}

// Equal all-to-all: slice p of `send` goes to rank p and lands as slice `rank` of its `recv`, tile by tile behind flags.
int TileXRHostAllToAll(const void *send, void *recv, uint64_t bytesPerPeer, uint32_t tileBytes, TileXRCommPtr comm)
{
    if (send == nullptr || recv == nullptr || send == recv || bytesPerPeer == 0 || tileBytes == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_ALL2ALL, static_cast<int64_t>(bytesPerPeer), &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t pairStride = (c.args->dataHalfBytes / c.R) & ~255ull;
    const uint64_t tiles = (bytesPerPeer + tileBytes - 1) / tileBytes;
    if (bytesPerPeer > pairStride || tiles > TILEXR_FLAGS_PER_PAIR) return TILEXR_ERROR_PARA_CHECK_FAIL;
    const uint8_t *in = static_cast<const uint8_t *>(send);
    uint8_t *out = static_cast<uint8_t *>(recv);
    for (uint64_t t = 0; t < tiles; ++t) {
        const uint64_t off = t * tileBytes;
        const uint64_t n = std::min<uint64_t>(tileBytes, bytesPerPeer - off);
        for (int i = 1; i < c.R; ++i) {
            const int peer = (c.rank + i) % c.R;
            WindowStore(DataHalf(c.args, peer, c.epoch) + c.rank * pairStride + off, in + peer * bytesPerPeer + off, n);
            if (!g_skipFlags) {
                SetFlag(FlagSlot(c.args, peer, TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(c.rank) * TILEXR_FLAGS_PER_PAIR + t),
                        c.epoch, static_cast<uint32_t>(t + 1));
            }
        }
        std::memcpy(out + c.rank * bytesPerPeer + off, in + c.rank * bytesPerPeer + off, n);
    }
    for (uint64_t t = 0; t < tiles && c.w.ok(); ++t) {
        const uint64_t off = t * tileBytes;
        const uint64_t n = std::min<uint64_t>(tileBytes, bytesPerPeer - off);
        for (int i = 1; i < c.R; ++i) {
            const int src = (c.rank + i) % c.R;
            const int64_t slot = TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(src) * TILEXR_FLAGS_PER_PAIR + t;
            if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), static_cast<uint32_t>(t + 1), src, slot)) break;
            WindowLoad(out + src * bytesPerPeer + off, DataHalf(c.args, c.rank, c.epoch) + src * pairStride + off, n);
        }
    }
    return End(c);
}

// Reduce-scatter: slice p of every rank's `send` (recvCount floats) is summed on rank p in rank order.
int TileXRHostReduceScatterSumF32(const float *send, float *recv, uint64_t recvCount, TileXRCommPtr comm)
{
    if (send == nullptr || recv == nullptr || recvCount == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_REDUCE_SCATTER, static_cast<int64_t>(recvCount), &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t pairStride = (c.args->dataHalfBytes / c.R) & ~255ull;
    const uint64_t bytes = recvCount * sizeof(float);
    if (bytes > pairStride) return TILEXR_ERROR_PARA_CHECK_FAIL;
    for (int i = 1; i < c.R; ++i) {
        const int peer = (c.rank + i) % c.R;
        WindowStore(DataHalf(c.args, peer, c.epoch) + c.rank * pairStride, send + static_cast<uint64_t>(peer) * recvCount, bytes);
        if (!g_skipFlags) {
            SetFlag(FlagSlot(c.args, peer, TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(c.rank) * TILEXR_FLAGS_PER_PAIR), c.epoch, 1);
        }
    }
    for (int s = 0; s < c.R && c.w.ok(); ++s) {
        if (s == c.rank) continue;
        const int64_t slot = TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(s) * TILEXR_FLAGS_PER_PAIR;
        WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), 1, s, slot);
    }
    if (c.w.ok()) {
        for (int s = 0; s < c.R; ++s) {
            if (s != c.rank) WindowRead(DataHalf(c.args, c.rank, c.epoch) + s * pairStride, bytes);
        }
        for (uint64_t i = 0; i < recvCount; ++i) {
            float acc = 0.f;
            for (int s = 0; s < c.R; ++s) {
                const float v = s == c.rank ? send[static_cast<uint64_t>(c.rank) * recvCount + i]
                                            : reinterpret_cast<const float *>(DataHalf(c.args, c.rank, c.epoch) + s * pairStride)[i];
                acc = s == 0 ? v : acc + v;
            }
            recv[i] = acc;
        }
    }
    return End(c);
}

// Broadcast: the root pushes its buffer into every peer's window tile by tile; the others copy tiles out as their flags show up.
int TileXRHostBroadcast(void *buf, uint64_t bytes, int root, uint32_t tileBytes, TileXRCommPtr comm)
{
    if (buf == nullptr || bytes == 0 || tileBytes == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_BROADCAST, static_cast<int64_t>(bytes), &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t pairStride = (c.args->dataHalfBytes / c.R) & ~255ull;
    const uint64_t tiles = (bytes + tileBytes - 1) / tileBytes;
    if (root < 0 || root >= c.R || bytes > pairStride || tiles > TILEXR_FLAGS_PER_PAIR) return TILEXR_ERROR_PARA_CHECK_FAIL;
    uint8_t *data = static_cast<uint8_t *>(buf);
    for (uint64_t t = 0; t < tiles && c.w.ok(); ++t) {
        const uint64_t off = t * tileBytes;
        const uint64_t n = std::min<uint64_t>(tileBytes, bytes - off);
        const int64_t slot = TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(root) * TILEXR_FLAGS_PER_PAIR + t;
        if (c.rank == root) {
            for (int i = 1; i < c.R; ++i) {
                const int peer = (c.rank + i) % c.R;
                WindowStore(DataHalf(c.args, peer, c.epoch) + root * pairStride + off, data + off, n);
                if (!g_skipFlags) SetFlag(FlagSlot(c.args, peer, slot), c.epoch, static_cast<uint32_t>(t + 1));
            }
        } else {
            if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), static_cast<uint32_t>(t + 1), root, slot)) break;
            WindowLoad(data + off, DataHalf(c.args, c.rank, c.epoch) + root * pairStride + off, n);
        }
    }
    return End(c);
}

int TileXRHostEpDispatch(const float *x, const int32_t *expertIds, int64_t bs, int64_t h, int64_t topK,
                         int64_t moeExpertNum, int64_t maxRecvRows, float *expandXOut, int32_t *assistOut,
                         int64_t *expertTokenNumsOut, int32_t *sendCountsOut, int32_t *recvTotalOut, TileXRCommPtr comm)
{
    if (x == nullptr || expertIds == nullptr || expandXOut == nullptr || assistOut == nullptr ||
        expertTokenNumsOut == nullptr || sendCountsOut == nullptr || bs <= 0 || h <= 0 || topK <= 0 || moeExpertNum <= 0 ||
        maxRecvRows <= 0) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_EP_DISPATCH, bs, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    if (moeExpertNum % c.R != 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    const int E = static_cast<int>(moeExpertNum);
    const int perRank = E / c.R;
    const uint64_t rowBytes = static_cast<uint64_t>(h) * sizeof(float);
    const uint64_t payloadOff = 0;
    const uint64_t assistOff = (static_cast<uint64_t>(maxRecvRows) * rowBytes + 255) & ~255ull;
    const uint64_t countOff = (assistOff + static_cast<uint64_t>(maxRecvRows) * 16 + 255) & ~255ull;
    const uint64_t total = countOff + static_cast<uint64_t>(c.R) * E * 4;
    if (total > c.args->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "host EP dispatch needs " << total << " window bytes, have " << c.args->dataHalfBytes;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    // 1. count and rank my routes per expert in (token, k) order
    std::vector<int32_t> count(E, 0), pos(bs * topK, 0);
    for (int64_t i = 0; i < bs * topK; ++i) {
        const int e = expertIds[i];
        if (e >= 0 && e < E) pos[i] = count[e]++;
    }
    // 2. publish counts
    for (int i = 0; i < c.R; ++i) {
        const int peer = (c.rank + i) % c.R;
        WindowStore(DataHalf(c.args, peer, c.epoch) + countOff + static_cast<uint64_t>(c.rank) * E * 4, count.data(), E * 4);
        if (!g_skipFlags) {
            SetFlag(FlagSlot(c.args, peer, TILEXR_FLAG_OP_BASE + static_cast<int64_t>(c.rank) * TILEXR_FLAGS_PER_PAIR + TILEXR_FLAGS_PER_PAIR - 1),
                    c.epoch, 1);
        }
    }
    for (int s = 0; s < c.R; ++s) {
        const int64_t slot = TILEXR_FLAG_OP_BASE + static_cast<int64_t>(s) * TILEXR_FLAGS_PER_PAIR + TILEXR_FLAGS_PER_PAIR - 1;
        if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), 1, s, slot)) return End(c);
    }
    const int32_t *matrix = reinterpret_cast<const int32_t *>(DataHalf(c.args, c.rank, c.epoch) + countOff);
    WindowRead(matrix, static_cast<uint64_t>(c.R) * E * 4);
    std::vector<int64_t> tot(E, 0), dstRow(E, 0);
    for (int e = 0; e < E; ++e) {
        for (int s = 0; s < c.R; ++s) tot[e] += matrix[s * E + e];
    }
    for (int e = 0; e < E; ++e) {
        const int first = e / perRank * perRank;
        int64_t row = 0;
        for (int p = first; p < e; ++p) row += tot[p];
        for (int s = 0; s < c.rank; ++s) row += matrix[s * E + e];
        dstRow[e] = row;
    }
    for (int d = 0; d < c.R; ++d) {
        int64_t rows = 0;
        for (int e = d * perRank; e < (d + 1) * perRank; ++e) rows += tot[e];
        if (rows > maxRecvRows) {
            RaiseFailure(c.w, TILEXR_DEV_BAD_ARGUMENT, d, 0, static_cast<uint64_t>(maxRecvRows), static_cast<uint64_t>(rows));
            return End(c);
        }
    }
    // 3. send rows to their final position
    for (int64_t t = 0; t < bs; ++t) {
        for (int64_t k = 0; k < topK; ++k) {
            const int e = expertIds[t * topK + k];
            if (e < 0 || e >= E) continue;
            const int dst = e / perRank;
            const int64_t r = dstRow[e] + pos[t * topK + k];
            uint8_t *half = DataHalf(c.args, dst, c.epoch);
            WindowStore(half + payloadOff + r * rowBytes, x + t * h, rowBytes);
            const int32_t tuple[4] = {c.rank, static_cast<int32_t>(t), static_cast<int32_t>(k), e};
            WindowStore(half + assistOff + r * 16, tuple, 16);
        }
    }
    if (!g_skipFlags) {
        for (int d = 0; d < c.R; ++d) {
            SetFlag(FlagSlot(c.args, d, TILEXR_FLAG_OP_BASE + static_cast<int64_t>(c.rank) * TILEXR_FLAGS_PER_PAIR), c.epoch, 1);
        }
    }
    // 4. receive
    for (int s = 0; s < c.R; ++s) {
        const int64_t slot = TILEXR_FLAG_OP_BASE + static_cast<int64_t>(s) * TILEXR_FLAGS_PER_PAIR;
        if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), 1, s, slot)) return End(c);
    }
    int64_t rows = 0;
    int64_t running = 0;
    for (int le = 0; le < perRank; ++le) {
        const int e = c.rank * perRank + le;
        rows += tot[e];
        for (int s = 0; s < c.R; ++s) {
            running += matrix[s * E + e];
            sendCountsOut[le * c.R + s] = static_cast<int32_t>(running);
        }
        expertTokenNumsOut[le] = tot[e];
    }
    const uint8_t *half = DataHalf(c.args, c.rank, c.epoch);
    WindowLoad(expandXOut, half + payloadOff, rows * rowBytes);
    WindowLoad(assistOut, half + assistOff, rows * 16);
    if (recvTotalOut != nullptr) *recvTotalOut = static_cast<int32_t>(rows);
    return End(c);
}

int TileXRHostEpCombine(const float *expertOut, const int32_t *assist, int32_t rows, const int32_t *expertIds,
                        const float *expertScales, int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, float *yOut,
                        TileXRCommPtr comm)
{
    if (expertOut == nullptr || assist == nullptr || yOut == nullptr || rows < 0 || bs <= 0 || h <= 0 || topK <= 0) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_EP_COMBINE, bs, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t rowBytes = static_cast<uint64_t>(h) * sizeof(float);
    if (static_cast<uint64_t>(bs) * topK * rowBytes > c.args->dataHalfBytes || bs * topK > TILEXR_FLAG_SLOT_SLOTS) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    for (int32_t r = 0; r < rows; ++r) {
        const int src = assist[r * 4];
        const int64_t slot = static_cast<int64_t>(assist[r * 4 + 1]) * topK + assist[r * 4 + 2];
        if (src < 0 || src >= c.R || slot < 0 || slot >= bs * topK) continue;
        WindowStore(DataHalf(c.args, src, c.epoch) + slot * rowBytes, expertOut + static_cast<int64_t>(r) * h, rowBytes);
        if (!g_skipFlags) SetFlag(FlagSlot(c.args, src, TILEXR_FLAG_SLOT_BASE + slot), c.epoch, 1);
    }
    const uint8_t *half = DataHalf(c.args, c.rank, c.epoch);
    for (int64_t t = 0; t < bs && c.w.ok(); ++t) {
        float *y = yOut + t * h;
        std::fill(y, y + h, 0.f);
        for (int64_t k = 0; k < topK; ++k) {
            const int e = expertIds != nullptr ? expertIds[t * topK + k] : 0;
            if (e < 0 || e >= moeExpertNum) continue;
            const int64_t slot = t * topK + k;
            // the row comes from the rank that holds expert e
            const int producer = static_cast<int>(e / std::max<int64_t>(1, moeExpertNum / c.R));
            if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, TILEXR_FLAG_SLOT_BASE + slot), 1, producer, slot)) break;
            const float wgt = expertScales != nullptr ? expertScales[slot] : 1.0f;
            const float *row = reinterpret_cast<const float *>(half + slot * rowBytes);
            WindowRead(row, rowBytes);
            for (int64_t j = 0; j < h; ++j) y[j] = wgt * row[j] + y[j];
        }
    }
    return End(c);
}

// ---- MoonEP stages by plan (fp32 rows) ---------------------------------------------------------------------------------------
// dst[i] = r * nvS + row for route i of this rank (token i / topK), negative = the route sends nothing; dstLocal[row] >= 0 marks
// the rows of this rank that some route fills.  Rows and their route weights land in the destination's window; one flag per
// source says "all my rows for you are there"; filled rows are copied out, the others are zero.
int TileXRHostMoonDispatch(const float *hidden, const float *routeWeights, const int32_t *dst, const int32_t *dstLocal, int64_t routes,
                           int64_t topK, int64_t h, int64_t nvS, float *hiddenOut, float *weightsOut, TileXRCommPtr comm)
{
    if (hidden == nullptr || dst == nullptr || dstLocal == nullptr || hiddenOut == nullptr || routes <= 0 || topK <= 0 || h <= 0 || nvS <= 0) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if ((routeWeights == nullptr) != (weightsOut == nullptr)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_MOONEP_DISPATCH, routes, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const uint64_t rowBytes = static_cast<uint64_t>(h) * sizeof(float);
    const uint64_t weightOff = static_cast<uint64_t>(nvS) * rowBytes;
    if (weightOff + static_cast<uint64_t>(nvS) * sizeof(float) > c.args->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "host MoonEP dispatch needs " << weightOff + nvS * sizeof(float) << " window bytes, have " << c.args->dataHalfBytes;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    for (int64_t i = 0; i < routes && c.w.ok(); ++i) {
        const int32_t raw = dst[i];
        if (raw < 0) continue;
        const int dstRank = static_cast<int>(raw / nvS);
        const int64_t row = raw - static_cast<int64_t>(dstRank) * nvS;
        if (dstRank >= c.R) {
            RaiseFailure(c.w, TILEXR_DEV_BAD_ARGUMENT, c.rank, i, static_cast<uint64_t>(c.R), static_cast<uint64_t>(raw));
            return End(c);
        }
        uint8_t *half = DataHalf(c.args, dstRank, c.epoch);
        WindowStore(half + row * rowBytes, hidden + (i / topK) * h, rowBytes);
        if (routeWeights != nullptr) WindowStore(half + weightOff + row * sizeof(float), routeWeights + i, sizeof(float));
    }
    if (!g_skipFlags) {
        for (int p = 0; p < c.R; ++p) {
            SetFlag(FlagSlot(c.args, p, TILEXR_FLAG_OP_BASE + static_cast<int64_t>(c.rank) * TILEXR_FLAGS_PER_PAIR), c.epoch, 1);
        }
    }
    for (int s = 0; s < c.R; ++s) {
        const int64_t slot = TILEXR_FLAG_OP_BASE + static_cast<int64_t>(s) * TILEXR_FLAGS_PER_PAIR;
        if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, slot), 1, s, slot)) return End(c);
    }
    const uint8_t *half = DataHalf(c.args, c.rank, c.epoch);
    for (int64_t row = 0; row < nvS; ++row) {
        if (dstLocal[row] >= 0) {
            WindowLoad(hiddenOut + row * h, half + row * rowBytes, rowBytes);
            if (weightsOut != nullptr) WindowLoad(weightsOut + row, half + weightOff + row * sizeof(float), sizeof(float));
        } else {
            std::fill(hiddenOut + row * h, hiddenOut + (row + 1) * h, 0.f);
            if (weightsOut != nullptr) weightsOut[row] = 0.f;
        }
    }
    return End(c);
}

// Combine: dstLocal[row] = source rank * routesPerRank + route for the rows this rank holds (negative: padding).  Every row goes
// back to its source's window at its route's position behind a flag per route; the source adds a token's topK rows in route
// order in fp32.  Route weights travel back unchanged when given.
int TileXRHostMoonCombine(const float *rows, const float *weightsNvs, const int32_t *dstLocal, const int32_t *dst, int64_t nvS, int64_t tokens,
                          int64_t topK, int64_t h, float *hiddenOut, float *weightsOut, TileXRCommPtr comm)
{
    if (rows == nullptr || dstLocal == nullptr || dst == nullptr || hiddenOut == nullptr || nvS <= 0 || tokens <= 0 || topK <= 0 || h <= 0) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    HostCtx c;
    int ret = Begin(comm, TILEXR_OP_MOONEP_COMBINE, tokens, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const int64_t routes = tokens * topK;
    const uint64_t rowBytes = static_cast<uint64_t>(h) * sizeof(float);
    const uint64_t weightOff = static_cast<uint64_t>(routes) * rowBytes;
    if (weightOff + static_cast<uint64_t>(routes) * sizeof(float) > c.args->dataHalfBytes || routes > TILEXR_FLAG_SLOT_SLOTS) return TILEXR_ERROR_PARA_CHECK_FAIL;
    for (int64_t row = 0; row < nvS; ++row) {
        const int32_t v = dstLocal[row];
        if (v < 0) continue;
        const int src = static_cast<int>(v / routes);
        const int64_t route = v - static_cast<int64_t>(src) * routes;
        if (src >= c.R) continue;
        uint8_t *half = DataHalf(c.args, src, c.epoch);
        WindowStore(half + route * rowBytes, rows + row * h, rowBytes);
        if (weightsNvs != nullptr) WindowStore(half + weightOff + route * sizeof(float), weightsNvs + row, sizeof(float));
        if (!g_skipFlags) SetFlag(FlagSlot(c.args, src, TILEXR_FLAG_SLOT_BASE + route), c.epoch, 1);
    }
    const uint8_t *half = DataHalf(c.args, c.rank, c.epoch);
    for (int64_t t = 0; t < tokens && c.w.ok(); ++t) {
        float *y = hiddenOut + t * h;
        std::fill(y, y + h, 0.f);
        for (int64_t k = 0; k < topK; ++k) {
            const int64_t route = t * topK + k;
            const int32_t raw = dst[route];
            if (weightsOut != nullptr) weightsOut[route] = 0.f;
            if (raw < 0) continue;
            const int producer = static_cast<int>(raw / nvS);
            if (!WaitFlagGE(c.w, FlagSlot(c.args, c.rank, TILEXR_FLAG_SLOT_BASE + route), 1, producer, route)) break;
            const float *row = reinterpret_cast<const float *>(half + route * rowBytes);
            WindowRead(row, rowBytes);
            for (int64_t j = 0; j < h; ++j) y[j] += row[j];
            if (weightsOut != nullptr) weightsOut[route] = reinterpret_cast<const float *>(half + weightOff)[route];
        }
    }
    return End(c);
}

} // extern "C"
