// Host side of the expert-parallel library: shape validation, window layout, launch.
// Validation rules follow the reference's memory route (src/ep/host/ep_dispatch_memory_host.cpp:44-107,
// ep_memory_layout.cpp:67-306) where they still apply on this hardware.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include <cuda_runtime_api.h>

#include "ep_kernels.cuh"
#include "../collectives/perf_trace_session.h"
#include "tilexr_ep.h"
#include "tilexr_log.h"

using namespace TileXR;
using namespace TileXREp;

namespace {

uint64_t Align(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

long EnvLong(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

bool DispatchLayout(int64_t h, int64_t numExperts, int64_t rankSize, int64_t maxRecvRows, int64_t quantMode,
                    int64_t elemSize, int64_t grid, bool zeroCopy, EpDispatchWindow *win)
{
    if (h <= 0 || numExperts <= 0 || rankSize <= 0 || maxRecvRows <= 0 || grid <= 0) return false;
    const bool mx = quantMode == TILEXR_EP_QUANT_MXFP8_E4M3 || quantMode == TILEXR_EP_QUANT_MXFP8_E5M2;
    const bool int8 = quantMode == TILEXR_EP_QUANT_STATIC_INT8 || quantMode == TILEXR_EP_QUANT_DYNAMIC_INT8;
    const bool quant = mx || int8 || quantMode == TILEXR_EP_QUANT_FP8_1X128;
    win->rowBytes = static_cast<uint32_t>(quant ? h : h * elemSize);
    // fp32 scale per 128 elements, one E8M0 exponent byte per 32 elements, or one fp32 per row (in a 16-byte cell)
    win->scaleRowBytes = mx ? static_cast<uint32_t>(h / 32)
                         : quantMode == TILEXR_EP_QUANT_DYNAMIC_INT8 ? 16u
                         : quantMode == TILEXR_EP_QUANT_FP8_1X128 ? static_cast<uint32_t>(h / 128 * 4) : 0u;
    uint64_t off = 0;
    win->payloadOff = off;
    if (!zeroCopy) off = Align(off + static_cast<uint64_t>(maxRecvRows) * win->rowBytes, 256);
    win->scalesOff = off;
    off = Align(off + static_cast<uint64_t>(maxRecvRows) * win->scaleRowBytes, 256);
    win->assistOff = off;
    off = Align(off + static_cast<uint64_t>(maxRecvRows) * 16, 256);
    win->extOff = off;
    off = Align(off + static_cast<uint64_t>(maxRecvRows) * 8, 256);
    win->blockCountOff = off;
    off = Align(off + static_cast<uint64_t>(grid) * numExperts * 4, 256);
    win->totalBytes = off;
    return true;
}

// ep_tp.cu
}
namespace TileXR {
int EpTpExpand(const int32_t *ids, const float *weights, const uint8_t *routeMask, int64_t routes, int T, int experts, int perGroup,
               int32_t *idsOut, float *weightsOut, uint8_t *routeMaskOut, cudaStream_t stream);
int EpTpLaneCounts(const int32_t *sendCounts, int entries, int R, int T, int32_t *tpRecvCounts, cudaStream_t stream);
}
namespace {

struct Ctx {
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int rank = 0, rankSize = 0;
};

int Prepare(TileXRCommPtr comm, Ctx *c)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    int ret = TileXRGetCommArgsHost(comm, &c->hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &c->devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (c->hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_ERROR_NOT_SUPPORT;
    c->rank = c->hostArgs->rank;
    c->rankSize = c->hostArgs->rankSize;
    return TILEXR_SUCCESS;
}

// Fills `topo` and checks the expert placement: shared experts on the leading ranks, routed experts on the others.
int MakeTopology(int64_t moeExpertNum, int64_t topK, int rankSize, int64_t sharedExpertNum, int64_t sharedExpertRankNum, EpTopology *topo)
{
    if (sharedExpertNum < 0 || sharedExpertRankNum < 0 || (sharedExpertNum == 0) != (sharedExpertRankNum == 0)) {
        TILEXR_LOG(ERROR) << "EP: sharedExpertNum and sharedExpertRankNum must both be zero or both be positive";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (sharedExpertNum > 0 && (sharedExpertRankNum % sharedExpertNum != 0 || sharedExpertRankNum >= rankSize)) {
        TILEXR_LOG(ERROR) << "EP: sharedExpertRankNum must be a multiple of sharedExpertNum and leave ranks for the routed experts";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const int64_t moeRanks = rankSize - sharedExpertRankNum;
    if (moeExpertNum % moeRanks != 0) {
        TILEXR_LOG(ERROR) << "EP: " << moeExpertNum << " experts do not divide over " << moeRanks << " ranks";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (topK + sharedExpertNum > 32 || sharedExpertRankNum + moeExpertNum > EP_MAX_EXPERTS) {
        TILEXR_LOG(ERROR) << "EP: topK + sharedExpertNum <= 32 and sharedExpertRankNum + experts <= " << EP_MAX_EXPERTS << " required";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    topo->sharedRanks = static_cast<int32_t>(sharedExpertRankNum);
    topo->sharedExperts = static_cast<int32_t>(sharedExpertNum);
    topo->moePerRank = static_cast<int32_t>(moeExpertNum / moeRanks);
    return TILEXR_SUCCESS;
}

int ValidateShape(int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, int rankSize, int dtype)
{
    if (dtype != TILEXR_DATA_TYPE_FP16 && dtype != TILEXR_DATA_TYPE_BFP16) {
        TILEXR_LOG(ERROR) << "EP: x must be fp16 or bf16";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (bs <= 0 || h <= 0 || topK <= 0 || moeExpertNum <= 0) {
        TILEXR_LOG(ERROR) << "EP: bs, h, topK and moeExpertNum must be positive";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (topK > EP_MAX_TOPK || topK > moeExpertNum || moeExpertNum > EP_MAX_EXPERTS) {
        TILEXR_LOG(ERROR) << "EP: topK <= " << EP_MAX_TOPK << ", topK <= experts <= " << EP_MAX_EXPERTS << " required";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    (void)rankSize;
    if ((h * 2) % 16 != 0) {
        TILEXR_LOG(ERROR) << "EP: hidden size must be a multiple of 8 elements";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (bs * 32 > TILEXR_FLAG_SLOT_SLOTS && bs * topK > TILEXR_FLAG_SLOT_SLOTS) {
        TILEXR_LOG(ERROR) << "EP: bs*topK exceeds the " << TILEXR_FLAG_SLOT_SLOTS << " slot flags of a window";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return TILEXR_SUCCESS;
}

// ---- tensor parallelism inside expert parallelism: see ep_tp.cu ---------------------------------------------------

struct TpStaging {
    int32_t *ids = nullptr;
    float *weights = nullptr;
    uint8_t *mask = nullptr;
};

int ValidateTp(const Ctx &c, int64_t tpWorldSize, int64_t tpRankId, int64_t topK, int64_t moeExpertNum, int64_t sharedExpertRankNum,
               const char *what)
{
    const int64_t T = tpWorldSize;
    if (T > c.rankSize || c.rankSize % T != 0 || tpRankId != c.rank % T) {
        TILEXR_LOG(ERROR) << what << ": tpWorldSize " << T << " must divide the " << c.rankSize << " ranks and tpRankId must be rank % tpWorldSize";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const int64_t groups = c.rankSize / T;
    if (sharedExpertRankNum != 0 || topK * T > EP_MAX_TOPK || moeExpertNum % groups != 0 || moeExpertNum * T > EP_MAX_EXPERTS) {
        TILEXR_LOG(ERROR) << what << " with tensor parallelism: no shared-expert ranks, topK * tpWorldSize <= " << EP_MAX_TOPK
                          << ", experts divisible by the " << groups << " groups, experts * tpWorldSize <= " << EP_MAX_EXPERTS;
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    return TILEXR_SUCCESS;
}

// Carves the widened per-route arrays out of the communicator's scratch buffer (dispatch uses its first half, combine
// the second, so a combine queued behind a dispatch on another stream does not overwrite what that dispatch reads).
int StageTp(TileXRCommPtr comm, bool forCombine, int64_t routes, int T, bool ids, bool weights, bool mask, TpStaging *out)
{
    const uint64_t wide = static_cast<uint64_t>(routes) * T;
    const uint64_t half = Align(wide * 4, 256) * 2 + Align(wide, 256);
    void *base = nullptr;
    const int ret = TileXRGetOperatorScratch(comm, 2 * half, &base);
    if (ret != TILEXR_SUCCESS) return ret;
    uint8_t *p = static_cast<uint8_t *>(base) + (forCombine ? half : 0);
    if (ids) out->ids = reinterpret_cast<int32_t *>(p);
    if (weights) out->weights = reinterpret_cast<float *>(p + Align(wide * 4, 256));
    if (mask) out->mask = p + 2 * Align(wide * 4, 256);
    return TILEXR_SUCCESS;
}

int DispatchWithTp(const TileXREpDispatchParams *p, TileXRCommPtr comm, TileXRStream stream, const Ctx &c)
{
    const int T = static_cast<int>(p->tpWorldSize);
    if (p->tpRecvCountsOut == nullptr || p->expertIds == nullptr || p->gateLogits != nullptr) {
        TILEXR_LOG(ERROR) << "EP dispatch with tensor parallelism needs tpRecvCountsOut and explicit expertIds (no fused routing)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    int ret = ValidateTp(c, p->tpWorldSize, p->tpRankId, p->topK, p->moeExpertNum, p->sharedExpertRankNum, "EP dispatch");
    if (ret != TILEXR_SUCCESS) return ret;
    const int groups = c.rankSize / T;
    const int perGroup = static_cast<int>(p->moeExpertNum / groups);
    const bool routeMask = p->xActiveMask != nullptr && p->activeMaskType == TILEXR_EP_ACTIVE_MASK_EXPERT;
    TpStaging st;
    ret = StageTp(comm, false, p->bs * p->topK, T, true, p->expertScales != nullptr, routeMask, &st);
    if (ret != TILEXR_SUCCESS) return ret;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (EpTpExpand(p->expertIds, p->expertScales, routeMask ? reinterpret_cast<const uint8_t *>(p->xActiveMask) : nullptr, p->bs * p->topK, T,
                   static_cast<int>(p->moeExpertNum), perGroup, st.ids, st.weights, st.mask, cs) != 0) {
        return TILEXR_ERROR_RUNTIME;
    }
    TileXREpDispatchParams q = *p;
    q.tpWorldSize = 1;
    q.tpRankId = 0;
    q.tpRecvCountsOut = nullptr;
    q.topK = p->topK * T;
    q.moeExpertNum = p->moeExpertNum * T;
    q.expertIds = st.ids;
    if (st.weights != nullptr) q.expertScales = st.weights;
    if (routeMask) q.xActiveMask = reinterpret_cast<const bool *>(st.mask);
    q.topkIdsOut = nullptr;           // [bs, topK] buffers of the caller: the kernel would write topK * T columns
    q.topkWeightsOut = nullptr;
    ret = TileXRMoeEpDispatchFused(&q, comm, stream);
    if (ret != TILEXR_SUCCESS) return ret;
    const int32_t *sendCounts = p->sendCountsOut;
    int32_t *laneCounts = p->tpRecvCountsOut;
    const int entries = perGroup * c.rankSize, R = c.rankSize;
    return RunAfterLaunch(comm, [=]() { return EpTpLaneCounts(sendCounts, entries, R, T, laneCounts, cs) == 0 ? TILEXR_SUCCESS : TILEXR_ERROR_RUNTIME; });
}

int CombineWithTp(const TileXREpCombineParams *p, TileXRCommPtr comm, TileXRStream stream, const Ctx &c)
{
    const int T = static_cast<int>(p->tpWorldSize);
    int ret = ValidateTp(c, p->tpWorldSize, p->tpRankId, p->topK, p->moeExpertNum, p->sharedExpertRankNum, "EP combine");
    if (ret != TILEXR_SUCCESS) return ret;
    const int groups = c.rankSize / T;
    const int perGroup = static_cast<int>(p->moeExpertNum / groups);
    const bool routeMask = p->xActiveMask != nullptr && p->activeMaskType == TILEXR_EP_ACTIVE_MASK_EXPERT;
    TpStaging st;
    ret = StageTp(comm, true, p->bs * p->topK, T, p->expertIds != nullptr, p->expertScales != nullptr, routeMask, &st);
    if (ret != TILEXR_SUCCESS) return ret;
    if (st.ids != nullptr || st.weights != nullptr || st.mask != nullptr) {
        if (EpTpExpand(p->expertIds, p->expertScales, routeMask ? reinterpret_cast<const uint8_t *>(p->xActiveMask) : nullptr,
                       p->bs * p->topK, T, static_cast<int>(p->moeExpertNum), perGroup, st.ids, st.weights, st.mask,
                       static_cast<cudaStream_t>(stream)) != 0) {
            return TILEXR_ERROR_RUNTIME;
        }
    }
    TileXREpCombineParams q = *p;
    q.tpWorldSize = 1;
    q.tpRankId = 0;
    q.topK = p->topK * T;
    q.moeExpertNum = p->moeExpertNum * T;
    if (st.ids != nullptr) q.expertIds = st.ids;
    if (st.weights != nullptr) q.expertScales = st.weights;
    if (routeMask) q.xActiveMask = reinterpret_cast<const bool *>(st.mask);
    return TileXRMoeEpCombineFused(&q, comm, stream);
}

} // namespace

extern "C" {

uint64_t TileXREpDispatchWindowBytes(int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, int64_t rankSize,
                                     int64_t maxRecvRows, int64_t quantMode, int64_t elemSize, int64_t grid, int zeroCopy)
{
    (void)bs;
    (void)topK;
    EpDispatchWindow win;
    if (!DispatchLayout(h, moeExpertNum, rankSize, maxRecvRows, quantMode, elemSize, grid, zeroCopy != 0, &win)) return 0;
    return win.totalBytes;
}

uint64_t TileXREpCombineWindowBytes(int64_t bs, int64_t h, int64_t topK, int64_t elemSize)
{
    if (bs <= 0 || h <= 0 || topK <= 0 || elemSize <= 0) return 0;
    return static_cast<uint64_t>(bs) * topK * h * elemSize;
}

uint64_t TileXREpAbiStamp(void) { return TILEXR_EP_ABI_STAMP; }

int TileXRMoeEpDispatchFused(const TileXREpDispatchParams *p, TileXRCommPtr comm, TileXRStream stream)
{
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    if (p == nullptr || p->x == nullptr || p->expandXOut == nullptr || p->assistInfoForCombineOut == nullptr ||
        p->expertTokenNumsOut == nullptr || p->sendCountsOut == nullptr) {
        TILEXR_LOG(ERROR) << "EP dispatch: null tensor";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (p->tpWorldSize > 1) return DispatchWithTp(p, comm, stream, c);
    if ((p->expertIds == nullptr) == (p->gateLogits == nullptr)) {
        TILEXR_LOG(ERROR) << "EP dispatch: give either expertIds or gateLogits";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (p->gateLogits != nullptr && (p->topkIdsOut == nullptr || p->topkWeightsOut == nullptr)) {
        TILEXR_LOG(ERROR) << "EP dispatch: fused routing needs topkIdsOut and topkWeightsOut";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    ret = ValidateShape(p->bs, p->h, p->topK, p->moeExpertNum, c.rankSize, p->dtype);
    if (ret != TILEXR_SUCCESS) return ret;
    EpTopology topo;
    ret = MakeTopology(p->moeExpertNum, p->topK, c.rankSize, p->sharedExpertNum, p->sharedExpertRankNum, &topo);
    if (ret != TILEXR_SUCCESS) return ret;
    const int64_t numCols = topo.sharedRanks + p->moeExpertNum;
    const int64_t routesPerToken = p->topK + topo.sharedExperts;
    const int64_t smemCols = std::max<int64_t>(numCols, static_cast<int64_t>(topo.moePerRank) * c.rankSize);
    if (static_cast<int64_t>(c.rankSize) * ((numCols + 3) / 3) * 16 > TILEXR_WIN_LL_HALF_BYTES) {
        TILEXR_LOG(ERROR) << "EP: the count vectors of " << c.rankSize << " ranks x " << numCols << " columns exceed the low-latency plane";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (p->bs * routesPerToken > TILEXR_FLAG_SLOT_SLOTS) {
        TILEXR_LOG(ERROR) << "EP: bs * (topK + sharedExpertNum) exceeds the " << TILEXR_FLAG_SLOT_SLOTS << " slot flags of a window";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const bool fp8Mode = p->quantMode == TILEXR_EP_QUANT_FP8_1X128 || p->quantMode == TILEXR_EP_QUANT_MXFP8_E4M3 ||
                         p->quantMode == TILEXR_EP_QUANT_MXFP8_E5M2;
    const bool int8Mode = p->quantMode == TILEXR_EP_QUANT_STATIC_INT8 || p->quantMode == TILEXR_EP_QUANT_DYNAMIC_INT8;
    if (p->quantMode != TILEXR_EP_QUANT_NONE && !fp8Mode && !int8Mode) {
        TILEXR_LOG(ERROR) << "EP dispatch: unknown quantMode " << p->quantMode;
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    if (int8Mode) {
        if (p->h % 16 != 0 || (p->quantMode == TILEXR_EP_QUANT_STATIC_INT8 && p->scales == nullptr) ||
            (p->quantMode == TILEXR_EP_QUANT_DYNAMIC_INT8 && p->dynamicScalesOut == nullptr)) {
            TILEXR_LOG(ERROR) << "EP dispatch: int8 modes need h % 16 == 0; static needs scales, dynamic needs dynamicScalesOut";
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
    }
    if (fp8Mode) {
        if (p->dynamicScalesOut == nullptr || p->h % 512 != 0 || p->h > EP_FP8_MAX_H) {
            TILEXR_LOG(ERROR) << "EP dispatch: fp8 mode needs dynamicScalesOut and h a multiple of 512 up to " << EP_FP8_MAX_H;
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
    }
    if (p->activeMaskType != TILEXR_EP_ACTIVE_MASK_NONE && p->xActiveMask == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (p->activeMaskType < 0 || p->activeMaskType > TILEXR_EP_ACTIVE_MASK_EXPERT) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (p->maxRecvRows <= 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (p->dedup != 0 && (p->assistExtOut == nullptr || (p->gateLogits == nullptr && p->expertScales == nullptr))) {
        TILEXR_LOG(ERROR) << "EP dispatch: dedup needs assistExtOut and gate weights (fused routing or expertScales)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }

    // grid: one block per ~8 tokens per warp-set, capped by what can be co-resident
    const int ranksPerDevice = (c.hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? c.rankSize : 1;
    // At least minBlocks blocks even for a handful of tokens: the receive side of the kernel (rows from all
    // ranks) and the column split of the send side both want the parallelism; blocks may own no token.
    const int64_t capBlocks = std::min<int64_t>(EP_COUNT_FLAG_SLOT - 1, std::max<int64_t>(1, EnvLong("TILEXR_EP_BLOCKS", 296)));
    const int64_t minBlocks = std::min<int64_t>(capBlocks, std::max<int64_t>(1, EnvLong("TILEXR_EP_MIN_BLOCKS", 32)));
    const int64_t wantBlocks = std::max<int64_t>(minBlocks, std::min<int64_t>((p->bs + 15) / 16, capBlocks));
    unsigned grid = static_cast<unsigned>(wantBlocks);
    unsigned gridCap = 0;
    uint32_t tokensPerBlock = 0;
    size_t smem = 0;
    for (;;) {
        tokensPerBlock = static_cast<uint32_t>((p->bs + grid - 1) / grid);
        if (static_cast<int64_t>(tokensPerBlock) * routesPerToken > EP_MAX_ROUTES_PER_BLOCK) {
            TILEXR_LOG(ERROR) << "EP dispatch: " << tokensPerBlock << " tokens per block exceed the per-block route table; "
                              << "raise TILEXR_EP_BLOCKS";
            return TILEXR_ERROR_NOT_SUPPORT;
        }
        smem = EpDispatchSmemBytes(static_cast<int>(smemCols), static_cast<int>(tokensPerBlock * routesPerToken));
        unsigned maxGrid = 0;
        ret = MaxCooperativeGrid(comm, EpDispatchKernelEntry(), EP_BLOCK_THREADS, smem, ranksPerDevice, &maxGrid);
        if (ret != TILEXR_SUCCESS) return ret;
        if (maxGrid == 0) return TILEXR_ERROR_NOT_SUPPORT;
        gridCap = maxGrid;
        if (grid <= maxGrid) break;
        grid = maxGrid;
    }
    grid = static_cast<unsigned>(std::max<int64_t>((p->bs + tokensPerBlock - 1) / tokensPerBlock, std::min<int64_t>(minBlocks, gridCap)));

    const size_t elemSize = TileXRDataTypeSize(p->dtype);
    const bool quant = fp8Mode || int8Mode;
    const uint64_t outBytes = static_cast<uint64_t>(p->maxRecvRows) * (quant ? p->h : p->h * elemSize);
    TileXRUDMAMemHandle handle = 0;
    uint64_t regionOffset = 0;
    const bool zeroCopy = EnvLong("TILEXR_EP_ZERO_COPY", 1) != 0 &&
                          TileXRFindRegistration(comm, p->expandXOut, outBytes, &handle, &regionOffset) == TILEXR_SUCCESS;

    EpDispatchArgs a;
    std::memset(&a, 0, sizeof(a));
    if (!DispatchLayout(p->h, numCols, c.rankSize, p->maxRecvRows, p->quantMode, elemSize, grid, zeroCopy, &a.win)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (a.win.totalBytes > c.hostArgs->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "EP dispatch needs " << a.win.totalBytes << " bytes of window per half, the communicator has "
                          << c.hostArgs->dataHalfBytes << "; create it with a larger buffer or register expandXOut";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    a.x = static_cast<const uint8_t *>(p->x);
    a.expertIds = p->expertIds;
    a.gateLogits = p->gateLogits;
    a.selectionBias = p->selectionBias;
    a.activeMask = reinterpret_cast<const uint8_t *>(p->xActiveMask);
    a.topkIdsOut = p->topkIdsOut;
    a.topkWeightsOut = p->topkWeightsOut;
    a.expandXOut = static_cast<uint8_t *>(p->expandXOut);
    a.dynamicScalesOut = p->dynamicScalesOut;
    a.assistOut = p->assistInfoForCombineOut;
    a.expertTokenNumsOut = p->expertTokenNumsOut;
    a.sendCountsOut = p->sendCountsOut;
    a.recvTotalOut = p->recvTotalOut;
    a.comm = reinterpret_cast<CommArgs *>(c.devArgs);
    a.bs = static_cast<int32_t>(p->bs);
    a.h = static_cast<int32_t>(p->h);
    a.topK = static_cast<int32_t>(p->topK);
    a.numExperts = static_cast<int32_t>(p->moeExpertNum);
    a.numCols = static_cast<int32_t>(numCols);
    a.topo = topo;
    a.maskType = static_cast<int32_t>(p->activeMaskType);
    a.quantMode = static_cast<int32_t>(p->quantMode);
    a.scoreFunc = static_cast<int32_t>(p->scoreFunc);
    a.renormalize = static_cast<int32_t>(p->renormalize);
    a.tokenNumsType = static_cast<int32_t>(p->expertTokenNumsType);
    a.routedScale = p->routedScalingFactor == 0.f ? 1.0f : p->routedScalingFactor;
    a.maxRecvRows = static_cast<uint32_t>(p->maxRecvRows);
    a.tokensPerBlock = tokensPerBlock;
    a.elemSize = static_cast<uint32_t>(elemSize);
    a.isBf16 = p->dtype == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
    a.zeroCopy = zeroCopy ? 1u : 0u;
    a.outHandle = handle;
    a.outOffset = regionOffset;
    a.routeRowsOut = p->routeRowsOut;
    a.expertScales = p->expertScales;
    a.expandScalesOut = p->expandScalesOut;
    a.assistExtOut = p->assistExtOut;
    a.quantScales = int8Mode ? p->scales : nullptr;
    // per-expert smoothing makes the rows of one token differ from expert to expert: nothing to share
    a.dedup = (p->dedup != 0 && c.rankSize > 1 && a.quantScales == nullptr) ? 1u : 0u;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    {
        PerfLaunchInfo info{static_cast<uint32_t>(TILEXR_OP_EP_DISPATCH), static_cast<uint32_t>(p->dtype),
                            static_cast<uint32_t>(c.rank), static_cast<uint32_t>(c.rankSize), grid,
                            static_cast<uint64_t>(p->bs) * p->h * elemSize};
        a.perfTrace = PerfTracePrepareLaunch(info, stream);
    }
    LaunchConfig cfg{grid, EP_BLOCK_THREADS, smem, true};
    return LaunchKernel(comm, EpDispatchKernelEntry(), &a, cfg, stream);
}

int TileXRMoeEpCombineFused(const TileXREpCombineParams *p, TileXRCommPtr comm, TileXRStream stream)
{
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    if (p == nullptr || p->expertOut == nullptr || p->assistInfoForCombine == nullptr || p->sendCounts == nullptr ||
        p->yOut == nullptr) {
        TILEXR_LOG(ERROR) << "EP combine: null tensor";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (p->tpWorldSize > 1) return CombineWithTp(p, comm, stream, c);
    ret = ValidateShape(p->bs, p->h, p->topK, p->moeExpertNum, c.rankSize, p->dtype);
    if (ret != TILEXR_SUCCESS) return ret;
    if (p->activeMaskType != TILEXR_EP_ACTIVE_MASK_NONE && p->xActiveMask == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    EpTopology topo;
    ret = MakeTopology(p->moeExpertNum, p->topK, c.rankSize, p->sharedExpertNum, p->sharedExpertRankNum, &topo);
    if (ret != TILEXR_SUCCESS) return ret;
    const int64_t slotsPerToken = p->topK + topo.sharedExperts;
    if (p->bs * slotsPerToken > TILEXR_FLAG_SLOT_SLOTS) return TILEXR_ERROR_PARA_CHECK_FAIL;
    const uint64_t need = TileXREpCombineWindowBytes(p->bs, p->h, slotsPerToken, 2);
    if (need > c.hostArgs->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "EP combine needs " << need << " bytes of window per half, the communicator has "
                          << c.hostArgs->dataHalfBytes;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    EpCombineArgs a;
    std::memset(&a, 0, sizeof(a));
    a.expertOut = static_cast<const uint8_t *>(p->expertOut);
    a.assist = p->assistInfoForCombine;
    a.sendCounts = p->sendCounts;
    a.expertIds = p->expertIds;
    a.expertScales = p->expertScales;
    a.activeMask = reinterpret_cast<const uint8_t *>(p->xActiveMask);
    a.sharedExpertX = static_cast<const uint8_t *>(p->sharedExpertX);
    a.yOut = static_cast<uint8_t *>(p->yOut);
    a.comm = reinterpret_cast<CommArgs *>(c.devArgs);
    a.bs = static_cast<int32_t>(p->bs);
    a.h = static_cast<int32_t>(p->h);
    a.topK = static_cast<int32_t>(p->topK);
    a.numExperts = static_cast<int32_t>(p->moeExpertNum);
    a.numCols = static_cast<int32_t>(topo.sharedRanks + p->moeExpertNum);
    a.topo = topo;
    a.maskType = static_cast<int32_t>(p->activeMaskType);
    a.rowBytes = static_cast<uint32_t>(p->h * 2);
    a.isBf16 = p->dtype == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
    a.sendCountEntries = static_cast<uint32_t>(EpRankCols(topo, c.rank) * c.rankSize);
    a.routeRows = p->expertIds != nullptr ? p->routeRows : nullptr;
    a.dedup = (p->dedup != 0 && c.rankSize > 1) ? 1u : 0u;
    a.assistExt = p->assistExt;
    if (a.dedup != 0 && (p->assistExt == nullptr || p->expertIds == nullptr)) {
        TILEXR_LOG(ERROR) << "EP combine: dedup needs assistExt from dispatch and expertIds";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    const int ranksPerDevice = (c.hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? c.rankSize : 1;
    unsigned maxGrid = 0;
    ret = MaxCooperativeGrid(comm, EpCombineKernelEntry(), EP_BLOCK_THREADS, 0, ranksPerDevice, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    const int64_t minBlocks = std::max<int64_t>(1, EnvLong("TILEXR_EP_MIN_BLOCKS", 32));
    const int64_t want = std::min<int64_t>(EnvLong("TILEXR_EP_BLOCKS", 296),
                                           std::max<int64_t>(minBlocks, (p->bs * slotsPerToken + 15) / 16));
    const unsigned grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(want, maxGrid)));
    // Work decomposition.  It depends on bs, topK, h and the grid cap only, so every rank derives the same one
    // (bs is the same on all ranks: the slot numbering of the windows relies on it already).
    {
        const int64_t warps = static_cast<int64_t>(want) * EP_WARPS;      // `want`, not `grid`: ranks may get different caps
        const int64_t routes = p->bs * slotsPerToken;
        const int64_t rowVecs = a.rowBytes / 16;
        // The rows that travel, estimated for uniform routing (one row per token and remote rank with dedup).
        double travel = static_cast<double>(routes) * (c.rankSize - 1) / c.rankSize;
        if (a.dedup != 0) {
            double miss = 1.0;
            for (int64_t k = 0; k < slotsPerToken; ++k) miss *= 1.0 - 1.0 / c.rankSize;
            travel = static_cast<double>(p->bs) * (c.rankSize - 1) * (1.0 - miss);
        }
        // one rank that knows the row of each of its own routes: nothing travels
        a.noSend = (c.rankSize == 1 && a.routeRows != nullptr && a.expertIds != nullptr) ? 1u : 0u;
        // Column parts: a warp should get through about eight send items in a row, so that rows leave in the
        // order of the queue (the reducers follow that order) instead of all at once; small batches are cut up
        // so that every warp has something to do.
        int64_t parts;
        if (a.noSend != 0) {
            parts = std::min<int64_t>(8, std::max<int64_t>(1, (4 * warps + routes - 1) / routes));
        } else {
            parts = static_cast<int64_t>(std::min(8.0, std::max(1.0, std::ceil(8.0 * warps / std::max(1.0, travel)))));
        }
        parts = std::min<int64_t>(parts, std::max<int64_t>(1, rowVecs / 32));
        parts = std::min<int64_t>(parts, std::max<int64_t>(1, TILEXR_FLAG_SLOT_SLOTS / routes));
        const int64_t partVecs = ((rowVecs + parts - 1) / parts + 31) / 32 * 32;
        parts = (rowVecs + partVecs - 1) / partVecs;                       // no empty part
        a.parts = static_cast<uint32_t>(parts);
        a.partVecs = static_cast<uint32_t>(partVecs);
        const bool overlap = c.rankSize > 1 && routes >= 8192 && grid >= 16;
        // Blocks that only reduce.  The senders are bound by the link (about 550 GB/s per GPU in an all-to-all of
        // eight) or by the rows they read and write; the reducers must keep up with what arrives.  With T the
        // time of the slower of the two, a share reduceTime / T of the blocks, plus a margin, reduces.
        const double sendRows = static_cast<double>(routes) * (c.rankSize - 1) / c.rankSize + travel;
        const double reduceRows = travel + static_cast<double>(routes) / c.rankSize + static_cast<double>(p->bs);
        const double tLink = travel * a.rowBytes / 550e9;
        const double tSend = sendRows * a.rowBytes / 5e12;
        const double tReduce = reduceRows * a.rowBytes / 5e12;
        const double share = 1.25 * tReduce / std::max(tLink, tSend + tReduce);
        const int64_t reducersAuto = static_cast<int64_t>(grid * std::min(0.5, std::max(0.125, share)));
        a.reducerBlocks = overlap ? static_cast<uint32_t>(std::min<int64_t>(grid / 2, std::max<int64_t>(1, EnvLong("TILEXR_EP_REDUCER_BLOCKS", reducersAuto)))) : 0u;
        a.buckets = overlap ? static_cast<uint32_t>(std::min<int64_t>(EP_MAX_BUCKETS, std::max<int64_t>(1, p->bs / 512))) : 1u;
        // bucket lists live behind the slots in the same data half, when there is room for every row of the worst case
        a.listOff = (need + 255) & ~static_cast<uint64_t>(255);
        const uint64_t listRoom = c.hostArgs->dataHalfBytes > a.listOff ? (c.hostArgs->dataHalfBytes - a.listOff) / (4ull * a.buckets) : 0;
        a.listCap = static_cast<uint32_t>(std::min<uint64_t>(listRoom, static_cast<uint64_t>(routes) * c.rankSize));
        if (a.listCap < static_cast<uint64_t>(routes)) a.buckets = 1;
        a.bucketTokens = static_cast<uint32_t>((p->bs + a.buckets - 1) / a.buckets);
        // Unsorted walk: a send item looks at the tuples of chunkRows rows; about one travelling row per item
        // keeps the queue fine-grained without paying a cursor update for nothing.
        int64_t chunkRows = 32;
        while (chunkRows > 1 && (static_cast<double>(routes) / std::max(1.0, travel) < chunkRows ||
                                 (routes / chunkRows) * parts < 2 * warps)) {
            chunkRows /= 2;
        }
        a.chunkRows = static_cast<uint32_t>(chunkRows);
    }
    {
        PerfLaunchInfo info{static_cast<uint32_t>(TILEXR_OP_EP_COMBINE), static_cast<uint32_t>(p->dtype),
                            static_cast<uint32_t>(c.rank), static_cast<uint32_t>(c.rankSize), grid,
                            static_cast<uint64_t>(p->bs) * a.rowBytes};
        a.perfTrace = PerfTracePrepareLaunch(info, stream);
    }
    LaunchConfig cfg{grid, EP_BLOCK_THREADS, 0, true};
    return LaunchKernel(comm, EpCombineKernelEntry(), &a, cfg, stream);
}

// ---- reference-shaped wrappers -----------------------------------------------------------------------------

int TileXRMoeEpDispatchMemoryV2(void *x, int32_t *expertIds, void *scales, bool *xActiveMask, int64_t activeMaskType,
                                void *expertScales, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK,
                                int64_t moeExpertNum, int64_t epWorldSize, int64_t epRankId, int64_t tpWorldSize,
                                int64_t tpRankId, int64_t expertShardType, int64_t sharedExpertNum,
                                int64_t sharedExpertRankNum, int64_t quantMode, int64_t globalBs,
                                int64_t expertTokenNumsType, void *expandXOut, void *dynamicScalesOut,
                                int32_t *assistInfoForCombineOut, int64_t *expertTokenNumsOut, int32_t *sendCountsOut,
                                int32_t *tpRecvCountsOut, void *expandScalesOut, TileXRDataType dtype,
                                TileXRDataType expandXOutDtype, TileXRStream stream)
{
    (void)expertShardType;
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    if (scales != nullptr) {
        TILEXR_LOG(ERROR) << "EP dispatch: static scales are not supported (the reference rejects them too)";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    // epWorldSize counts the ranks that exchange rows: all of them (every route reaches all lanes of its group), or, as the
    // reference counts it, the expert groups
    const int64_t T = tpWorldSize > 1 ? tpWorldSize : 1;
    if (!((epWorldSize == c.rankSize && epRankId == c.rank) || (T > 1 && epWorldSize == c.rankSize / T && epRankId == c.rank / T))) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (globalBs != 0 && globalBs != bs * c.rankSize) {
        TILEXR_LOG(ERROR) << "EP dispatch: globalBs must be bs * epWorldSize";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (quantMode != TILEXR_EP_QUANT_NONE) {
        const TileXRDataType want = quantMode == TILEXR_EP_QUANT_MXFP8_E5M2 ? TILEXR_DATA_TYPE_FP8E5M2 : TILEXR_DATA_TYPE_FP8E4M3;
        if (expandXOutDtype != want) {
            TILEXR_LOG(ERROR) << "EP dispatch: quantMode " << quantMode << " writes " << (want == TILEXR_DATA_TYPE_FP8E5M2 ? "e5m2" : "e4m3");
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
    }
    TileXREpDispatchParams p;
    std::memset(&p, 0, sizeof(p));
    p.x = x;
    p.expertIds = expertIds;
    p.xActiveMask = xActiveMask;
    p.activeMaskType = activeMaskType;
    p.bs = bs;
    p.h = h;
    p.topK = topK;
    p.moeExpertNum = moeExpertNum;
    p.quantMode = quantMode;
    p.expertTokenNumsType = expertTokenNumsType;
    p.sharedExpertNum = sharedExpertNum;
    p.sharedExpertRankNum = sharedExpertRankNum;
    // worst case, as the reference sizes it: every token of every rank with all its routes on this rank
    p.maxRecvRows = bs * c.rankSize * std::min<int64_t>(topK, moeExpertNum / std::max<int64_t>(1, c.rankSize / T - sharedExpertRankNum));
    p.tpWorldSize = T;
    p.tpRankId = tpRankId;
    p.tpRecvCountsOut = tpRecvCountsOut;
    p.expertScales = static_cast<const float *>(expertScales);
    p.expandScalesOut = static_cast<float *>(expandScalesOut);
    p.expandXOut = expandXOut;
    p.dynamicScalesOut = static_cast<float *>(dynamicScalesOut);
    p.assistInfoForCombineOut = assistInfoForCombineOut;
    p.expertTokenNumsOut = expertTokenNumsOut;
    p.sendCountsOut = sendCountsOut;
    p.dtype = dtype;
    return TileXRMoeEpDispatchFused(&p, comm, stream);
}

int TileXRMoeEpDispatchMemory(void *x, int32_t *expertIds, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK,
                              int64_t moeExpertNum, void *expandXOut, int64_t *expertTokenNumsOut, int32_t *sendCountsOut,
                              int32_t *assistInfoForCombineOut, TileXRDataType dtype, TileXRStream stream)
{
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    return TileXRMoeEpDispatchMemoryV2(x, expertIds, nullptr, nullptr, TILEXR_EP_ACTIVE_MASK_NONE, nullptr, comm, bs, h, topK,
                                       moeExpertNum, c.rankSize, c.rank, 1, 0, 0, 0, 0, TILEXR_EP_QUANT_NONE, bs * c.rankSize,
                                       TILEXR_EP_TOKEN_NUMS_COUNT, expandXOut, nullptr, assistInfoForCombineOut,
                                       expertTokenNumsOut, sendCountsOut, nullptr, nullptr, dtype, dtype, stream);
}

// The reference's slot-window ("MVP") route has the same observable semantics as its memory
// route; both names run the same kernels here.
int TileXRMoeEpDispatch(void *x, int32_t *expertIds, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK,
                        int64_t moeExpertNum, void *expandXOut, int64_t *expertTokenNumsOut, int32_t *epRecvCountsOut,
                        int32_t *assistInfoForCombineOut, TileXRDataType dtype, TileXRStream stream)
{
    return TileXRMoeEpDispatchMemory(x, expertIds, comm, bs, h, topK, moeExpertNum, expandXOut, expertTokenNumsOut,
                                     epRecvCountsOut, assistInfoForCombineOut, dtype, stream);
}

int TileXRMoeEpDispatchV2(void *x, int32_t *expertIds, void *scales, bool *xActiveMask, void *expertScales,
                          TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum,
                          int64_t epWorldSize, int64_t epRankId, int64_t tpWorldSize, int64_t tpRankId,
                          int64_t expertShardType, int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t quantMode,
                          int64_t globalBs, int64_t expertTokenNumsType, void *expandXOut, void *dynamicScalesOut,
                          int32_t *assistInfoForCombineOut, int64_t *expertTokenNumsOut, int32_t *epRecvCountsOut,
                          int32_t *tpRecvCountsOut, void *expandScalesOut, void *workspace, TileXRDataType dtype,
                          TileXRStream stream)
{
    (void)workspace;
    return TileXRMoeEpDispatchMemoryV2(x, expertIds, scales, xActiveMask,
                                       xActiveMask != nullptr ? TILEXR_EP_ACTIVE_MASK_TOKEN : TILEXR_EP_ACTIVE_MASK_NONE,
                                       expertScales, comm, bs, h, topK, moeExpertNum, epWorldSize, epRankId, tpWorldSize,
                                       tpRankId, expertShardType, sharedExpertNum, sharedExpertRankNum, quantMode, globalBs,
                                       expertTokenNumsType, expandXOut, dynamicScalesOut, assistInfoForCombineOut,
                                       expertTokenNumsOut, epRecvCountsOut, tpRecvCountsOut, expandScalesOut, dtype,
                                       quantMode == TILEXR_EP_QUANT_NONE ? dtype : TILEXR_DATA_TYPE_FP8E4M3, stream);
}

int TileXRMoeEpCombineMemoryV2(void *expertOut, int32_t *assistInfoForCombine, int32_t *sendCounts, float *expertScales,
                               bool *xActiveMask, int64_t activeMaskType, void *sharedExpertX, TileXRCommPtr comm,
                               int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, int64_t epWorldSize,
                               int64_t epRankId, int64_t tpWorldSize, int64_t tpRankId, int64_t expertShardType,
                               int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t quantMode, int64_t globalBs,
                               void *yOut, TileXRDataType dtype, TileXRStream stream)
{
    (void)expertShardType;
    (void)globalBs;
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    const int64_t T = tpWorldSize > 1 ? tpWorldSize : 1;
    if (quantMode != TILEXR_EP_QUANT_NONE) {
        TILEXR_LOG(ERROR) << "EP combine: rows travel in their own dtype; communication quantisation is not supported";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    if (!((epWorldSize == c.rankSize && epRankId == c.rank) || (T > 1 && epWorldSize == c.rankSize / T && epRankId == c.rank / T))) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    TileXREpCombineParams p;
    std::memset(&p, 0, sizeof(p));
    p.tpWorldSize = T;
    p.tpRankId = tpRankId;
    p.expertOut = expertOut;
    p.assistInfoForCombine = assistInfoForCombine;
    p.sendCounts = sendCounts;
    p.expertScales = expertScales;
    p.xActiveMask = xActiveMask;
    p.activeMaskType = activeMaskType;
    p.sharedExpertX = sharedExpertX;
    p.sharedExpertNum = sharedExpertNum;
    p.sharedExpertRankNum = sharedExpertRankNum;
    p.bs = bs;
    p.h = h;
    p.topK = topK;
    p.moeExpertNum = moeExpertNum;
    p.yOut = yOut;
    p.dtype = dtype;
    return TileXRMoeEpCombineFused(&p, comm, stream);
}

int TileXRMoeEpCombineMemory(void *expertOut, int32_t *assistInfoForCombine, int32_t *epRecvCounts, TileXRCommPtr comm,
                             int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, void *yOut, TileXRDataType dtype,
                             TileXRStream stream)
{
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_SUCCESS) return ret;
    return TileXRMoeEpCombineMemoryV2(expertOut, assistInfoForCombine, epRecvCounts, nullptr, nullptr,
                                      TILEXR_EP_ACTIVE_MASK_NONE, nullptr, comm, bs, h, topK, moeExpertNum, c.rankSize, c.rank,
                                      1, 0, 0, 0, 0, TILEXR_EP_QUANT_NONE, bs * c.rankSize, yOut, dtype, stream);
}

int TileXRMoeEpCombine(void *expertOut, int32_t *assistInfoForCombine, int32_t *epRecvCounts, TileXRCommPtr comm,
                       int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, void *yOut, TileXRDataType dtype,
                       TileXRStream stream)
{
    return TileXRMoeEpCombineMemory(expertOut, assistInfoForCombine, epRecvCounts, comm, bs, h, topK, moeExpertNum, yOut, dtype,
                                    stream);
}

int TileXRMoeEpCombineV2(void *expertOut, int32_t *assistInfoForCombine, int32_t *epRecvCounts, TileXRCommPtr comm,
                         int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, void *yOut, void *workspace,
                         TileXRDataType dtype, TileXRStream stream)
{
    (void)workspace;
    return TileXRMoeEpCombineMemory(expertOut, assistInfoForCombine, epRecvCounts, comm, bs, h, topK, moeExpertNum, yOut, dtype,
                                    stream);
}

// ---- stand-alone ops ------------------------------------------------------------------------------------------

int TileXRMoeRoutingTopK(const float *gateLogits, const float *selectionBias, int64_t bs, int64_t moeExpertNum,
                         int64_t topK, int64_t scoreFunc, int64_t renormalize, float routedScalingFactor,
                         int32_t *topkIdsOut, float *topkWeightsOut, TileXRStream stream)
{
    if (gateLogits == nullptr || topkIdsOut == nullptr || topkWeightsOut == nullptr || bs <= 0 || moeExpertNum <= 0 ||
        moeExpertNum > EP_MAX_EXPERTS || topK <= 0 || topK > EP_MAX_TOPK || topK > moeExpertNum ||
        (scoreFunc != TILEXR_EP_SCORE_SOFTMAX && scoreFunc != TILEXR_EP_SCORE_SIGMOID)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    RoutingArgs a{gateLogits, selectionBias, topkIdsOut, topkWeightsOut, static_cast<int32_t>(bs),
                  static_cast<int32_t>(moeExpertNum), static_cast<int32_t>(topK), static_cast<int32_t>(scoreFunc),
                  static_cast<int32_t>(renormalize), routedScalingFactor == 0.f ? 1.0f : routedScalingFactor};
    return LaunchRoutingTopK(a, stream);
}

static bool HalfType(int dtype) { return dtype == TILEXR_DATA_TYPE_FP16 || dtype == TILEXR_DATA_TYPE_BFP16; }

int TileXRFp8Quant1x128(const void *x, int64_t rows, int64_t h, TileXRDataType dtype, void *yOut, float *scalesOut,
                        TileXRStream stream)
{
    if (x == nullptr || yOut == nullptr || scalesOut == nullptr || rows <= 0 || h <= 0 || h % 128 != 0 || !HalfType(dtype)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return LaunchFp8Quant1x128(x, rows, h, dtype == TILEXR_DATA_TYPE_BFP16, yOut, scalesOut, stream);
}

int TileXRFp8Dequant1x128(const void *y, const float *scales, int64_t rows, int64_t h, TileXRDataType dtype, void *xOut,
                          TileXRStream stream)
{
    if (y == nullptr || xOut == nullptr || scales == nullptr || rows <= 0 || h <= 0 || h % 128 != 0 || !HalfType(dtype)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return LaunchFp8Dequant1x128(y, scales, rows, h, dtype == TILEXR_DATA_TYPE_BFP16, xOut, stream);
}

int TileXRMxfp8Quant(const void *x, int64_t rows, int64_t h, TileXRDataType dtype, TileXRDataType fp8Type, void *yOut,
                     uint8_t *scalesOut, TileXRStream stream)
{
    if (x == nullptr || yOut == nullptr || scalesOut == nullptr || rows <= 0 || h <= 0 || !HalfType(dtype) ||
        (fp8Type != TILEXR_DATA_TYPE_FP8E4M3 && fp8Type != TILEXR_DATA_TYPE_FP8E5M2)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return LaunchMxfp8Quant(x, rows, h, dtype == TILEXR_DATA_TYPE_BFP16, fp8Type == TILEXR_DATA_TYPE_FP8E5M2, yOut, scalesOut,
                            stream);
}

int TileXRMxfp8Dequant(const void *y, const uint8_t *scales, int64_t rows, int64_t h, TileXRDataType fp8Type,
                       TileXRDataType dtype, void *xOut, TileXRStream stream)
{
    if (y == nullptr || xOut == nullptr || scales == nullptr || rows <= 0 || h <= 0 || !HalfType(dtype) ||
        (fp8Type != TILEXR_DATA_TYPE_FP8E4M3 && fp8Type != TILEXR_DATA_TYPE_FP8E5M2)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return LaunchMxfp8Dequant(y, scales, rows, h, fp8Type == TILEXR_DATA_TYPE_FP8E5M2, dtype == TILEXR_DATA_TYPE_BFP16, xOut,
                              stream);
}

int TileXRRmsNorm(const void *x, void *residualInOut, const void *gamma, float eps, int64_t rows, int64_t h,
                  TileXRDataType dtype, void *yOut, TileXRStream stream)
{
    if (x == nullptr || gamma == nullptr || yOut == nullptr || rows <= 0 || h <= 0 || h % 8 != 0 || h > 16384 ||
        !HalfType(dtype)) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return LaunchRmsNorm(x, residualInOut, gamma, eps, rows, h, dtype == TILEXR_DATA_TYPE_BFP16, yOut, stream);
}

} // extern "C"
