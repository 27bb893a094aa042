// Host side of the second-generation MoonEP planner: route/target helpers, the CPU oracle, workspace sizing and
// the kernel launch.  Contract in tilexr_ep_plan.h.
#include <algorithm>
#include <cstring>
#include <vector>

#include <cuda_runtime_api.h>

#include "plan_v2_kernel.h"
#include "tilexr_launch.h"
#include "tilexr_log.h"
#include "tilexr_moonep_planner.h"
#include "tilexr_types.h"

using namespace TileXR;

namespace {

constexpr int64_t kI32Max = 0x7fffffff;

uint64_t Mix(uint64_t h, uint64_t v)
{
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return h * 0xff51afd7ed558ccdull;
}

// What all ranks must agree on before their plans can fit together.
uint64_t HeaderHash(int64_t R, int64_t s, int64_t k, int64_t e, const TileXRMoonEPPlanConfig &c)
{
    uint64_t h = 0x54584d4f4f4e3256ull;
    const int64_t words[] = {R, s, k, e, c.prefetchSlots, c.rankTokenCapacity, c.nvS, c.tokenPadding, c.tokenRouteLimitPerPair,
                             c.cardsPerServer, c.cardsPerCabinet, c.crossCandidateCount, TILEXR_MOONEP_PLAN_METADATA_V2_ABI_VERSION};
    for (int64_t w : words) h = Mix(h, static_cast<uint64_t>(w));
    return h;
}

int RankOf(TileXRCommPtr comm, int *rank, int *rankSize)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    TileXRCommArgs *hostArgs = nullptr;
    const int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    *rank = hostArgs->rank;
    *rankSize = hostArgs->rankSize;
    return TILEXR_SUCCESS;
}

int LaunchPlan(const int32_t *topk, const int32_t *tpe, const int32_t *globalIds, TileXRCommPtr comm, int64_t s, int64_t k, int64_t e,
               const TileXRMoonEPPlanConfig *config, const plan2::Outputs &out, void *workspace, uint64_t workspaceBytes,
               TileXRStream stream, const TileXRMoonEPStageTables *stage = nullptr)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_ERROR_NOT_SUPPORT;
    if (topk == nullptr || tpe == nullptr || globalIds == nullptr || config == nullptr || out.dst == nullptr || out.cuSeqlens == nullptr ||
        out.expertsToCopy == nullptr || out.remoteStats == nullptr || out.status == nullptr || workspace == nullptr ||
        ((out.remoteExperts == nullptr) != (out.expertTargets == nullptr))) {
        TILEXR_LOG(ERROR) << "MoonEP plan v2: null argument";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const int R = hostArgs->rankSize;
    if (plan2::ValidateConfig(hostArgs->rank, R, s, k, e, *config) != PLAN_OK) {
        TILEXR_LOG(ERROR) << "MoonEP plan v2: configuration rejected (capacity must be s*k, nvS >= capacity, topology constants 8/64/3)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    PlanV2Args a;
    std::memset(&a, 0, sizeof(a));
    a.dims = plan2::MakeDims(hostArgs->rank, R, s, k, e, *config);
    if (workspaceBytes < plan2::TableInts(a.dims) * sizeof(int32_t) || reinterpret_cast<uintptr_t>(workspace) % 8 != 0) {
        TILEXR_LOG(ERROR) << "MoonEP plan v2: workspace of " << workspaceBytes << " bytes, need " << plan2::TableInts(a.dims) * 4
                          << " (8-byte aligned)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    a.mailStride = static_cast<uint32_t>((16 + static_cast<uint64_t>(e) * 4 + 15) / 16 * 16);
    a.dstLocalOff = (static_cast<uint64_t>(a.mailStride) * R + 255) / 256 * 256;
    const uint64_t windowBytes = a.dstLocalOff + (stage != nullptr ? static_cast<uint64_t>(a.dims.nvS) * 8 : 0);
    if (windowBytes > hostArgs->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "MoonEP plan v2: the exchange needs " << windowBytes << " window bytes";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (stage != nullptr) {
        if (stage->dst == nullptr || stage->zeroFillRanges == nullptr || stage->dstLocal == nullptr || stage->status == nullptr) {
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
        a.stageDst = stage->dst;
        a.stageZeroFill = stage->zeroFillRanges;
        a.stageDstLocal = stage->dstLocal;
        a.stageStatus = stage->status;
    }
    a.topk = topk;
    a.tpe = tpe;
    a.globalIds = globalIds;
    a.out = out;
    a.tables = static_cast<int32_t *>(workspace);
    a.comm = reinterpret_cast<CommArgs *>(devArgs);
    a.headerHash = HeaderHash(R, s, k, e, *config);
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    a.magic = magic;
    // shared memory for the balancing tables, the histogram table and the segment list, when they fit
    const int64_t stagedWords = 6ll * R + 5ll * R * e + static_cast<int64_t>(R) * a.dims.B + 2ll * R * R + e + static_cast<int64_t>(R) * e +
                                static_cast<int64_t>(a.dims.segCapacity) * (sizeof(plan2::Segment) / 4);
    size_t smem = 0;
    if (stagedWords * 4 <= 200 * 1024) {
        smem = static_cast<size_t>(stagedWords) * 4;
        a.stagedWords = static_cast<uint32_t>(stagedWords);
    }
    LaunchConfig cfg{1, PLAN_V2_THREADS, smem, true};
    return LaunchKernel(comm, PlanV2KernelEntry(), &a, cfg, stream);
}

} // namespace

extern "C" {

int TileXRMoonEPEncodeGlobalTokenId(int32_t srcRank, int32_t tokenId, int32_t topKId, int64_t rankSize, int64_t s, int64_t topK,
                                    uint64_t *globalTokenId)
{
    if (globalTokenId == nullptr || rankSize <= 0 || s <= 0 || topK <= 0 || srcRank < 0 || srcRank >= rankSize || tokenId < 0 ||
        tokenId >= s || topKId < 0 || topKId >= topK) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    const unsigned __int128 id = (static_cast<unsigned __int128>(srcRank) * static_cast<uint64_t>(s) + static_cast<uint64_t>(tokenId)) *
                                     static_cast<uint64_t>(topK) + static_cast<uint64_t>(topKId);
    if (id >= static_cast<unsigned __int128>(TILEXR_MOONEP_INVALID_GLOBAL_TOKEN_ID)) return PLAN_ERROR_CONFIG_MISMATCH;
    *globalTokenId = static_cast<uint64_t>(id);
    return PLAN_OK;
}

int TileXRMoonEPDecodeGlobalTokenId(uint64_t globalTokenId, int64_t rankSize, int64_t s, int64_t topK, int32_t *srcRank,
                                    int32_t *tokenId, int32_t *topKId)
{
    if (srcRank == nullptr || tokenId == nullptr || topKId == nullptr || rankSize <= 0 || s <= 0 || topK <= 0 ||
        globalTokenId == TILEXR_MOONEP_INVALID_GLOBAL_TOKEN_ID) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    const uint64_t token = globalTokenId / static_cast<uint64_t>(topK);
    const uint64_t rank = token / static_cast<uint64_t>(s);
    const uint64_t inRank = token % static_cast<uint64_t>(s);
    const uint64_t kk = globalTokenId % static_cast<uint64_t>(topK);
    if (rank >= static_cast<uint64_t>(rankSize) || inRank > static_cast<uint64_t>(kI32Max) || kk > static_cast<uint64_t>(kI32Max)) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    *srcRank = static_cast<int32_t>(rank);
    *tokenId = static_cast<int32_t>(inRank);
    *topKId = static_cast<int32_t>(kk);
    return PLAN_OK;
}

int TileXRMoonEPDecodeDst(int32_t encoded, int64_t nvS, int64_t rankSize, TileXRMoonEPRouteTarget *target)
{
    if (target == nullptr || nvS <= 0 || nvS > kI32Max || rankSize <= 0 || rankSize > 128 || rankSize * nvS > kI32Max + 1) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    const int32_t raw = encoded >= 0 ? encoded : ~encoded;
    const int64_t rank = raw / nvS, slot = raw % nvS;
    if (rank >= rankSize) return PLAN_ERROR_CONFIG_MISMATCH;
    target->rawDst = raw;
    target->dstRank = static_cast<int32_t>(rank);
    target->recvSlot = static_cast<int32_t>(slot);
    target->sendHidden = encoded >= 0 ? 1 : 0;
    target->writeRouteWeight = 1;
    return PLAN_OK;
}

int TileXRMoonEPBuildRouteDescriptor(int32_t srcRank, int32_t tokenId, int32_t topKId, int32_t encodedDst, int64_t rankSize,
                                     int64_t s, int64_t topK, int64_t nvS, TileXRMoonEPRouteDescriptor *descriptor)
{
    if (descriptor == nullptr) return PLAN_ERROR_CONFIG_MISMATCH;
    uint64_t id = 0;
    int st = TileXRMoonEPEncodeGlobalTokenId(srcRank, tokenId, topKId, rankSize, s, topK, &id);
    if (st != PLAN_OK) return st;
    TileXRMoonEPRouteTarget t;
    st = TileXRMoonEPDecodeDst(encodedDst, nvS, rankSize, &t);
    if (st != PLAN_OK) return st;
    descriptor->srcRank = srcRank;
    descriptor->tokenId = tokenId;
    descriptor->topKId = topKId;
    descriptor->globalTokenId = id;
    descriptor->rawDst = t.rawDst;
    descriptor->dstRank = t.dstRank;
    descriptor->recvSlot = t.recvSlot;
    descriptor->sendHidden = t.sendHidden;
    descriptor->writeRouteWeight = t.writeRouteWeight;
    return PLAN_OK;
}

int TileXRMoonEPBuildExpertTargets(const int32_t *remoteExperts, int64_t rankSize, int64_t expertNum, int64_t prefetchSlots,
                                   int32_t ownerRank, uint64_t *expertTargets, uint64_t expertTargetsCount)
{
    if (remoteExperts == nullptr || expertTargets == nullptr || rankSize <= 0 || rankSize > 128 || expertNum <= 0 ||
        expertNum % rankSize != 0 || prefetchSlots < 0 || ownerRank < 0 || ownerRank >= rankSize) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    const int64_t L = expertNum / rankSize, words = (rankSize + 63) / 64;
    if (expertTargetsCount != static_cast<uint64_t>(L * words)) return PLAN_ERROR_CONFIG_MISMATCH;
    std::memset(expertTargets, 0, expertTargetsCount * sizeof(uint64_t));
    for (int64_t dst = 0; dst < rankSize; ++dst) {
        for (int64_t slot = 0; slot < prefetchSlots; ++slot) {
            const int32_t e = remoteExperts[dst * prefetchSlots + slot];
            if (e < 0) continue;
            if (e >= expertNum) return PLAN_ERROR_INTERNAL_INVARIANT;
            if (e / L == ownerRank) expertTargets[(e - ownerRank * L) * words + dst / 64] |= 1ull << (dst % 64);
        }
    }
    return PLAN_OK;
}

int TileXRMoonEPBuildDuplicateMetadata(const TileXRMoonEPReceivedRoute *records, int64_t recordCount, int64_t rankSize, int64_t s,
                                       int64_t topK, int64_t nvS, int32_t *dupGroups, int32_t *dupLoffs, int32_t *dupCounts)
{
    if ((records == nullptr && recordCount != 0) || recordCount < 0 || rankSize <= 0 || rankSize > 128 || s <= 0 || topK <= 0 ||
        topK > 32 || nvS <= 0 || nvS > kI32Max || dupGroups == nullptr || dupLoffs == nullptr || dupCounts == nullptr ||
        s > INT64_MAX / topK || rankSize > INT64_MAX / (s * topK) || recordCount > rankSize * s * topK) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    for (int64_t i = 0; i < nvS * 3; ++i) dupGroups[i] = -1;
    for (int64_t i = 0; i < nvS; ++i) dupLoffs[i] = -1;
    dupCounts[0] = 0;
    dupCounts[1] = 0;
    // order the records by (source rank, token, topK index): groups come out in that order, duplicates in topK order
    std::vector<uint64_t> keys(static_cast<size_t>(recordCount));
    for (int64_t i = 0; i < recordCount; ++i) {
        const TileXRMoonEPReceivedRoute &r = records[i];
        if (r.srcRank < 0 || r.srcRank >= rankSize || r.tokenId < 0 || r.tokenId >= s || r.topKId < 0 || r.topKId >= topK ||
            r.recvSlot < 0 || r.recvSlot >= nvS || (r.isPrimary != 0 && r.isPrimary != 1)) {
            return PLAN_ERROR_CONFIG_MISMATCH;
        }
        const uint64_t id = (static_cast<uint64_t>(r.srcRank) * static_cast<uint64_t>(s) + static_cast<uint64_t>(r.tokenId)) *
                                static_cast<uint64_t>(topK) + static_cast<uint64_t>(r.topKId);
        keys[static_cast<size_t>(i)] = id;
    }
    std::vector<int64_t> order(static_cast<size_t>(recordCount));
    for (int64_t i = 0; i < recordCount; ++i) order[static_cast<size_t>(i)] = i;
    std::sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return keys[static_cast<size_t>(a)] < keys[static_cast<size_t>(b)]; });
    for (int64_t i = 1; i < recordCount; ++i) {
        if (keys[static_cast<size_t>(order[static_cast<size_t>(i)])] == keys[static_cast<size_t>(order[static_cast<size_t>(i - 1)])]) {
            return PLAN_ERROR_INTERNAL_INVARIANT;   // the same route twice
        }
    }
    int32_t groups = 0, dups = 0;
    for (int64_t first = 0; first < recordCount;) {
        const uint64_t token = keys[static_cast<size_t>(order[static_cast<size_t>(first)])] / static_cast<uint64_t>(topK);
        int64_t last = first;
        while (last < recordCount && keys[static_cast<size_t>(order[static_cast<size_t>(last)])] / static_cast<uint64_t>(topK) == token) ++last;
        int32_t primaries = 0, primarySlot = -1;
        for (int64_t i = first; i < last; ++i) {
            const TileXRMoonEPReceivedRoute &r = records[order[static_cast<size_t>(i)]];
            if (r.isPrimary) {
                ++primaries;
                primarySlot = r.recvSlot;
            }
        }
        if (primaries != 1) return PLAN_ERROR_INTERNAL_INVARIANT;
        const int32_t extra = static_cast<int32_t>(last - first - 1);
        if (extra > 0) {
            if (groups >= nvS || dups > nvS - extra) return PLAN_ERROR_MOVE_RECORD_OVERFLOW;
            dupGroups[groups * 3] = primarySlot;
            dupGroups[groups * 3 + 1] = dups;
            dupGroups[groups * 3 + 2] = extra;
            for (int64_t i = first; i < last; ++i) {
                const TileXRMoonEPReceivedRoute &r = records[order[static_cast<size_t>(i)]];
                if (!r.isPrimary) dupLoffs[dups++] = r.recvSlot;
            }
            ++groups;
        }
        first = last;
    }
    dupCounts[0] = groups;
    dupCounts[1] = dups;
    return PLAN_OK;
}

int TileXRMoeEpPlanV2GetWorkspaceSize(int64_t rankSize, int64_t s, int64_t topK, int64_t expertNum,
                                      const TileXRMoonEPPlanConfig *config, uint64_t *localWorkspaceBytes,
                                      uint64_t *registeredMetaBytes)
{
    if (config == nullptr || localWorkspaceBytes == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (plan2::ValidateConfig(0, rankSize, s, topK, expertNum, *config) != PLAN_OK) return TILEXR_ERROR_PARA_CHECK_FAIL;
    const plan2::Dims d = plan2::MakeDims(0, rankSize, s, topK, expertNum, *config);
    *localWorkspaceBytes = (plan2::TableInts(d) * sizeof(int32_t) + 63) / 64 * 64;
    if (registeredMetaBytes != nullptr) *registeredMetaBytes = 0;
    return TILEXR_SUCCESS;
}

int TileXRMoeEpPlanV2Reference(int32_t rank, int64_t rankSize, const int32_t *topkExperts, const int32_t *tokensPerExpert,
                               const int32_t *globalRankIds, int64_t s, int64_t topK, int64_t expertNum,
                               const TileXRMoonEPPlanConfig *config, int32_t *dst, int32_t *cuSeqlens, int32_t *expertsToCopy,
                               int32_t *remoteStats, int32_t *remoteExperts, uint64_t *expertTargets, int32_t *status)
{
    if (status == nullptr) return PLAN_ERROR_CONFIG_MISMATCH;
    for (int i = 0; i < TILEXR_MOONEP_PLAN_STATUS_WORDS; ++i) status[i] = 0;
    status[0] = PLAN_ERROR_CONFIG_MISMATCH;
    if (topkExperts == nullptr || tokensPerExpert == nullptr || globalRankIds == nullptr || config == nullptr || dst == nullptr ||
        cuSeqlens == nullptr || expertsToCopy == nullptr || remoteStats == nullptr ||
        ((remoteExperts == nullptr) != (expertTargets == nullptr)) ||
        plan2::ValidateConfig(rank, rankSize, s, topK, expertNum, *config) != PLAN_OK) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    const plan2::Dims d = plan2::MakeDims(rank, rankSize, s, topK, expertNum, *config);
    std::vector<int32_t> storage(plan2::TableInts(d) + 2);
    int32_t *base = storage.data();
    if (reinterpret_cast<uintptr_t>(base) % 8 != 0) ++base;
    plan2::Tables t;
    plan2::Carve(d, base, &t);
    const plan2::Inputs in{topkExperts, tokensPerExpert, globalRankIds};
    const plan2::Outputs out{dst, cuSeqlens, expertsToCopy, remoteStats, remoteExperts, expertTargets, status};
    const int32_t v = plan2::PlanValidate(d, in, t);
    if (v != PLAN_OK) {
        status[0] = v;
        return v;
    }
    plan2::Progress g;
    plan2::PlanInitSerial(d, in, t);
    plan2::PlanBalance(d, in, out, t, g);
    bool routesOk = true;
    for (int32_t i = 0; i < d.cap; ++i) dst[i] = 0;
    if (plan2::PlanHasDestinations(g)) {
        plan2::PlanOrdinalsSerial(d, in, t);
        for (int32_t i = 0; i < d.cap; ++i) {
            const int32_t raw = plan2::PlanRouteDst(d, in, t, g, i);
            routesOk = routesOk && raw >= 0;
            dst[i] = raw < 0 ? 0 : raw;
        }
        if (routesOk) {
            for (int32_t tok = 0; tok < d.S; ++tok) plan2::PlanMarkDuplicates(d, dst, tok);
        }
    }
    return plan2::PlanFinish(d, t, g, routesOk, status);
}

int TileXRMoeEpPlanV2(const int32_t *topkExperts, const int32_t *tokensPerExpert, const int32_t *globalRankIds, TileXRCommPtr comm,
                      int64_t s, int64_t topK, int64_t expertNum, const TileXRMoonEPPlanConfig *config, TileXRMoonEPPlanDesc *plan,
                      void *localWorkspace, uint64_t localWorkspaceBytes, void *registeredMetaWorkspace,
                      uint64_t registeredMetaBytes, TileXRStream stream)
{
    (void)registeredMetaWorkspace;
    (void)registeredMetaBytes;
    if (plan == nullptr || config == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    const plan2::Outputs out{plan->dst, plan->cuSeqlens, plan->expertsToCopy, plan->remoteStats, nullptr, nullptr, plan->status};
    const int ret = LaunchPlan(topkExperts, tokensPerExpert, globalRankIds, comm, s, topK, expertNum, config, out, localWorkspace,
                               localWorkspaceBytes, stream);
    if (ret != TILEXR_SUCCESS) return ret;
    int rank = 0, rankSize = 0;
    RankOf(comm, &rank, &rankSize);
    plan->s = s;
    plan->k = topK;
    plan->r = rankSize;
    plan->e = expertNum;
    plan->b = config->prefetchSlots;
    plan->cap = s * topK;
    plan->nvS = config->nvS;
    plan->tokenPadding = config->tokenPadding;
    plan->epoch += 1;
    return TILEXR_SUCCESS;
}

int TileXRMoeEpPlanV2WithMetadata(const int32_t *topkExperts, const int32_t *tokensPerExpert, const int32_t *globalRankIds,
                                  TileXRCommPtr comm, int64_t s, int64_t topK, int64_t expertNum,
                                  const TileXRMoonEPPlanConfig *config, TileXRMoonEPPlanMetadataV2 *m, void *localWorkspace,
                                  uint64_t localWorkspaceBytes, void *registeredMetaWorkspace, uint64_t registeredMetaBytes,
                                  TileXRStream stream)
{
    (void)registeredMetaWorkspace;
    (void)registeredMetaBytes;
    return TileXRMoeEpPlanV2WithStageTables(topkExperts, tokensPerExpert, globalRankIds, comm, s, topK, expertNum, config, m, nullptr,
                                            localWorkspace, localWorkspaceBytes, stream);
}

int TileXRMoeEpPlanV2WithStageTables(const int32_t *topkExperts, const int32_t *tokensPerExpert, const int32_t *globalRankIds,
                                     TileXRCommPtr comm, int64_t s, int64_t topK, int64_t expertNum,
                                     const TileXRMoonEPPlanConfig *config, TileXRMoonEPPlanMetadataV2 *m,
                                     const TileXRMoonEPStageTables *stage, void *localWorkspace, uint64_t localWorkspaceBytes,
                                     TileXRStream stream)
{
    if (m == nullptr || config == nullptr || m->structSize < sizeof(TileXRMoonEPPlanMetadataV2) ||
        m->abiVersion != TILEXR_MOONEP_PLAN_METADATA_V2_ABI_VERSION) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    int rank = 0, rankSize = 0;
    if (RankOf(comm, &rank, &rankSize) != TILEXR_SUCCESS || rankSize <= 0) return TILEXR_ERROR_NOT_INITIALIZED;
    const uint64_t R = static_cast<uint64_t>(rankSize), B = static_cast<uint64_t>(config->prefetchSlots);
    const uint64_t E = static_cast<uint64_t>(expertNum), words = (R + 63) / 64;
    if (m->dstCount != static_cast<uint64_t>(s * topK) || m->cuSeqlensCount != E + B || m->remoteExpertsCount != R * B ||
        m->expertTargetsCount != E / R * words || m->remoteStatsCount != 2 || m->statusCount != TILEXR_MOONEP_PLAN_STATUS_WORDS ||
        m->remoteExperts == nullptr || m->expertTargets == nullptr) {
        TILEXR_LOG(ERROR) << "MoonEP plan v2: metadata table sizes do not match the call";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    // The slot table of this rank is row `rank` of remoteExperts: the kernel needs a separate expertsToCopy table
    // only for the descriptor form, so that row is used for both.
    const plan2::Outputs out{m->dst, m->cuSeqlens, m->remoteExperts + static_cast<uint64_t>(rank) * B, m->remoteStats, m->remoteExperts,
                             m->expertTargets, m->status};
    const int ret = LaunchPlan(topkExperts, tokensPerExpert, globalRankIds, comm, s, topK, expertNum, config, out, localWorkspace,
                               localWorkspaceBytes, stream, stage);
    if (ret != TILEXR_SUCCESS) return ret;
    m->s = s;
    m->k = topK;
    m->r = rankSize;
    m->e = expertNum;
    m->b = config->prefetchSlots;
    m->nvS = config->nvS;
    m->epoch += 1;
    return TILEXR_SUCCESS;
}

} // extern "C"

// ---- the older call shape: one workspace, no configuration (tilexr_moonep_planner.h) ------------------------------------------
namespace {

struct CompatLayout {
    uint64_t tablesBytes, rankIdsOff, statusOff, totalBytes;
};

TileXRMoonEPPlanConfig CompatConfig(int64_t rankSize, int64_t s, int64_t k, int64_t expertCount)
{
    TileXRMoonEPPlanConfig c;
    std::memset(&c, 0, sizeof(c));
    c.prefetchSlots = expertCount / rankSize;
    c.rankTokenCapacity = s * k;
    c.nvS = c.rankTokenCapacity;
    c.tokenPadding = 1;
    c.tokenRouteLimitPerPair = 0;
    c.cardsPerServer = TILEXR_MOONEP_PLAN_CARDS_PER_SERVER;
    c.cardsPerCabinet = TILEXR_MOONEP_PLAN_CARDS_PER_CABINET;
    c.crossCandidateCount = TILEXR_MOONEP_PLAN_CROSS_CANDIDATES;
    return c;
}

int CompatLayoutOf(int64_t rankSize, int64_t s, int64_t k, int64_t expertCount, CompatLayout *out)
{
    if (rankSize <= 0 || s <= 0 || k <= 0 || expertCount <= 0 || expertCount % rankSize != 0 || s > kI32Max / k) return TILEXR_ERROR_PARA_CHECK_FAIL;
    const TileXRMoonEPPlanConfig c = CompatConfig(rankSize, s, k, expertCount);
    uint64_t tables = 0;
    const int ret = TileXRMoeEpPlanV2GetWorkspaceSize(rankSize, s, k, expertCount, &c, &tables, nullptr);
    if (ret != TILEXR_SUCCESS) return ret;
    auto align = [](uint64_t v) { return (v + 63) / 64 * 64; };
    out->tablesBytes = tables;
    out->rankIdsOff = align(tables);
    out->statusOff = align(out->rankIdsOff + static_cast<uint64_t>(rankSize) * sizeof(int32_t));
    out->totalBytes = align(out->statusOff + TILEXR_MOONEP_PLAN_STATUS_WORDS * sizeof(int32_t));
    return TILEXR_SUCCESS;
}

} // namespace

extern "C" {

int TileXRMoonEpPlannerGetWorkspaceSizeV2(TileXRCommPtr comm, int64_t s, int64_t k, int64_t expertCount, uint64_t *workspaceBytes,
                                          int64_t *dispatchedCapacity)
{
    if (workspaceBytes == nullptr || dispatchedCapacity == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *workspaceBytes = 0;
    *dispatchedCapacity = 0;
    int rank = 0, rankSize = 0;
    int ret = RankOf(comm, &rank, &rankSize);
    if (ret != TILEXR_SUCCESS) return ret;
    CompatLayout layout;
    ret = CompatLayoutOf(rankSize, s, k, expertCount, &layout);
    if (ret != TILEXR_SUCCESS) return ret;
    *workspaceBytes = layout.totalBytes;
    *dispatchedCapacity = s * k;
    return TILEXR_SUCCESS;
}

int TileXRMoonEpPlannerV2(const int32_t *topkExpertIds, const int32_t *tokensPerExpert, TileXRCommPtr comm, int64_t s, int64_t k,
                          int64_t expertCount, void *workspace, uint64_t workspaceBytes, int32_t *dst, int32_t *cuSeqlens,
                          int32_t *expertsToCopy, int32_t *remoteStats, int32_t *plannerStatus, uint64_t waitIterations,
                          TileXRStream stream)
{
    if (topkExpertIds == nullptr || tokensPerExpert == nullptr || workspace == nullptr || dst == nullptr || cuSeqlens == nullptr ||
        expertsToCopy == nullptr || remoteStats == nullptr || plannerStatus == nullptr || waitIterations == 0 ||
        reinterpret_cast<uintptr_t>(workspace) % 64 != 0) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    TileXRCommArgs *hostArgs = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_ERROR_NOT_SUPPORT;      // the planner is a CUDA kernel
    const int rankSize = hostArgs->rankSize, local = hostArgs->localRankSize;
    CompatLayout layout;
    ret = CompatLayoutOf(rankSize, s, k, expertCount, &layout);
    if (ret != TILEXR_SUCCESS || workspaceBytes < layout.totalBytes || local <= 0 || rankSize % local != 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    // a rank's place in its server decides the balancing order: local ranks fill a server of eight cards from its first card
    std::vector<int32_t> ids(static_cast<size_t>(rankSize));
    for (int r = 0; r < rankSize; ++r) ids[static_cast<size_t>(r)] = (r / local) * TILEXR_MOONEP_PLAN_CARDS_PER_SERVER + r % local;
    uint8_t *base = static_cast<uint8_t *>(workspace);
    int32_t *idsDev = reinterpret_cast<int32_t *>(base + layout.rankIdsOff);
    int32_t *statusDev = reinterpret_cast<int32_t *>(base + layout.statusOff);
    // pageable source: the call returns once the ids are staged, so the vector may go
    if (cudaMemcpyAsync(idsDev, ids.data(), ids.size() * sizeof(int32_t), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        return TILEXR_ERROR_MKIRT;
    }
    const TileXRMoonEPPlanConfig config = CompatConfig(rankSize, s, k, expertCount);
    const plan2::Outputs out{dst, cuSeqlens, expertsToCopy, remoteStats, nullptr, nullptr, statusDev};
    ret = LaunchPlan(topkExpertIds, tokensPerExpert, idsDev, comm, s, k, expertCount, &config, out, base, layout.tablesBytes, stream);
    if (ret != TILEXR_SUCCESS) return ret;
    // behind the planner's launch (a communicator of an emulated world only queues it until its group closes)
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    return RunAfterLaunch(comm, [=]() {
        return cudaMemcpyAsync(plannerStatus, statusDev, sizeof(int32_t), cudaMemcpyDeviceToDevice, cs) == cudaSuccess ? TILEXR_SUCCESS : TILEXR_ERROR_MKIRT;
    });
}

} // extern "C"
