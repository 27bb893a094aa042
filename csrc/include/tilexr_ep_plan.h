// MoonEP planner, second generation: a topology- and priority-aware balance plan with duplicate-route encoding.
//
// Every rank holds s tokens with topK routes each (cap = s * topK routes) and E / R "home" experts.  The plan moves
// whole expert shares from overloaded ranks to underloaded ones until every rank computes exactly `cap` routes:
// first inside a server (cardsPerServer consecutive global rank ids), then across servers, where a receiver only
// considers the crossCandidateCount senders closest to it (XOR distance of global rank ids).  A rank that computes
// a foreign expert needs that expert's weights in one of its `prefetchSlots` slots.  Outputs, per rank:
//   dst[cap]            destination of each route: dstRank * nvS + row; a route whose token already has an earlier
//                       route to the same rank is stored as ~raw (the hidden state travels once)
//   cuSeqlens[E + B]    padded end row of each group: experts 0..E-1 (computed here, not from a slot), then slots
//   expertsToCopy[B]    foreign experts in this rank's slots (-1 = free)
//   remoteStats[2]      {foreign experts here, slots on other ranks that hold experts of this rank}
//   remoteExperts[R,B]  every rank's slots;  expertTargets[E/R, ceil(R/64)] bitmap of ranks that copy each home expert
//   status[8]           {status, intra rounds, inter rounds, total deficit, max remote, local end row, expert moves,
//                        local segments}
// All ranks run the same deterministic algorithm on the same histograms, so no plan data is exchanged; the kernel
// exchanges a header hash, each rank's own histogram row (checked against the caller's table) and the final status
// through the communicator's windows, with bounded waits, and every rank returns the same status.
//
// Counterpart of the reference's src/include/tilexr_ep_plan.h:11-147 and
// src/moonep/planner_v2/common/ep_plan_algorithm_impl.h; the algorithm source here is
// csrc/moonep/plan_v2_algorithm.h, compiled for host (CPU oracle) and device (kernel) alike.
#ifndef TILEXR_EP_PLAN_H
#define TILEXR_EP_PLAN_H

#include <stdint.h>

#include "tilexr_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct TileXRMoonEPPlanConfig {
    int64_t prefetchSlots;
    int64_t rankTokenCapacity;        // must equal s * topK
    int64_t nvS;                      // rows per rank, >= rankTokenCapacity
    int64_t tokenPadding;
    int64_t tokenRouteLimitPerPair;   // 0 = unlimited
    int32_t cardsPerServer;           // 8
    int32_t cardsPerCabinet;          // 64
    int32_t crossCandidateCount;      // 3
    int32_t reserved;
} TileXRMoonEPPlanConfig;

#define TILEXR_MOONEP_PLAN_METADATA_V2_ABI_VERSION 2u
#define TILEXR_MOONEP_INVALID_GLOBAL_TOKEN_ID UINT64_MAX
#define TILEXR_MOONEP_PLAN_STATUS_WORDS 8
#define TILEXR_MOONEP_PLAN_CARDS_PER_SERVER 8
#define TILEXR_MOONEP_PLAN_CARDS_PER_CABINET 64
#define TILEXR_MOONEP_PLAN_CROSS_CANDIDATES 3

// Counts are element counts.  tokenRemap-style tables of the later stages are not filled by the planner.
typedef struct TileXRMoonEPPlanMetadataV2 {
    uint32_t structSize;
    uint32_t abiVersion;
    int32_t *dst;            uint64_t dstCount;             // s * k
    int32_t *cuSeqlens;      uint64_t cuSeqlensCount;       // e + b
    int32_t *remoteExperts;  uint64_t remoteExpertsCount;   // r * b
    uint64_t *expertTargets; uint64_t expertTargetsCount;   // e / r * ceil(r / 64)
    int32_t *remoteStats;    uint64_t remoteStatsCount;     // 2
    int32_t *status;         uint64_t statusCount;          // 8
    int32_t *dupGroups;      uint64_t dupGroupsCount;       // nvS * 3   (filled by the receiving side, see below)
    int32_t *dupLoffs;       uint64_t dupLoffsCount;        // nvS
    int32_t *dupCounts;      uint64_t dupCountsCount;       // 2
    int64_t s, k, r, e, b, nvS;
    uint64_t epoch;
} TileXRMoonEPPlanMetadataV2;

typedef struct TileXRMoonEPPlanDesc {
    int32_t *dst;
    int32_t *cuSeqlens;
    int32_t *expertsToCopy;
    int32_t *remoteStats;
    int32_t *dupGroups;
    int32_t *dupLoffs;
    int32_t *dupCounts;
    int32_t *status;
    int64_t s, k, r, e, b, cap, nvS, tokenPadding;
    uint64_t epoch;
} TileXRMoonEPPlanDesc;

typedef enum TileXRMoonEPPlanStatus {
    PLAN_OK = 0,
    PLAN_PARTIAL_NO_FEASIBLE_PAIR = 1,
    PLAN_PARTIAL_PREFETCH_SLOT_EXHAUSTED = 2,
    PLAN_PARTIAL_TOKEN_SUPPLY = 3,
    PLAN_ERROR_CONFIG_MISMATCH = 4,
    PLAN_ERROR_TPE_MISMATCH = 5,
    PLAN_ERROR_LAYOUT_EXCEEDS_NVS = 6,
    PLAN_ERROR_MOVE_RECORD_OVERFLOW = 7,
    PLAN_ERROR_INTERNAL_INVARIANT = 8
} TileXRMoonEPPlanStatus;

typedef struct TileXRMoonEPRouteTarget {
    int32_t rawDst, dstRank, recvSlot, sendHidden, writeRouteWeight;
} TileXRMoonEPRouteTarget;

typedef struct TileXRMoonEPRouteDescriptor {
    int32_t srcRank, tokenId, topKId;
    uint64_t globalTokenId;
    int32_t rawDst, dstRank, recvSlot, sendHidden, writeRouteWeight;
} TileXRMoonEPRouteDescriptor;

typedef struct TileXRMoonEPReceivedRoute {
    int32_t srcRank, tokenId, topKId, recvSlot, isPrimary;
} TileXRMoonEPReceivedRoute;

// ---- helpers shared by planner, dispatch and combine (host) ---------------------------------------------------
// globalTokenId = (srcRank * s + tokenId) * topK + topKId.
int TileXRMoonEPEncodeGlobalTokenId(int32_t srcRank, int32_t tokenId, int32_t topKId, int64_t rankSize, int64_t s, int64_t topK,
                                    uint64_t *globalTokenId);
int TileXRMoonEPDecodeGlobalTokenId(uint64_t globalTokenId, int64_t rankSize, int64_t s, int64_t topK, int32_t *srcRank,
                                    int32_t *tokenId, int32_t *topKId);
// encoded >= 0: raw, the hidden state is sent; encoded < 0: raw = ~encoded, only the route weight is written.
int TileXRMoonEPDecodeDst(int32_t encoded, int64_t nvS, int64_t rankSize, TileXRMoonEPRouteTarget *target);
int TileXRMoonEPBuildRouteDescriptor(int32_t srcRank, int32_t tokenId, int32_t topKId, int32_t encodedDst, int64_t rankSize,
                                     int64_t s, int64_t topK, int64_t nvS, TileXRMoonEPRouteDescriptor *descriptor);
// Owner-side bitmap from the destination-side slot table.
int TileXRMoonEPBuildExpertTargets(const int32_t *remoteExperts, int64_t rankSize, int64_t expertNum, int64_t prefetchSlots,
                                   int32_t ownerRank, uint64_t *expertTargets, uint64_t expertTargetsCount);
// Receiving side: groups the rows of one token on this rank.  dupGroups[g] = {primary row, first index into dupLoffs,
// number of duplicates}; dupLoffs lists the duplicate rows in topK order; dupCounts = {groups, duplicates}.
int TileXRMoonEPBuildDuplicateMetadata(const TileXRMoonEPReceivedRoute *records, int64_t recordCount, int64_t rankSize, int64_t s,
                                       int64_t topK, int64_t nvS, int32_t *dupGroups, int32_t *dupLoffs, int32_t *dupCounts);

// ---- planner ------------------------------------------------------------------------------------------------------
// localWorkspaceBytes: device memory for the algorithm's tables.  registeredMetaBytes is 0: the exchange between the
// ranks goes through the communicator's own windows, no caller-registered memory is needed.
int TileXRMoeEpPlanV2GetWorkspaceSize(int64_t rankSize, int64_t s, int64_t topK, int64_t expertNum,
                                      const TileXRMoonEPPlanConfig *config, uint64_t *localWorkspaceBytes,
                                      uint64_t *registeredMetaBytes);

// topkExperts [s, topK], tokensPerExpert [R, E] (every rank's histogram, as all-gathered by the caller) and
// globalRankIds [R] (distinct, non-negative) are device pointers; so are the plan's output tables.
int TileXRMoeEpPlanV2(const int32_t *topkExperts, const int32_t *tokensPerExpert, const int32_t *globalRankIds, TileXRCommPtr comm,
                      int64_t s, int64_t topK, int64_t expertNum, const TileXRMoonEPPlanConfig *config, TileXRMoonEPPlanDesc *plan,
                      void *localWorkspace, uint64_t localWorkspaceBytes, void *registeredMetaWorkspace,
                      uint64_t registeredMetaBytes, TileXRStream stream);

int TileXRMoeEpPlanV2WithMetadata(const int32_t *topkExperts, const int32_t *tokensPerExpert, const int32_t *globalRankIds,
                                  TileXRCommPtr comm, int64_t s, int64_t topK, int64_t expertNum,
                                  const TileXRMoonEPPlanConfig *config, TileXRMoonEPPlanMetadataV2 *metadata, void *localWorkspace,
                                  uint64_t localWorkspaceBytes, void *registeredMetaWorkspace, uint64_t registeredMetaBytes,
                                  TileXRStream stream);

// The same call, which also fills the tables that this library's dispatch / combine stage kernels take
// (TileXRMoonEpPlanV1 in tilexr_moonep.h): destinations with duplicates decoded (every route carries its hidden state
// to its own row), the rows dispatch has to clear, for every row the route that fills it, and a one-word status
// (0 = usable; a partially balanced plan whose layout fits is usable).  All four are device pointers.
typedef struct TileXRMoonEPStageTables {
    int32_t *dst;             // [s * k]
    int32_t *zeroFillRanges;  // [(e + b) * 2]: {first row, number of rows} per group
    int32_t *dstLocal;        // [nvS]
    int32_t *status;          // [1]
} TileXRMoonEPStageTables;

int TileXRMoeEpPlanV2WithStageTables(const int32_t *topkExperts, const int32_t *tokensPerExpert, const int32_t *globalRankIds,
                                     TileXRCommPtr comm, int64_t s, int64_t topK, int64_t expertNum,
                                     const TileXRMoonEPPlanConfig *config, TileXRMoonEPPlanMetadataV2 *metadata,
                                     const TileXRMoonEPStageTables *stage, void *localWorkspace, uint64_t localWorkspaceBytes,
                                     TileXRStream stream);

// CPU oracle: the same algorithm source on host memory, for rank `rank` of `rankSize`.  remoteExperts and
// expertTargets may both be null.  Returns the plan status (also in status[0]).
int TileXRMoeEpPlanV2Reference(int32_t rank, int64_t rankSize, const int32_t *topkExperts, const int32_t *tokensPerExpert,
                               const int32_t *globalRankIds, int64_t s, int64_t topK, int64_t expertNum,
                               const TileXRMoonEPPlanConfig *config, int32_t *dst, int32_t *cuSeqlens, int32_t *expertsToCopy,
                               int32_t *remoteStats, int32_t *remoteExperts, uint64_t *expertTargets, int32_t *status);

#ifdef __cplusplus
}
#endif

#endif // TILEXR_EP_PLAN_H
