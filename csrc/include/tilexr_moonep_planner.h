// MoonEP planners, direct C entry points (reference: src/include/tilexr_moonep_planner.h:13-40).
//
//   V3  the balance planner of this library's stage kernels: one cooperative kernel per rank builds the histogram, exchanges
//       it through the windows, balances and lays out (csrc/moonep/moonep_kernels.cu).
//   V2  the topology-aware planner (tilexr_ep_plan.h) behind the older call shape: one workspace, no configuration.  The
//       call plans with prefetchSlots = experts per rank, nvS = s * k rows per rank, token padding 1, no pair limit, and
//       global rank ids (rank / localRankSize) * 8 + rank % localRankSize, as the reference's compatibility entry does
//       (src/moonep/planner_v2/host/tilexr_moonep_planner.cpp:242-255, 336-417).
#ifndef TILEXR_MOONEP_PLANNER_H
#define TILEXR_MOONEP_PLANNER_H

#include <stdint.h>

#include "tilexr_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum TileXRMoonEpPlannerStatus {
    TILEXR_MOONEP_PLANNER_STATUS_SUCCESS = 0,
    TILEXR_MOONEP_PLANNER_STATUS_TIMEOUT_BASE = 1000,
} TileXRMoonEpPlannerStatus;

// workspaceBytes: device memory the V2 call needs (tables, rank ids, status words); dispatchedCapacity = s * k.
int TileXRMoonEpPlannerGetWorkspaceSizeV2(TileXRCommPtr comm, int64_t s, int64_t k, int64_t expertCount, uint64_t *workspaceBytes,
                                          int64_t *dispatchedCapacity);

// topkExpertIds int32 [s, k], tokensPerExpert int32 [R, expertCount] (every rank's histogram), outputs: dst int32 [s * k]
// (duplicates as ~raw), cuSeqlens int32 [expertCount + expertCount / R], expertsToCopy int32 [expertCount / R],
// remoteStats int32 [2], plannerStatus int32 [1] (TileXRMoonEPPlanStatus of tilexr_ep_plan.h).  All device pointers;
// `workspace` is 64-byte aligned.  `waitIterations` must be non-zero; the waits are bounded by the communicator's time
// budget (TILEXR_WAIT_TIMEOUT_MS), not by an iteration count.
int TileXRMoonEpPlannerV2(const int32_t *topkExpertIds, const int32_t *tokensPerExpert, TileXRCommPtr comm, int64_t s, int64_t k,
                          int64_t expertCount, void *workspace, uint64_t workspaceBytes, int32_t *dst, int32_t *cuSeqlens,
                          int32_t *expertsToCopy, int32_t *remoteStats, int32_t *plannerStatus, uint64_t waitIterations,
                          TileXRStream stream);

int TileXRMoonEpPlannerGetWorkspaceSizeV3(TileXRCommPtr comm, int64_t s, int64_t k, int64_t expertCount, int64_t b, int64_t tokenPadding,
                                          uint64_t *workspaceBytes, int64_t *nvS);
int TileXRMoonEpPlannerGetDstLocalOffsetV3(TileXRCommPtr comm, int64_t s, int64_t k, int64_t expertCount, int64_t b, int64_t tokenPadding,
                                           uint64_t *dstLocalOffset);
// workspace: at least ...GetWorkspaceSizeV3 bytes of device memory; dstLocal (int32 [nvS]) is written at
// ...GetDstLocalOffsetV3 inside it.
int TileXRMoonEpPlannerV3(const int32_t *topkExpertIds, const int32_t *tokensPerExpert, TileXRCommPtr comm, int64_t s, int64_t k,
                          int64_t expertCount, int64_t b, int64_t tokenPadding, void *workspace, uint64_t workspaceBytes, int32_t *dst,
                          int32_t *cuSeqlens, int32_t *expertsToCopy, int32_t *zeroFillRanges, int32_t *remoteStats, int32_t *dupCounts,
                          int32_t *plannerStatus, uint64_t waitIterations, TileXRStream stream);

#ifdef __cplusplus
}
#endif

#endif // TILEXR_MOONEP_PLANNER_H
