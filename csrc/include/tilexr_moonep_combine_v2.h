// MoonEP combine, second generation (reference API: src/include/tilexr_moonep_combine_v2.h:12-41).
//
// The expert rank sums the rows that one token has on it and sends one row per (source, token) group; see
// csrc/moonep/moonep_combine_v2.cu for the scheme and its numerics.  The caller supplies a workspace in device
// memory (any allocation of this process; nothing in it is read by peers) that holds the group index, the
// per-block profile records (tilexr_moonep_trace.h) and, for the workspace-resident form, the input and the two
// output regions.
#ifndef TILEXR_MOONEP_COMBINE_V2_H
#define TILEXR_MOONEP_COMBINE_V2_H

#include <stdint.h>

#include "tilexr_moonep.h"

#ifdef __cplusplus
extern "C" {
#endif

// Size of the workspace for [bs, h] tokens with topK routes and nvS rows per rank, and where inside it the profile
// records ([TILEXR_MOONEP_COMBINE_PROFILE_MAX_BLOCKS] TileXRMoonEpCombineProfileRecord) and the two output regions
// of TileXRMoonEpCombineV2 lie.  The input region of that form starts at offset 0.
int TileXRMoonEpCombineGetWorkspaceSizeV2(int64_t bs, int64_t h, int64_t topK, int64_t nvS, uint32_t dtype, uint64_t *workspaceBytes,
                                          uint64_t *profileOffset, uint64_t *outputEpoch0Offset, uint64_t *outputEpoch1Offset);

// Rows in the workspace's input region, result in one of its two output regions (they alternate from call to call);
// *activeOutputOffset says which.  aivCoreNum is accepted for source compatibility and ignored.
int TileXRMoonEpCombineV2(void *registeredWorkspace, const int32_t *dstLocal, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK, int64_t nvS,
                          uint32_t aivCoreNum, uint64_t *activeOutputOffset, uint32_t dtype, TileXRStream stream);

// hiddenSh [bs, h] = per token the sum of its topK processed rows; routeWeightsSk [bs, topK] (optional) = the weights
// that travelled with the rows.  dstLocal int32 [nvS]: srcRank * (bs * topK) + route of the row in that slot, or negative.
int TileXRMoonEpCombineStageV2(void *registeredWorkspace, uint64_t registeredWorkspaceBytes, const int32_t *dstLocal, TileXRCommPtr comm,
                               int64_t bs, int64_t h, int64_t topK, int64_t nvS, uint32_t aivCoreNum, const void *hiddenNvsh, void *hiddenSh,
                               const float *routeWeightsNvs, float *routeWeightsSk, uint32_t dtype, TileXRStream stream);

// The same with the reference's second communicator for the weights (checked to describe the same ranks, otherwise unused:
// weights and rows travel in one kernel here).
int TileXRMoonEpCombineStageV2Fused(void *registeredWorkspace, uint64_t registeredWorkspaceBytes, const int32_t *dstLocal, TileXRCommPtr comm,
                                    TileXRCommPtr weightMemoryComm, int64_t bs, int64_t h, int64_t topK, int64_t nvS, uint32_t aivCoreNum,
                                    const void *hiddenNvsh, void *hiddenSh, const float *routeWeightsNvs, float *routeWeightsSk, uint32_t dtype,
                                    TileXRStream stream);

#ifdef __cplusplus
}
#endif

#endif // TILEXR_MOONEP_COMBINE_V2_H
