// MoonEP: load-balanced expert parallelism for training, in five stages.
//
//   Planning        histogram of the routes, exchange, balance plan: every rank receives exactly
//                   N = S*K rows (capacity NvS with padding); whole expert segments move off
//                   overloaded owners.  Outputs dst[N], expertsToCopy[R,B], cuSeqlens[E+B], ...
//   Dispatch        hidden rows (+ fp32 route weights) travel to slot dst[i] of their destination
//   PrefetchWeight  a destination that received tokens of a remote expert pulls that expert's
//                   weight rows from its owner into local slot E/R + b
//   Combine         processed rows travel back by dstLocal and the K rows of a token are summed
//                   in fp32 with one final rounding
//   ReduceGrad      the owner pulls the gradients accumulated in borrowed slots and adds them in
//                   ascending (source rank, slot) order
//
// The C ABI (versioned structs that start with {structSize, abiVersion}) follows the reference
// (src/include/tilexr_moonep.h:15-287) so that callers written against it keep working; only
// the stream type changes.  On B200 every stage is a kernel over NVLink peer memory: "registered
// workspace" arguments are accepted and ignored, and a tensor that lives in registered memory
// (TileXRSymmAlloc) is written by the peers directly.
#ifndef TILEXR_MOONEP_H
#define TILEXR_MOONEP_H

#include <stddef.h>
#include <stdint.h>

#include "tilexr_api.h"
#include "tilexr_moonep_planner.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TILEXR_MOONEP_ABI_VERSION_V1 UINT32_C(1)
#define TILEXR_MOONEP_ABI_VERSION_V2 UINT32_C(2)
#define TILEXR_MOONEP_MAX_TENSOR_RANK UINT32_C(4)
#define TILEXR_MOONEP_FLAG_NONE UINT64_C(0)
#define TILEXR_MOONEP_FLAG_BUILD_DEDUP (UINT64_C(1) << 0)
#define TILEXR_MOONEP_FLAG_SKIP_INTER_RANK_SYNC (UINT64_C(1) << 1)
#define TILEXR_MOONEP_FLAG_ZERO_COPY (UINT64_C(1) << 2)
#define TILEXR_MOONEP_FLAG_COMBINE_PUBLISH_ONLY (UINT64_C(1) << 3)
#define TILEXR_MOONEP_FLAG_COMBINE_CONSUME_ONLY (UINT64_C(1) << 4)
#define TILEXR_MOONEP_FLAG_RESET_STATUS (UINT64_C(1) << 5)
#define TILEXR_MOONEP_REDUCE_GRAD_DEFAULT_CHUNK_BYTES UINT64_C(8388608)
#define TILEXR_MOONEP_REDUCE_GRAD_WORKSPACE_ALIGNMENT UINT64_C(2097152)
#define TILEXR_MOONEP_MAX_TOPK 32

typedef enum TileXRMoonEpStatus {
    TILEXR_MOONEP_SUCCESS = 0,
    TILEXR_MOONEP_ERROR_INVALID_ARGUMENT = -3,
    TILEXR_MOONEP_ERROR_INTERNAL = -4,
    TILEXR_MOONEP_ERROR_NOT_SUPPORTED = -6
} TileXRMoonEpStatus;

typedef enum TileXRMoonEpDType {
    TILEXR_MOONEP_DTYPE_INT32 = 2,
    TILEXR_MOONEP_DTYPE_FLOAT16 = 3,
    TILEXR_MOONEP_DTYPE_FLOAT32 = 4,
    TILEXR_MOONEP_DTYPE_BFLOAT16 = 11
} TileXRMoonEpDType;

typedef enum TileXRMoonEpStage {
    TILEXR_MOONEP_STAGE_PLANNING = 1u << 0,
    TILEXR_MOONEP_STAGE_DISPATCH = 1u << 1,
    TILEXR_MOONEP_STAGE_PREFETCH_WEIGHT = 1u << 2,
    TILEXR_MOONEP_STAGE_COMBINE = 1u << 3,
    TILEXR_MOONEP_STAGE_REDUCE_GRAD = 1u << 4
} TileXRMoonEpStage;

// Value left in plan.status[0] by a stage whose bounded wait gave up: base + peer.
#define TILEXR_MOONEP_STATUS_PLANNER_TIMEOUT_BASE 1000
#define TILEXR_MOONEP_STATUS_DISPATCH_TIMEOUT_BASE 2100
#define TILEXR_MOONEP_STATUS_COMBINE_TIMEOUT_BASE 3100
#define TILEXR_MOONEP_STATUS_PREFETCH_TIMEOUT_BASE 4100
#define TILEXR_MOONEP_STATUS_REDUCE_TIMEOUT_BASE 5100
#define TILEXR_MOONEP_STATUS_LAYOUT_OVERFLOW 900

typedef struct TileXRMoonEpTensorV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    void *data;
    uint64_t elementCount;
    uint32_t dtype;
    uint32_t rank;
    int64_t shape[TILEXR_MOONEP_MAX_TENSOR_RANK];
} TileXRMoonEpTensorV1;

// n = S*K routes per rank, r ranks, e experts, b prefetch slots, nvS row capacity, k = top-k.
// dst int32[n]: dstRank*nvS + slot (a negative value ~raw marks a duplicate of an earlier
// route of the same token to the same rank; it is delivered like any other route).
typedef struct TileXRMoonEpPlanV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    int64_t n, r, e, b, nvS, k;
    void *dst;              // int32 [n]
    void *expertsToCopy;    // int32 [r, b]   expert placed in slot b of rank r, or -1
    void *zeroFillRanges;   // int32 [e+b, 2] {first row, rows} to clear after dispatch
    void *remoteStats;      // int32 [2]      {remote experts this rank needs, times this rank's experts are copied}
    void *dupGroups;        // int32 [nvS, 3] unused by the balance planner (zero counts)
    void *dupLoffs;         // int32 [nvS]
    void *dupCounts;        // int32 [2]
    void *status;           // int32 [1]      0, or a TILEXR_MOONEP_STATUS_* code
} TileXRMoonEpPlanV1;

typedef struct TileXRMoonEpPlanningArgsV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRCommPtr comm;
    const TileXRMoonEpTensorV1 *topkExperts;      // int32 [S, K]
    const TileXRMoonEpTensorV1 *tokensPerExpert;  // optional, recomputed by the kernel
    void *workspace;                              // int32 [nvS] receives dstLocal (see ...GetDstLocalOffsetV3)
    uint64_t workspaceBytes;
    TileXRMoonEpTensorV1 *cuSeqlens;              // int32 [E + B]
    TileXRMoonEpPlanV1 *plan;
    uint64_t waitIterations;                      // ignored: waits are bounded by the communicator's time budget
    uint64_t flags;
} TileXRMoonEpPlanningArgsV1;

typedef struct TileXRMoonEpDispatchTraceV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    void *buffer;
    uint64_t bufferBytes;
    uint32_t iteration, iterationCount, eventCapacity, reserved;
} TileXRMoonEpDispatchTraceV1;

typedef struct TileXRMoonEpDispatchArgsV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRCommPtr comm;
    const TileXRMoonEpPlanV1 *plan;
    const TileXRMoonEpTensorV1 *hiddenSh;         // [S, H] fp16/bf16, or fp32 for gradients
    const TileXRMoonEpTensorV1 *routeWeightsSk;   // optional fp32 [S, K]
    TileXRMoonEpTensorV1 *hiddenNvsh;             // [nvS, H]
    TileXRMoonEpTensorV1 *routeWeightsNvs;        // optional fp32 [nvS]
    uint64_t flags;
    void *registeredWorkspace;                    // accepted for compatibility, unused
    uint64_t registeredWorkspaceBytes;
    const TileXRMoonEpDispatchTraceV1 *trace;
} TileXRMoonEpDispatchArgsV1;
typedef TileXRMoonEpDispatchArgsV1 TileXRMoonEpDispatchArgsV2;

// gate / up / down: [E/R + B, rowElems] each, in registered memory at the same offset on every
// rank; rows [0, E/R) are the rank's own experts, rows E/R + b are the prefetch slots.
typedef struct TileXRMoonEpPrefetchWeightArgsV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRCommPtr comm;
    const TileXRMoonEpPlanV1 *plan;
    const TileXRMoonEpTensorV1 *gate;
    const TileXRMoonEpTensorV1 *up;
    const TileXRMoonEpTensorV1 *down;
    uint64_t flags;
} TileXRMoonEpPrefetchWeightArgsV1;

typedef struct TileXRMoonEpCombineArgsV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRCommPtr comm;
    const TileXRMoonEpPlanV1 *plan;
    const int32_t *dstLocal;                      // int32 [nvS]: srcRank*n + route, or -1
    const TileXRMoonEpTensorV1 *hiddenNvsh;
    const TileXRMoonEpTensorV1 *routeWeightsNvs;
    TileXRMoonEpTensorV1 *hiddenSh;
    TileXRMoonEpTensorV1 *routeWeightsSk;
    uint64_t flags;
} TileXRMoonEpCombineArgsV1;

typedef struct TileXRMoonEpReduceGradArgsV1 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRCommPtr comm;
    const TileXRMoonEpPlanV1 *plan;
    const TileXRMoonEpTensorV1 *input;            // fp32 [E/R + B, rowElems], registered
    TileXRMoonEpTensorV1 *output;                 // same tensor or a separate fp32 [E/R, rowElems]
    uint64_t flags;
} TileXRMoonEpReduceGradArgsV1;

typedef struct TileXRMoonEpReduceGradWorkspaceQueryV2 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRCommPtr comm;
    const TileXRMoonEpPlanV1 *plan;
    const TileXRMoonEpTensorV1 *gate;
    const TileXRMoonEpTensorV1 *up;
    const TileXRMoonEpTensorV1 *down;
    uint64_t requestedUdmaChunkBytes;
    uint64_t flags;
} TileXRMoonEpReduceGradWorkspaceQueryV2;

typedef struct TileXRMoonEpReduceGradWorkspaceInfoV2 {
    uint32_t structSize;
    uint32_t abiVersion;
    uint64_t workspaceBytes;
    uint64_t workspaceAlignment;
    uint64_t udmaChunkBytes;
    uint64_t laneStateBytes;
    uint64_t laneStateStrideBytes;
    uint64_t bankStrideBytes;
    uint64_t laneStrideBytes;
    uint64_t rowBytes[3];
    uint64_t chunkCounts[3];
    uint32_t projectionQpCounts[3];
    uint32_t qpCount;
    uint32_t blockDim;
    uint32_t reserved;
} TileXRMoonEpReduceGradWorkspaceInfoV2;

typedef struct TileXRMoonEpReduceGradSourceSliceV2 {
    void *data;
    uint64_t bytes;
    void *registrationBase;
    uint64_t registrationBytes;
} TileXRMoonEpReduceGradSourceSliceV2;

typedef void *TileXRMoonEpReduceGradPreparedV2;

typedef struct TileXRMoonEpReduceGradPrepareArgsV2 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRCommPtr comm;
    const TileXRMoonEpPlanV1 *plan;
    TileXRMoonEpTensorV1 *gate;
    TileXRMoonEpTensorV1 *up;
    TileXRMoonEpTensorV1 *down;
    TileXRMoonEpReduceGradSourceSliceV2 sources[3];
    void *workspace;
    uint64_t workspaceBytes;
    uint64_t requestedUdmaChunkBytes;
    uint64_t flags;
} TileXRMoonEpReduceGradPrepareArgsV2;

typedef struct TileXRMoonEpReduceGradArgsV2 {
    uint32_t structSize;
    uint32_t abiVersion;
    TileXRMoonEpReduceGradPreparedV2 prepared;
    const TileXRMoonEpPlanV1 *plan;
    TileXRMoonEpTensorV1 *gate;
    TileXRMoonEpTensorV1 *up;
    TileXRMoonEpTensorV1 *down;
    TileXRMoonEpReduceGradSourceSliceV2 sources[3];
    TileXRMoonEpTensorV1 *status;
    uint64_t waitIterations;
    uint64_t flags;
} TileXRMoonEpReduceGradArgsV2;

uint32_t TileXRMoonEpGetAbiVersion(void);
int TileXRMoonEpGetCapabilitiesV1(uint64_t *nativeStages, uint64_t *stubStages);
int TileXRMoonEpGetCapabilitiesV2(uint64_t *nativeStages, uint64_t *stubStages);

int TileXRMoonEpPlanningGetWorkspaceSizeV1(TileXRCommPtr comm, int64_t s, int64_t k, int64_t e, int64_t b,
                                           int64_t tokenPadding, uint64_t *workspaceBytes, int64_t *nvS);
int TileXRMoonEpPlanningV1(const TileXRMoonEpPlanningArgsV1 *args, TileXRStream stream);
int TileXRMoonEpDispatchGetWorkspaceSizeV1(TileXRCommPtr comm, int64_t s, int64_t k, int64_t h, uint32_t hiddenDtype,
                                           uint64_t *workspaceBytes, uint64_t *workspaceAlignment);
int TileXRMoonEpDispatchGetWorkspaceSizeV2(TileXRCommPtr comm, int64_t s, int64_t k, int64_t h, uint32_t hiddenDtype,
                                           uint64_t *workspaceBytes, uint64_t *workspaceAlignment);
int TileXRMoonEpDispatchV1(const TileXRMoonEpDispatchArgsV1 *args, TileXRStream stream);
int TileXRMoonEpDispatchV2(const TileXRMoonEpDispatchArgsV2 *args, TileXRStream stream);
int TileXRMoonEpPrefetchWeightV1(const TileXRMoonEpPrefetchWeightArgsV1 *args, TileXRStream stream);
int TileXRMoonEpCombineV1(const TileXRMoonEpCombineArgsV1 *args, TileXRStream stream);
int TileXRMoonEpReduceGradV1(const TileXRMoonEpReduceGradArgsV1 *args, TileXRStream stream);
int TileXRMoonEpReduceGradGetWorkspaceSizeV2(const TileXRMoonEpReduceGradWorkspaceQueryV2 *query,
                                             TileXRMoonEpReduceGradWorkspaceInfoV2 *info);
int TileXRMoonEpReduceGradPrepareV2(const TileXRMoonEpReduceGradPrepareArgsV2 *args, TileXRMoonEpReduceGradPreparedV2 *prepared);
int TileXRMoonEpReduceGradDestroyPreparedV2(TileXRMoonEpReduceGradPreparedV2 prepared);
int TileXRMoonEpReduceGradV2(const TileXRMoonEpReduceGradArgsV2 *args, TileXRStream stream);

// The planners' direct entry points (TileXRMoonEpPlannerV2 / V3 and their size queries) are in tilexr_moonep_planner.h.

// ---- CPU reference of the whole protocol (single process, all ranks) --------------------------------------
// allTopk int32 [r, s*k].  Outputs for rank `rank`; any output pointer may be null.
int TileXRMoonEpReferencePlan(int rank, int64_t r, int64_t s, int64_t k, int64_t e, int64_t b, int64_t tokenPadding,
                              const int32_t *allTopk, int32_t *dst, int32_t *cuSeqlens, int32_t *expertsToCopyAll,
                              int32_t *zeroFillRanges, int32_t *remoteStats, int64_t *nvS);

#ifdef __cplusplus
}
#endif

#endif // TILEXR_MOONEP_H
