// Expert-parallel MoE dispatch and combine ("memory" full-mesh route of the reference,
// src/include/tilexr_ep.h:25-69), as single fused kernels over NVLink peer windows.
//
// Dispatch sends every (token, k) route to the rank that owns the chosen expert and returns
// the received rows grouped local-expert-major, then by source rank, in source order:
//   expandXOut[row]          the token row (input dtype, or fp8 e4m3 when quantMode = FP8_1X128)
//   dynamicScalesOut[row]    h/128 fp32 dequantisation scales of that row (quantised modes)
//   assistInfoForCombineOut  4 x int32 per row: {srcRank, tokenIdx, k, expertId}
//   expertTokenNumsOut[e]    rows of local expert e (count, or inclusive prefix sum)
//   sendCountsOut[e*R + s]   running row count in (local expert, source rank) order
// Combine sends each processed row back to its source, where the K rows of a token are summed
// in k order in fp32 with the gate weights and rounded once (the reference's fixed order,
// tests/ep/demo/tilexr_ep_dispatch_demo.cpp:986-1047).
//
// The *Fused entry points take raw gate logits and do the routing (softmax or sigmoid scores,
// top-k, optional renormalisation) inside the dispatch kernel.
#ifndef TILEXR_EP_H
#define TILEXR_EP_H

#include "tilexr_api.h"
#include "tilexr_types.h"

#ifdef __cplusplus
namespace TileXREp {
#endif
enum TileXREpActiveMaskType {
    TILEXR_EP_ACTIVE_MASK_NONE = 0,
    TILEXR_EP_ACTIVE_MASK_TOKEN = 1,    // bool[bs]
    TILEXR_EP_ACTIVE_MASK_EXPERT = 2,   // bool[bs, topK]
};
enum TileXREpQuantMode {
    TILEXR_EP_QUANT_NONE = 0,
    TILEXR_EP_QUANT_STATIC_INT8 = 1,     // q = rint(x * scales[expert]) saturated to int8; `scales` [moeExpertNum, h] required
    TILEXR_EP_QUANT_DYNAMIC_INT8 = 2,    // per row: scale = amax(x * scales[expert]) / 127 -> dynamicScalesOut[row] (fp32), q = rint(x / scale)
    TILEXR_EP_QUANT_MXFP8_E5M2 = 3,      // fused: 1x32 blocks with E8M0 exponent bytes (dynamicScalesOut is [rows, h/32] uint8)
    TILEXR_EP_QUANT_MXFP8_E4M3 = 4,      // fused, the reference's production quantisation (quantMode 4)
    TILEXR_EP_QUANT_FP8_1X128 = 5,       // e4m3 with one fp32 scale per 128 elements
};
enum TileXREpScoreFunc { TILEXR_EP_SCORE_SOFTMAX = 0, TILEXR_EP_SCORE_SIGMOID = 1 };
enum TileXREpTokenNumsType { TILEXR_EP_TOKEN_NUMS_PREFIX = 0, TILEXR_EP_TOKEN_NUMS_COUNT = 1 };
#ifdef __cplusplus
} // namespace TileXREp
extern "C" {
#define TXR_DT TileXR::TileXRDataType
#else
#define TXR_DT enum TileXRDataType
#endif

// Everything a fused dispatch needs; zero-initialise, then fill.
typedef struct TileXREpDispatchParams {
    const void *x;                 // [bs, h] fp16/bf16
    const int32_t *expertIds;      // [bs, topK], or null when gateLogits is given
    const float *gateLogits;       // [bs, moeExpertNum] fp32, or null
    const float *selectionBias;    // [moeExpertNum] added to the score for selection only, or null
    const bool *xActiveMask;       // per activeMaskType, or null
    int64_t activeMaskType;
    int64_t bs, h, topK, moeExpertNum;
    int64_t quantMode;             // NONE or FP8_1X128
    int64_t scoreFunc;             // TileXREpScoreFunc (fused routing)
    int64_t renormalize;           // divide the top-k scores by their sum
    float routedScalingFactor;     // multiplies the gate weights (0 is read as 1)
    int64_t expertTokenNumsType;
    int64_t maxRecvRows;           // rows expandXOut can hold; the SAME value on every rank (peers place rows by it)
    // outputs
    int32_t *topkIdsOut;           // [bs, topK]  (fused routing; may be null otherwise)
    float *topkWeightsOut;         // [bs, topK]  (fused routing)
    void *expandXOut;              // [maxRecvRows, h]
    float *dynamicScalesOut;       // FP8_1X128: [maxRecvRows, h/128] fp32; MXFP8: [maxRecvRows, h/32] bytes behind this pointer
    int32_t *assistInfoForCombineOut;   // [maxRecvRows, 4]
    int64_t *expertTokenNumsOut;   // [moeExpertNum / R]
    int32_t *sendCountsOut;        // [moeExpertNum / R * R]
    int32_t *recvTotalOut;         // [1] rows received; may be null
    TXR_DT dtype;                  // dtype of x
    int32_t *routeRowsOut;         // [bs, topK] row of each route at its destination rank (-1 = inactive); may be null
    // Gate weights travel with the rows (the reference's expertScales / expandScalesOut pair,
    // src/include/tilexr_ep.h:47-52).  With fused routing the kernel's own weights are used and
    // expertScales is ignored.
    const float *expertScales;     // [bs, topK] fp32, or null
    float *expandScalesOut;        // [maxRecvRows] weight of each received row, or null
    // dedup != 0: a token with several experts on one REMOTE rank crosses NVLink once; the receiving rank
    // copies the row to the other experts' positions.  Needs weights (fused routing or expertScales) and
    // assistExtOut; the matching combine must get the same flag.
    int64_t dedup;
    int32_t *assistExtOut;         // [maxRecvRows, 2] {link, weight bits} for combine; needed when dedup != 0
    const float *scales;           // int8 modes: [moeExpertNum, h] fp32 smoothing scales (required for static, optional for dynamic)
    // Shared experts on dedicated ranks: the first sharedExpertRankNum ranks hold them (shared expert g on
    // sharedExpertRankNum / sharedExpertNum of them), the other ranks hold moeExpertNum / (R - sharedExpertRankNum)
    // routed experts each.  Every active token then has topK + sharedExpertNum routes; shared routes use slot
    // topK + g and weight 1.  Per-rank outputs have one entry per expert the rank holds.
    int64_t sharedExpertNum;
    int64_t sharedExpertRankNum;
    // Tensor parallelism inside expert parallelism (0 or 1 = none).  With tpWorldSize = T > 1 the ranks form R / T
    // groups of T consecutive ranks that hold the same moeExpertNum / (R / T) experts (each a slice of their weights);
    // tpRankId must be rank % T.  Every route is delivered to all T ranks of its expert's group, in one hop.  The
    // per-route outputs and inputs then have T entries per route, slot k * T + l for lane l: routeRowsOut and the k
    // field of the assist tuples use these slots, and the expert field holds the lane expert
    // ((group * T + l) * expertsPerGroup + local expert).  expertTokenNumsOut has one entry per expert of the group,
    // sendCountsOut expertsPerGroup * R.  tpRecvCountsOut [T] (required) receives the rows that came from the ranks
    // of each lane.  Needs explicit expertIds, no shared-expert ranks, and topK * T <= 32.
    int64_t tpWorldSize;
    int64_t tpRankId;
    int32_t *tpRecvCountsOut;
} TileXREpDispatchParams;

typedef struct TileXREpCombineParams {
    const void *expertOut;         // [rows, h], dtype
    const int32_t *assistInfoForCombine;   // [rows, 4] from dispatch
    const int32_t *sendCounts;     // from dispatch (its last entry is the row count)
    const int32_t *expertIds;      // [bs, topK] of THIS rank's tokens (negative = inactive route), or null = all active
    const float *expertScales;     // [bs, topK] gate weights; null = 1
    const bool *xActiveMask;
    int64_t activeMaskType;
    const void *sharedExpertX;     // [bs, h] added with weight 1, or null
    int64_t bs, h, topK, moeExpertNum;
    void *yOut;                    // [bs, h]
    TXR_DT dtype;
    // [bs, topK] from dispatch, or null.  With it (and expertIds) the routes whose expert lives on this rank
    // are read straight from expertOut: they take no staging copy and no flag.
    const int32_t *routeRows;
    // dedup != 0 (dispatch ran with dedup): the rows of one token on this rank are summed with their gate
    // weights here and cross NVLink once; needs assistExt from dispatch and expertIds.
    int64_t dedup;
    const int32_t *assistExt;      // [rows, 2] from dispatch
    int64_t sharedExpertNum;       // as given to dispatch
    int64_t sharedExpertRankNum;
    // As given to dispatch.  With tpWorldSize = T > 1 every rank of a group returns its partial output of each row and
    // the origin adds the T of them: y = sum_k w[k] * sum_l partial(k, l).  expertIds, expertScales and an
    // expert-type mask stay [bs, topK]; routeRows is dispatch's [bs, topK * T].
    int64_t tpWorldSize;
    int64_t tpRankId;
} TileXREpCombineParams;

int TileXRMoeEpDispatchFused(const TileXREpDispatchParams *params, TileXRCommPtr comm, TileXRStream stream);
// Sizes of the two parameter structs as the library was compiled, (dispatch << 32) | combine.  A caller built
// against other headers compares it with TILEXR_EP_ABI_STAMP before its first call.
uint64_t TileXREpAbiStamp(void);
#define TILEXR_EP_ABI_STAMP (((uint64_t)sizeof(TileXREpDispatchParams) << 32) | (uint64_t)sizeof(TileXREpCombineParams))
int TileXRMoeEpCombineFused(const TileXREpCombineParams *params, TileXRCommPtr comm, TileXRStream stream);

// Bytes of window each half must offer for a dispatch / combine of this shape (0 on bad shape).
uint64_t TileXREpDispatchWindowBytes(int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, int64_t rankSize,
                                     int64_t maxRecvRows, int64_t quantMode, int64_t elemSize, int64_t grid, int zeroCopy);
uint64_t TileXREpCombineWindowBytes(int64_t bs, int64_t h, int64_t topK, int64_t elemSize);

// ---- reference-shaped entry points (src/include/tilexr_ep.h:25-69) -----------------------------------
int TileXRMoeEpDispatchMemory(void *x, int32_t *expertIds, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK,
                              int64_t moeExpertNum, void *expandXOut, int64_t *expertTokenNumsOut, int32_t *sendCountsOut,
                              int32_t *assistInfoForCombineOut, TXR_DT dtype, TileXRStream stream);
int TileXRMoeEpDispatch(void *x, int32_t *expertIds, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK,
                        int64_t moeExpertNum, void *expandXOut, int64_t *expertTokenNumsOut, int32_t *epRecvCountsOut,
                        int32_t *assistInfoForCombineOut, TXR_DT dtype, TileXRStream stream);
int TileXRMoeEpCombineMemory(void *expertOut, int32_t *assistInfoForCombine, int32_t *epRecvCounts, TileXRCommPtr comm,
                             int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, void *yOut, TXR_DT dtype,
                             TileXRStream stream);
int TileXRMoeEpCombine(void *expertOut, int32_t *assistInfoForCombine, int32_t *epRecvCounts, TileXRCommPtr comm,
                       int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, void *yOut, TXR_DT dtype,
                       TileXRStream stream);
int TileXRMoeEpCombineV2(void *expertOut, int32_t *assistInfoForCombine, int32_t *epRecvCounts, TileXRCommPtr comm,
                         int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, void *yOut, void *workspace,
                         TXR_DT dtype, TileXRStream stream);
int TileXRMoeEpDispatchMemoryV2(void *x, int32_t *expertIds, void *scales, bool *xActiveMask, int64_t activeMaskType,
                                void *expertScales, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK,
                                int64_t moeExpertNum, int64_t epWorldSize, int64_t epRankId, int64_t tpWorldSize,
                                int64_t tpRankId, int64_t expertShardType, int64_t sharedExpertNum,
                                int64_t sharedExpertRankNum, int64_t quantMode, int64_t globalBs,
                                int64_t expertTokenNumsType, void *expandXOut, void *dynamicScalesOut,
                                int32_t *assistInfoForCombineOut, int64_t *expertTokenNumsOut, int32_t *sendCountsOut,
                                int32_t *tpRecvCountsOut, void *expandScalesOut, TXR_DT dtype, TXR_DT expandXOutDtype,
                                TileXRStream stream);
int TileXRMoeEpDispatchV2(void *x, int32_t *expertIds, void *scales, bool *xActiveMask, void *expertScales,
                          TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum,
                          int64_t epWorldSize, int64_t epRankId, int64_t tpWorldSize, int64_t tpRankId,
                          int64_t expertShardType, int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t quantMode,
                          int64_t globalBs, int64_t expertTokenNumsType, void *expandXOut, void *dynamicScalesOut,
                          int32_t *assistInfoForCombineOut, int64_t *expertTokenNumsOut, int32_t *epRecvCountsOut,
                          int32_t *tpRecvCountsOut, void *expandScalesOut, void *workspace, TXR_DT dtype,
                          TileXRStream stream);
int TileXRMoeEpCombineMemoryV2(void *expertOut, int32_t *assistInfoForCombine, int32_t *sendCounts, float *expertScales,
                               bool *xActiveMask, int64_t activeMaskType, void *sharedExpertX, TileXRCommPtr comm,
                               int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, int64_t epWorldSize,
                               int64_t epRankId, int64_t tpWorldSize, int64_t tpRankId, int64_t expertShardType,
                               int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t quantMode, int64_t globalBs,
                               void *yOut, TXR_DT dtype, TileXRStream stream);

// ---- stand-alone hot ops -------------------------------------------------------------------------------
// Routing: scores (softmax / sigmoid) -> top-k ids and gate weights.  Local kernel, no communicator.
int TileXRMoeRoutingTopK(const float *gateLogits, const float *selectionBias, int64_t bs, int64_t moeExpertNum,
                         int64_t topK, int64_t scoreFunc, int64_t renormalize, float routedScalingFactor,
                         int32_t *topkIdsOut, float *topkWeightsOut, TileXRStream stream);
// Block-scaled fp8: y = e4m3(x / s), s = max(amax over 128 elements, 1e-4) / 448, scales fp32 [rows, h/128].
int TileXRFp8Quant1x128(const void *x, int64_t rows, int64_t h, TXR_DT dtype, void *yOut, float *scalesOut,
                        TileXRStream stream);
int TileXRFp8Dequant1x128(const void *y, const float *scales, int64_t rows, int64_t h, TXR_DT dtype, void *xOut,
                          TileXRStream stream);
// MXFP8 (OCP microscaling): 32-element blocks, shared E8M0 exponent, e4m3 or e5m2 elements
// (reference: src/ep/kernels/tilexr_ep_mxfp8_quant.h:36-105).  scalesOut uint8 [rows, ceil(h/32)].
int TileXRMxfp8Quant(const void *x, int64_t rows, int64_t h, TXR_DT dtype, TXR_DT fp8Type, void *yOut, uint8_t *scalesOut,
                     TileXRStream stream);
int TileXRMxfp8Dequant(const void *y, const uint8_t *scales, int64_t rows, int64_t h, TXR_DT fp8Type, TXR_DT dtype,
                       void *xOut, TileXRStream stream);
// RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gamma, optionally x += residual first (and the sum is written back).
int TileXRRmsNorm(const void *x, void *residualInOut, const void *gamma, float eps, int64_t rows, int64_t h, TXR_DT dtype,
                  void *yOut, TileXRStream stream);

#ifdef __cplusplus
}
#endif
#undef TXR_DT

#endif // TILEXR_EP_H
