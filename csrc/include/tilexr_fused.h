// Compute fused with communication: tensor-parallel building blocks.
//
//   TileXRAllReduceRmsNorm   y = RMSNorm(all_reduce(x) + residual) * gamma, residual updated in
//                            place; one-shot or two-shot chosen by size (decode / prefill).
//   TileXRAllGatherMatmul    C = all_gather(A) x B^T on tcgen05 tensor cores; A shards are pushed
//                            into every rank's staging buffer tile by tile and each GEMM tile
//                            starts as soon as the rows it needs have landed.
//   TileXRMatmulReduceScatter  C_rank = reduce_scatter(A x B^T); partial tiles are pushed to the
//                            owner from the GEMM epilogue and summed there in rank order.
//   TileXRMatmul             the same tcgen05 GEMM without communication.
//
// The reference only keeps the operator ids of the last three (src/include/tilexr_types.h:108-125,
// the kernels were removed from it); the all-reduce it ships is unfused
// (src/collectives/kernels/allreduce_*.h).
#ifndef TILEXR_FUSED_H
#define TILEXR_FUSED_H

#include "tilexr_api.h"
#include "tilexr_types.h"

#ifdef __cplusplus
extern "C" {
#define TXR_DT TileXR::TileXRDataType
#else
#define TXR_DT enum TileXRDataType
#endif

enum TileXRAllReduceAlgo { TILEXR_AR_AUTO = 0, TILEXR_AR_ONE_SHOT = 1, TILEXR_AR_TWO_SHOT = 2 };

// x [rows, h] holds this rank's partial sums.  residualInOut [rows, h] may be null (no residual
// add).  yOut and residualInOut are complete on every rank when the kernel finishes.  If both
// live in registered memory at the same offset on every rank, the two-shot path writes them
// directly.  fp16 / bf16, h a multiple of 8 up to 16384.
int TileXRAllReduceRmsNorm(const void *x, void *residualInOut, const void *gamma, float eps, int64_t rows, int64_t h,
                           TXR_DT dtype, void *yOut, int algo, TileXRCommPtr comm, TileXRStream stream);

// C[M,N] = A[M,K] x B[N,K]^T on tcgen05 tensor cores; fp16 or bf16, K and N multiples of 8,
// all pointers 16-byte aligned.  `status` (device int32, may be null) is set non-zero if a
// pipeline wait inside the kernel gave up.
int TileXRMatmul(const void *a, const void *b, void *c, int64_t m, int64_t n, int64_t k, TXR_DT dtype, int32_t *status,
                 TileXRStream stream);

// Grouped GEMM (the expert FFN of a MoE layer): the rows of A [maxRows, K] are grouped -- groupRows[0] rows of
// group 0, then groupRows[1] rows of group 1, ... -- and group g is multiplied with its own weight
// B[g] ([groups, N, K] contiguous): C[row] = A[row] x B[g(row)]^T.  groupRows is a DEVICE array of int64 (e.g. the
// expertTokenNums output of dispatch): nothing is read back to the host, and the tile list is built inside the
// kernel.  Rows at and past the sum of the counts are not written.  Same type and alignment rules as TileXRMatmul.
// epilogue 0 stores the product, C [maxRows, N].  epilogue 1 (TILEXR_GEMM_EPILOGUE_SWIGLU) takes weight row 2i as
// gate row i and row 2i+1 as up row i and stores silu(gate) * up, C [maxRows, N / 2]: the first GEMM of a SwiGLU
// feed-forward with its activation, without the [rows, N] intermediate.
#define TILEXR_GEMM_EPILOGUE_STORE 0
#define TILEXR_GEMM_EPILOGUE_SWIGLU 1
int TileXRGroupedMatmul(const void *a, const void *b, const int64_t *groupRows, void *c, int64_t maxRows, int64_t n, int64_t k,
                        int64_t groups, TXR_DT dtype, int epilogue, int32_t *status, TileXRStream stream);

// C = alpha * A x B^T with fp8 operands (e4m3 or e5m2, both the same type; K a multiple of 16) and fp32 accumulation on
// the 8-bit tensor-core path (tcgen05.mma kind::f8f6f4, twice the rate of 16-bit operands); C is fp16 or bf16.  `alpha`
// is the product of the operands' per-tensor dequantisation scales.
int TileXRMatmulFp8(const void *a, const void *b, void *c, int64_t m, int64_t n, int64_t k, TXR_DT inDtype, TXR_DT outDtype,
                    float alpha, int32_t *status, TileXRStream stream);

// Block-scaled fp8: C[m, n] = sum over 128-wide blocks kb of K of scaleA[m, kb] * scaleB[n / 128, kb] * (A x B^T restricted to
// kb).  A [M, K] and B [N, K] are e4m3 or e5m2, scaleA is [M, K/128] fp32 (one scale per row and block: the layout the
// expert-parallel dispatch emits), scaleB is [ceil(N/128), K/128] fp32 (one scale per 128 x 128 block of the weight).
// K a multiple of 128.  The tensor cores form each block's product exactly in fp32; CUDA cores fold the blocks
// together with their scales while the next block is being multiplied.
int TileXRMatmulFp8BlockScaled(const void *a, const float *scaleA, const void *b, const float *scaleB, void *c, int64_t m, int64_t n,
                               int64_t k, TXR_DT inDtype, TXR_DT outDtype, int32_t *status, TileXRStream stream);

// The block-scaled fp8 GEMM fused with the collectives of a tensor-parallel layer (same scale layouts as above; rows per
// rank a multiple of 256).
//   AllGather: A = all_gather(aShard) along rows, with its scales; aStaging [R * shardRows, K] (8-bit) and scaleStaging
//   [R * shardRows, K / 128] (fp32) are registered buffers (TileXRSymmAlloc) that every rank fills on every other rank while
//   the tiles are computed; K a multiple of 512.  C [R * shardRows, N].
//   ReduceScatter: out [shardRows, N] = this rank's rows of the sum over ranks of A x B^T (A [R * shardRows, K] holds this
//   rank's K slice); partialStaging [R * shardRows, N] 16-bit, registered.  The R partial tiles are added in rank order in fp32.
int TileXRAllGatherMatmulFp8Block(const void *aShard, const float *scaleAShard, void *aStaging, float *scaleStaging, const void *b,
                                  const float *scaleB, void *c, int64_t shardRows, int64_t n, int64_t k, TXR_DT inDtype, TXR_DT outDtype,
                                  TileXRCommPtr comm, TileXRStream stream);
int TileXRMatmulReduceScatterFp8Block(const void *a, const float *scaleA, const void *b, const float *scaleB, void *partialStaging, void *out,
                                      int64_t shardRows, int64_t n, int64_t k, TXR_DT inDtype, TXR_DT outDtype, TileXRCommPtr comm,
                                      TileXRStream stream);

// C[R*shardRows, N] = all_gather(aShard)[R*shardRows, K] x B[N,K]^T.  `aStaging` is a registered
// buffer of R*shardRows*K elements at the same offset on every rank (TileXRSymmAlloc): the
// kernel pushes aShard into every peer's staging buffer and multiplies as rows arrive.  Row
// blocks of rank r's shard occupy rows [r*shardRows, (r+1)*shardRows) of C and of the staging
// buffer.  shardRows must be a multiple of 128.
int TileXRAllGatherMatmul(const void *aShard, void *aStaging, const void *b, void *c, int64_t shardRows, int64_t n, int64_t k,
                          TXR_DT dtype, TileXRCommPtr comm, TileXRStream stream);

// out[shardRows, N] = rows [rank*shardRows, ...) of sum over ranks of A_r[R*shardRows, K_r] x B_r[N, K_r]^T.
// `partialStaging` is a registered buffer of R*shardRows*N elements at the same offset on every
// rank; partial tiles travel in the 16-bit output type and are summed in rank order in fp32.
int TileXRMatmulReduceScatter(const void *a, const void *b, void *partialStaging, void *out, int64_t shardRows, int64_t n,
                              int64_t k, TXR_DT dtype, TileXRCommPtr comm, TileXRStream stream);

// Which algorithm TILEXR_AR_AUTO picks for a message of `bytes` on `rankSize` ranks.
int TileXRAllReduceRmsNormChoose(uint64_t bytes, int rankSize);

#ifdef __cplusplus
}
#endif
#undef TXR_DT

#endif // TILEXR_FUSED_H
