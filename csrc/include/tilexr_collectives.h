// Collectives library: all-gather, equal all-to-all, all-reduce, reduce-scatter, broadcast
// and the profile probe, issued as kernels on the caller's stream.  Same entry points as the
// reference (src/include/tilexr_collectives.h:23-40).  Differences worth knowing:
//   * all four reduce operators are implemented (the reference host accepts SUM only);
//   * all-to-all works for any rank count (the reference needs an even count on one topology);
//   * when the receive buffer lies inside a registered region (TileXRUDMARegister or
//     TileXRSymmAlloc on every rank, same offset) peers write into it directly and the
//     staging copy through the window is skipped.
#ifndef TILEXR_COLLECTIVES_H
#define TILEXR_COLLECTIVES_H

#include "tilexr_api.h"
#include "tilexr_types.h"

#ifdef __cplusplus
#define TXR_DT TileXR::TileXRDataType
#define TXR_OP TileXR::TileXRReduceOp
extern "C" {
#else
#define TXR_DT enum TileXRDataType
#define TXR_OP enum TileXRReduceOp
#endif

int TileXRAllGather(void *sendBuf, void *recvBuf, int64_t sendCount, TXR_DT dataType, TileXRCommPtr comm,
                    TileXRStream stream);
int TileXRAllToAll(void *sendBuf, void *recvBuf, int64_t sendCount /* per peer */, TXR_DT dataType, TileXRCommPtr comm,
                   TileXRStream stream);
int TileXRAllReduce(void *sendBuf, void *recvBuf, int64_t count, TXR_DT dataType, TXR_OP op, TileXRCommPtr comm,
                    TileXRStream stream);
int TileXRReduceScatter(void *sendBuf, void *recvBuf, int64_t recvCount, TXR_DT dataType, TXR_OP op, TileXRCommPtr comm,
                        TileXRStream stream);
int TileXRBroadcast(void *buf, int64_t count, TXR_DT dataType, int root, TileXRCommPtr comm, TileXRStream stream);
int TileXRProfileProbe(void *sendBuf, void *recvBuf, int64_t count, TXR_DT dataType, TileXRCommPtr comm,
                       TileXRStream stream);

// How a call would be split into launches; pure host arithmetic, exposed for tests and tools.
typedef struct TileXRCollPlanInfo {
    int32_t kind;            // CollKind
    uint32_t launches;       // kernel launches the call needs
    uint32_t tileBytes;
    uint32_t tilesPerLaunch; // tiles per (source, destination) pair in the first launch
    uint32_t producers;
    uint32_t reducers;
    uint32_t consumers;
    uint32_t grid;
    uint64_t bytesPerLaunch; // slice bytes covered by one launch
} TileXRCollPlanInfo;
int TileXRCollectivePlan(int opType, int64_t count, int dataType, int rankSize, uint64_t dataHalfBytes,
                         unsigned maxGrid, TileXRCollPlanInfo *info);

// All-to-all with transpose (the sequence-parallel <-> head-parallel exchange): sendBuf is a [rows, width] matrix
// (count = rows * width elements); rank p receives column block p of every rank's matrix, and recvBuf holds them as
// [rankSize][rows][width / rankSize].  A column block of one row is a multiple of 16 bytes.
// (Reference: TileXRAll2AllTranspose, selected when the all-to-all is called with op and root set, root = width:
// src/collectives/kernels/lccl_op.h:236-237.)
int TileXRAllToAllTranspose(void *sendBuf, void *recvBuf, int64_t count, int64_t width, TXR_DT dataType, TileXRCommPtr comm,
                            TileXRStream stream);

// All-reduce of int8 payloads with dequantisation: recvBuf[i] = sum over ranks of (sendBuf_r[i] + offset) *
// scale[i % scaleCount], fp16 or bf16 (`outType`; `scale` has that type, scaleCount 1 = one scale for all elements).
// `count` is a multiple of 16.  The first hop carries int8, the sum is formed in fp32 in rank order.
int TileXRAllReduceQuant(const void *sendBuf, void *recvBuf, int64_t count, TXR_DT outType, const void *scale,
                         int64_t scaleCount, float offset, TileXRCommPtr comm, TileXRStream stream);

// Collectives through the NVSwitch multicast object (NVLS).  `mcAddr` is the MULTICAST address of the message inside
// a symmetric buffer that every rank bound to one multicast object (the same offset on every rank); addresses
// and byte counts are multiples of 16.  Reductions run inside the switch with fp32 accumulation (bf16, fp16,
// fp32) and every rank receives bit-identical results.  Not available on emulated or host-memory communicators.
//   AllReduce       in place in the buffer: `bytes` of every rank's copy become the sum.
//   ReduceScatter   `out` (local, bytes / rankSize rounded up to 16) receives slice `rank` of the sum.
//   AllGather       `shard` (local) lands at mcAddr + rank * shardBytes in every copy.
//   Broadcast       the root's `in` (local; may be null elsewhere) lands at mcAddr in every copy.
int TileXRNvlsAllReduce(void *mcAddr, uint64_t bytes, TXR_DT dataType, TileXRCommPtr comm, TileXRStream stream);
int TileXRNvlsReduceScatter(void *mcAddr, void *out, uint64_t bytes, TXR_DT dataType, TileXRCommPtr comm, TileXRStream stream);
int TileXRNvlsAllGather(const void *shard, void *mcAddr, uint64_t shardBytes, TileXRCommPtr comm, TileXRStream stream);
int TileXRNvlsBroadcast(const void *in, void *mcAddr, uint64_t bytes, int root, TileXRCommPtr comm, TileXRStream stream);
// y = RMSNorm(sum over ranks of x + residual) * gamma and residual <- sum + residual, [rows, h] fp16 / bf16, in one
// kernel: a row's owner reduces it inside the switch, normalises it and multicasts y and the new residual.  mcX, mcY
// (may be equal) and mcResidual are multicast addresses of views at the same offset on every rank; residualLocal is
// this rank's own copy of the residual view (both null: no residual); gamma [h] is local.
int TileXRNvlsAllReduceRmsNorm(void *mcX, void *mcResidual, const void *residualLocal, const void *gamma, float eps, int64_t rows,
                               int64_t h, TXR_DT dataType, void *mcY, TileXRCommPtr comm, TileXRStream stream);

#ifdef __cplusplus
}
#endif
#undef TXR_DT
#undef TXR_OP

#endif // TILEXR_COLLECTIVES_H
