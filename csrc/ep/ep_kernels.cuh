// Argument blocks of the expert-parallel kernels and the window layout they agree on.
#ifndef TILEXR_EP_KERNELS_CUH
#define TILEXR_EP_KERNELS_CUH

#include <stdint.h>

#include "tilexr_comm_args.h"
#include "tilexr_launch.h"

namespace TileXR {

constexpr unsigned EP_BLOCK_THREADS = 512;
constexpr unsigned EP_WARPS = EP_BLOCK_THREADS / 32;
constexpr int EP_MAX_EXPERTS = 1024;
constexpr int EP_MAX_TOPK = 32;
constexpr int EP_MAX_ROUTES_PER_BLOCK = 4096;
constexpr int EP_FP8_MAX_H = 8192;      // register-resident quantised row: 16 x 512 elements
constexpr uint32_t EP_COUNT_FLAG_SLOT = TILEXR_FLAGS_PER_PAIR - 1;   // blocks of a dispatch stay below this flag slot
// Operator scratch of the control block (64-bit words from TILEXR_CTRL_SCRATCH_WORD) as the EP kernels use it.
constexpr int EP_SCRATCH_CURSOR_WORD = 0;     // combine: two 32-bit work cursors
constexpr int EP_SCRATCH_DONE_WORD = 1;       // dispatch: 32-bit count of blocks that have finished counting
constexpr int EP_SCRATCH_BUCKET_WORD = 2;     // combine: 32-bit rows per bucket, EP_MAX_BUCKETS of them
constexpr int EP_MAX_BUCKETS = 8;
constexpr int EP_SCRATCH_TOTALS_WORD = 8;     // dispatch: 32-bit routes per column of this rank, EP_MAX_EXPERTS at most
constexpr int EP_SCRATCH_READY_WORD = 640;    // dispatch: per block, epoch of the launch whose histogram it has written

// Where a dispatch puts things inside one data half of the DESTINATION's window.  Identical
// on every rank; computed by EpDispatchLayout() on the host.
struct EpDispatchWindow {
    uint64_t payloadOff;      // [maxRecvRows][rowBytes]           (unused when zeroCopy)
    uint64_t scalesOff;       // [maxRecvRows][scaleRowBytes]
    uint64_t assistOff;       // [maxRecvRows][16]
    uint64_t extOff;          // [maxRecvRows] 8 bytes: {link, gate weight} of each row
    uint64_t blockCountOff;   // [grid][numExperts] int32, local scratch of the sender
    uint64_t totalBytes;
    uint32_t rowBytes;
    uint32_t scaleRowBytes;
};

// Which rank holds which expert.  The first `sharedRanks` ranks hold the shared experts (one each; shared expert
// g is replicated on ranksPerShared = sharedRanks / sharedExperts ranks and a token of source rank s goes to
// rank s % ranksPerShared + g * ranksPerShared), the others `moePerRank` routed experts each (reference:
// tests/ep/demo/tilexr_ep_dispatch_demo.cpp:647-661).  Counts and row placement work on COLUMNS: column c <
// sharedRanks is the shared expert held by rank c, column sharedRanks + e is routed expert e.
#if defined(__CUDACC__)
#define TXR_EP_HD __host__ __device__
#else
#define TXR_EP_HD
#endif
struct EpTopology {
    int32_t sharedRanks;
    int32_t sharedExperts;
    int32_t moePerRank;
};
TXR_EP_HD inline int EpColRank(const EpTopology &t, int col)
{
    return col < t.sharedRanks ? col : t.sharedRanks + (col - t.sharedRanks) / t.moePerRank;
}
TXR_EP_HD inline int EpRankFirstCol(const EpTopology &t, int rank)
{
    return rank < t.sharedRanks ? rank : t.sharedRanks + (rank - t.sharedRanks) * t.moePerRank;
}
TXR_EP_HD inline int EpRankCols(const EpTopology &t, int rank) { return rank < t.sharedRanks ? 1 : t.moePerRank; }
TXR_EP_HD inline int EpSharedCol(const EpTopology &t, int srcRank, int g)
{
    const int per = t.sharedRanks / t.sharedExperts;
    return srcRank % per + g * per;
}

struct EpDispatchArgs {
    const uint8_t *x;
    const int32_t *expertIds;
    const float *gateLogits;
    const float *selectionBias;
    const uint8_t *activeMask;
    int32_t *topkIdsOut;
    float *topkWeightsOut;
    uint8_t *expandXOut;
    float *dynamicScalesOut;
    int32_t *assistOut;
    int64_t *expertTokenNumsOut;
    int32_t *sendCountsOut;
    int32_t *recvTotalOut;
    CommArgs *comm;
    int64_t magic;
    EpDispatchWindow win;
    int32_t bs, h, topK, numExperts, numCols;   // numCols = sharedRanks + numExperts
    EpTopology topo;
    int32_t maskType, quantMode, scoreFunc, renormalize, tokenNumsType;
    float routedScale;
    uint32_t maxRecvRows;
    uint32_t tokensPerBlock;
    uint32_t elemSize;
    uint32_t isBf16;
    uint32_t zeroCopy;
    uint32_t outHandle;
    uint64_t outOffset;
    void *perfTrace;                 // stage profiler buffer of this launch, or null
    int32_t *routeRowsOut;           // [bs, topK] destination row per route, or null
    const float *quantScales;        // int8 modes: [numExperts, h] smoothing scales, or null
    const float *expertScales;       // [bs, topK] gate weights when routing is not fused, or null
    float *expandScalesOut;          // [maxRecvRows] or null
    int32_t *assistExtOut;           // [maxRecvRows, 2] or null
    uint32_t dedup;
};

struct EpCombineArgs {
    const uint8_t *expertOut;
    const int32_t *assist;
    const int32_t *sendCounts;       // last entry = rows to send back
    const int32_t *expertIds;
    const float *expertScales;
    const uint8_t *activeMask;
    const uint8_t *sharedExpertX;
    uint8_t *yOut;
    CommArgs *comm;
    int64_t magic;
    int32_t bs, h, topK, numExperts, numCols;
    EpTopology topo;
    int32_t maskType;
    uint32_t rowBytes;
    uint32_t isBf16;
    uint32_t sendCountEntries;
    void *perfTrace;
    const int32_t *routeRows;        // [bs, topK] from dispatch: local routes bypass the window; or null
    const int32_t *assistExt;        // [rows, 2] {link, weight bits}
    uint32_t dedup;
    // Work decomposition, the same on every rank (the flag of (slot, part) is slot * parts + part):
    uint32_t parts;                  // column ranges a row is cut into (1 unless the batch is small)
    uint32_t partVecs;               // 16-byte vectors per part, a multiple of 32
    uint32_t chunkRows;              // rows whose tuples one send item examines, a power of two <= 32
    uint32_t buckets;                // ranges of the source token index that the senders walk in order
    uint32_t bucketTokens;           // tokens per bucket
    uint32_t reducerBlocks;          // trailing blocks that only reduce
    uint32_t noSend;                 // 1: no row leaves this rank, the send items are skipped
    uint64_t listOff;                // bucket lists of travelling rows inside this rank's data half: [buckets][listCap] int32
    uint32_t listCap;                // rows a list can hold; with more rows than that the senders walk the rows unsorted
};

// link word of a row: bit 31 = the row is a follower (its payload is a copy of its group's head row);
// low bits = 1 + the next row of the same (source, token) group on this rank, 0 at the end of the chain.
constexpr uint32_t EP_LINK_FOLLOWER = 0x80000000u;
constexpr uint32_t EP_LINK_NEXT_MASK = 0x7fffffffu;

struct RoutingArgs {
    const float *gateLogits;
    const float *selectionBias;
    int32_t *topkIdsOut;
    float *topkWeightsOut;
    int32_t bs, numExperts, topK, scoreFunc, renormalize;
    float routedScale;
};

const KernelEntry &EpDispatchKernelEntry();
const KernelEntry &EpCombineKernelEntry();

// Plain (non communicating) kernels, launched directly.
int LaunchRoutingTopK(const RoutingArgs &args, void *stream);
int LaunchFp8Quant1x128(const void *x, int64_t rows, int64_t h, bool bf16, void *y, float *scales, void *stream);
int LaunchFp8Dequant1x128(const void *y, const float *scales, int64_t rows, int64_t h, bool bf16, void *x, void *stream);
int LaunchMxfp8Quant(const void *x, int64_t rows, int64_t h, bool bf16, bool e5m2, void *y, uint8_t *scales, void *stream);
int LaunchMxfp8Dequant(const void *y, const uint8_t *scales, int64_t rows, int64_t h, bool e5m2, bool bf16, void *x,
                       void *stream);
int LaunchRmsNorm(const void *x, void *residual, const void *gamma, float eps, int64_t rows, int64_t h, bool bf16, void *y,
                  void *stream);

size_t EpDispatchSmemBytes(int numExperts, int routesPerBlock);

} // namespace TileXR

#endif
