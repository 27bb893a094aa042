// CPU execution of the tile-flag protocols over a host-memory communicator
// (TileXRCommInitRankHostMemory): windows are POSIX shared memory, one process per rank, and
// the "kernels" below run on the calling thread using the very same flag / epoch / reuse-guard
// primitives as the CUDA kernels (device/tilexr_sync.cuh compiled for the host).  This is the
// no-GPU plumbing mode: it exercises bootstrap, window mapping, magic epochs, bounded waits and
// the expert-parallel placement rules between real processes.
#ifndef TILEXR_HOSTSIM_H
#define TILEXR_HOSTSIM_H

#include "tilexr_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// All-gather of `bytes` per rank in tiles of `tileBytes`, each tile announced by its own
// magic-tagged flag; consumers copy a tile as soon as its flag shows up.
int TileXRHostAllGather(const void *send, void *recv, uint64_t bytes, uint32_t tileBytes, TileXRCommPtr comm);
int TileXRHostAllReduceSumF32(const float *send, float *recv, uint64_t count, TileXRCommPtr comm);
// Equal all-to-all (slice p of `send`, `bytesPerPeer` long, becomes slice `rank` of rank p's `recv`), reduce-scatter (slice p
// of every rank's `send` summed on rank p in rank order) and broadcast from `root`, over the same tiles and flags.
int TileXRHostAllToAll(const void *send, void *recv, uint64_t bytesPerPeer, uint32_t tileBytes, TileXRCommPtr comm);
int TileXRHostReduceScatterSumF32(const float *send, float *recv, uint64_t recvCount, TileXRCommPtr comm);
int TileXRHostBroadcast(void *buf, uint64_t bytes, int root, uint32_t tileBytes, TileXRCommPtr comm);

// fp32 expert-parallel dispatch / combine with the semantics of tilexr_ep.h.
int TileXRHostEpDispatch(const float *x, const int32_t *expertIds, int64_t bs, int64_t h, int64_t topK,
                         int64_t moeExpertNum, int64_t maxRecvRows, float *expandXOut, int32_t *assistOut,
                         int64_t *expertTokenNumsOut, int32_t *sendCountsOut, int32_t *recvTotalOut, TileXRCommPtr comm);
int TileXRHostEpCombine(const float *expertOut, const int32_t *assist, int32_t rows, const int32_t *expertIds,
                        const float *expertScales, int64_t bs, int64_t h, int64_t topK, int64_t moeExpertNum, float *yOut,
                        TileXRCommPtr comm);

// MoonEP dispatch and combine by plan on fp32 rows (plan tables as in tilexr_moonep.h: dst[i] = rank * nvS + row, dstLocal[row] =
// source rank * routes + route, negative where no route fills the row).  Dispatch delivers rows and route weights and leaves zeros
// in the rows nobody fills; Combine returns every row to its source, which adds a token's topK rows in route order.
int TileXRHostMoonDispatch(const float *hidden, const float *routeWeights, const int32_t *dst, const int32_t *dstLocal, int64_t routes,
                           int64_t topK, int64_t h, int64_t nvS, float *hiddenOut, float *weightsOut, TileXRCommPtr comm);
int TileXRHostMoonCombine(const float *rows, const float *weightsNvs, const int32_t *dstLocal, const int32_t *dst, int64_t nvS, int64_t tokens,
                          int64_t topK, int64_t h, float *hiddenOut, float *weightsOut, TileXRCommPtr comm);

// Test hook: the next host kernel of this process skips raising its flags, so that peers run
// into their wait budget (failure-detection tests make the failure on the host).
int TileXRHostInjectSkipFlags(int enable);

// Protocol trace of what the host kernels above (and the flag primitives under them) do on this rank, in the event
// format of the protocol checker, one JSON object per line.  Event ids are global over the ranks of the communicator
// (one counter in rank 0's window), so the ranks' files concatenate into one trace for TileXRCheckerCheckTrace /
// `tilexr_checker --trace`.  Start and stop on the thread that runs the kernels.
int TileXRHostTraceStart(TileXRCommPtr comm, const char *path);
int TileXRHostTraceStop(TileXRCommPtr comm, uint64_t *eventCount /* may be null */);

#ifdef __cplusplus
}
#endif

#endif
