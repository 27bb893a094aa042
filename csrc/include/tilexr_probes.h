// Small kernels that exercise the device primitives directly: registered-memory put / get with
// signal (the UDMA demo and bandwidth probe of the reference, tests/udma/demo/*), the
// device-initiated local copy (tests/sdma/demo/*), and a bounded wait on a signal word.
#ifndef TILEXR_PROBES_H
#define TILEXR_PROBES_H

#include "tilexr_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Data-as-flag round trip on the low-latency plane of the windows: every rank sends `bytes` (a multiple of 4) from src to the
// next rank as 16-byte units carrying the launch epoch, and receives the previous rank's bytes into dst.  Block
// `withheldBlock` of every rank sends nothing (pass 0xffffffff for a complete exchange): the receiver's wait then runs out
// of its budget and the communicator's device status says so.
int TileXRDataAsFlagProbe(TileXRCommPtr comm, void *dst, const void *src, uint64_t bytes, uint32_t withheldBlock, uint32_t blocks,
                          TileXRStream stream);

// The reference's device verb names (device/tilexr_udma.cuh) between neighbours: every warp of the launch puts its share of
// `bytes` (a multiple of 16) from src into registered region 0 of the next rank with a signal word behind it (the words start
// at `signalOffset` of the region, 8 bytes per warp, `blocks` x 16 warps), waits for its own word and gets the share back
// from the next rank into dst.
int TileXRNamedVerbsProbe(TileXRCommPtr comm, void *dst, const void *src, uint64_t bytes, uint64_t signalOffset, uint32_t blocks,
                          TileXRStream stream);

// Every rank writes `bytes` from `localSrc` into region `handle` of rank (rank+1) % R at
// `dstOffset`; each block then adds 1 to signal word `signalIndex` of that rank and waits until
// this rank's own word reaches `expectedSignal` (blocks x number of calls so far).
// Host-side self tests of the symmetric allocator's plumbing (csrc/comm/vmm.cpp); no GPU is involved.
int TileXRVmmQuerySupport(int device, int *vmm, int *multicast);
int TileXRVmmDescriptorSelfTest(uint64_t tag, int rank, int fd, int srcRank, int kind, int *received);
int TileXRVmmDescriptorNobodyThere(uint64_t tag, int rank, int fd);

int TileXRPutSignalProbe(TileXRCommPtr comm, TileXRUDMAMemHandle handle, uint64_t dstOffset, const void *localSrc,
                         uint64_t bytes, uint32_t signalIndex, uint64_t expectedSignal, uint32_t blocks, TileXRStream stream);
// Every rank reads `bytes` of region `handle` of rank (rank+1) % R at `srcOffset` into `localDst`.
int TileXRGetProbe(TileXRCommPtr comm, TileXRUDMAMemHandle handle, uint64_t srcOffset, void *localDst, uint64_t bytes,
                   uint32_t blocks, TileXRStream stream);
// Local copy driven by one thread per block through the TMA bulk pipeline.
int TileXRLocalCopyProbe(TileXRCommPtr comm, void *dst, const void *src, uint64_t bytes, uint32_t blocks, TileXRStream stream);
// Waits (bounded by the communicator's budget) for signal word `signalIndex` to reach `value`.
// When nobody raises it the kernel gives up, records TILEXR_DEV_WAIT_TIMEOUT and returns.
int TileXRSignalWaitProbe(TileXRCommPtr comm, uint32_t signalIndex, uint64_t value, TileXRStream stream);
// Out-of-range put: the device-side registry check refuses it and reports RMA_OUT_OF_RANGE in *deviceResult.
int TileXRRangeCheckProbe(TileXRCommPtr comm, TileXRUDMAMemHandle handle, uint64_t offset, uint64_t bytes, int32_t *deviceResult,
                          TileXRStream stream);

#ifdef __cplusplus
}
#endif

#endif
