// An entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc when they need a MoE token permutation:
// an inference server that measured free memory at start-up and handed every remaining byte
// to its KV-cache pool, a plugin that runs inside another framework's step and may not disturb
// that framework's allocator, or latency-critical code for which cudaMalloc's implicit
// device-wide synchronisation is not acceptable.  The communicator-based dispatch
// (TileXRMoeEpDispatchFused) keeps its per-block counters in a window that the communicator
// allocates; this variant keeps them in a fixed array that is part of the library image, so the
// call path contains no cudaMalloc, cudaFree or allocating library routine.
//
// This function has no counterpart in the reference.
#ifndef TILEXR_NOALLOC_H
#define TILEXR_NOALLOC_H

#include <stdint.h>

#include "tilexr_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch array (about 0.5 MiB, resident on every GPU that loads the
// library until the process exits).
#define TILEXR_NOALLOC_MAX_EXPERTS 1024
#define TILEXR_NOALLOC_MAX_BLOCKS 128
#define TILEXR_NOALLOC_MAX_ROUTES (TILEXR_NOALLOC_MAX_BLOCKS * 4096)

// Single-GPU MoE dispatch: groups the bs*topK routes by expert.  Same outputs as
// TileXRMoeEpDispatchFused on a one-rank communicator with explicit expert ids and no
// quantisation:
//   expandXOut [bs*topK, h]   row of the route's token; routes ordered by expert, then (token, k)
//   assistOut  [bs*topK, 4]   {0, token, k, expert}
//   expertTokenNumsOut [moeExpertNum] int64 rows per expert
//   sendCountsOut [moeExpertNum] int32 running row count
// dtype is TILEXR_DATA_TYPE_FP16 or TILEXR_DATA_TYPE_BFP16 (2-byte elements); h*2 must be a
// multiple of 16.  Expert ids outside [0, moeExpertNum) are skipped.
//
// Returns TILEXR_ERROR_PARA_CHECK_FAIL with a log line when moeExpertNum, bs*topK or the tokens
// per block exceed the limits above: nothing is launched in that case.
//
// The first call on each device looks up the scratch array's device address and clears its
// barrier word (a synchronous cudaMemset); make that first call outside any stream capture.
// Host threads may call concurrently: the lookup runs once per device and later callers wait
// for it.  All calls on a device share the scratch array, which keeps what the previous call
// left in it: the kernel overwrites every counter it later reads, and the barrier word carries
// the number of the call it belongs to, so a call starts it afresh whatever the previous call
// left there -- also after a call whose barrier gave up (status 5), which needs no clean-up.
// Two calls that overlap on the GPU (different streams) would race on the array, so issue
// calls for one device on one stream or order them with events.  The call number is a kernel
// argument: a captured call replayed from a CUDA graph repeats it, which the barrier accepts
// (a word that is complete or was given up counts as left over, whatever its number).
int TileXRMoeLocalDispatchNoAlloc(const void *x, const int32_t *expertIds, int64_t bs, int64_t h, int64_t topK,
                                  int64_t moeExpertNum, void *expandXOut, int32_t *assistOut, int64_t *expertTokenNumsOut,
                                  int32_t *sendCountsOut, int dtype, TileXRStream stream);

// Device status of the last call on the current device: 0, or 5 (grid barrier gave up).
// Synchronises the device.
int TileXRMoeLocalDispatchNoAllocStatus(int *status);

#ifdef __cplusplus
}
#endif

#endif // TILEXR_NOALLOC_H
