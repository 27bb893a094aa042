// Core runtime C API: communicator life cycle, access to the device CommArgs, launch epochs
// ("magic"), registered memory, local-copy transport and DFX.
//
// Names and argument order follow the reference (src/include/tilexr_api.h:22-83) with
// `aclrtStream` replaced by `cudaStream_t`.  The "UDMA" functions keep their names: on B200 a
// registered region is a peer-mapped allocation reachable by load/store over NVLink rather
// than an RDMA memory region, and a "QP" is an ordering lane (see device/tilexr_rma.cuh).
// Functions below the "additions" line have no counterpart in the reference.
#ifndef TILEXR_API_H
#define TILEXR_API_H

#include <stddef.h>
#include <stdint.h>
#ifndef __cplusplus
#include <stdbool.h>
#endif

#include "tilexr_comm_args.h"
#include "tilexr_types.h"

#ifdef __cplusplus
typedef TileXR::CommArgs TileXRCommArgs;
typedef TileXR::TileXRRegistry TileXRRegistryT;
typedef TileXR::TileXRPhysicalInfo TileXRPhysicalInfoT;
extern "C" {
#else
typedef struct CommArgs TileXRCommArgs;
typedef struct TileXRRegistry TileXRRegistryT;
typedef struct TileXRPhysicalInfo TileXRPhysicalInfoT;
#endif

typedef uint8_t *GM_ADDR;
typedef void *TileXRCommPtr;
typedef void *TileXRStream;   // cudaStream_t
typedef uint32_t TileXRUDMAMemHandle;
typedef uint32_t TileXRUDMAProfileHandle;
#define TILEXRUNIQUE_ID_BYTES 128
typedef struct { char internal[TILEXRUNIQUE_ID_BYTES]; } TileXRUniqueId;

// A profile keeps several registered regions resident at once under one handle.
#define TILEXR_PROFILE_MAX_REGIONS 8
typedef struct TileXRUDMAProfileDesc {
    uint32_t regionCount;
    void *base[TILEXR_PROFILE_MAX_REGIONS];
    size_t bytes[TILEXR_PROFILE_MAX_REGIONS];
} TileXRUDMAProfileDesc;
typedef struct TileXRUDMAProfileView {
    uint32_t regionCount;
    TileXRUDMAMemHandle handles[TILEXR_PROFILE_MAX_REGIONS];
    uint64_t generation;
} TileXRUDMAProfileView;
// Which peers are directly reachable (all of them behind one NVSwitch).
typedef struct TileXRUDMAFullmeshHostView {
    uint32_t slotCount;
    uint32_t reserved;
    uint64_t peerMask[2];      // bit r set: rank r is load/store reachable
    uint64_t generation;
} TileXRUDMAFullmeshHostView;

int TileXRGetUniqueId(TileXRUniqueId *uniqueId, int commDomain);
int TileXRCommInitRankLocal(int rankSize, int rank, TileXRCommPtr *comm);
int TileXRCommInitRank(TileXRUniqueId commId, int rankSize, int rank, TileXRCommPtr *comm);
int TileXRCommInitRankWithCustDomainSize(int commDomain, int bufferSizeMB, int rankSize, int rank, TileXRCommPtr *comm);
int TileXRCommInitRankWithDomain(int commDomain, int rankSize, int rank, TileXRCommPtr *comm);
int TileXRCommInitRankWithSharedQpDomain(int commDomain, int rankSize, int rank, TileXRCommPtr *comm);
int TileXRCommInitRankMemoryDomain(int commDomain, int rankSize, int rank, TileXRCommPtr *comm);
int TileXRCommInit(int rank, int rankSize, TileXRCommPtr *comm);
int TileXRCommInitAll(uint32_t ndev, int32_t *devices, TileXRCommPtr *comms);
int TileXRCommInitThread(int rank, int rankSize, const char *uid, TileXRCommPtr *comm);
int TileXRCommDestroy(TileXRCommPtr comm);

int TileXRGetCommArgsDev(TileXRCommPtr comm, GM_ADDR *commArgsPtr);
int TileXRGetCommArgsHost(TileXRCommPtr comm, TileXRCommArgs **commArgsPtr);
int TileXRCommNextMagic(TileXRCommPtr comm, int64_t *magic);

int TileXRUDMARegister(TileXRCommPtr comm, GM_ADDR localPtr, size_t bytes, TileXRUDMAMemHandle *handle);
int TileXRUDMAUnregister(TileXRCommPtr comm, TileXRUDMAMemHandle handle);
int TileXRUDMAProfileRegister(TileXRCommPtr comm, const TileXRUDMAProfileDesc *desc, TileXRUDMAProfileHandle *handle);
int TileXRUDMAProfileUnregister(TileXRCommPtr comm, TileXRUDMAProfileHandle handle);
int TileXRUDMAProfileQuery(TileXRCommPtr comm, TileXRUDMAProfileHandle handle, TileXRUDMAProfileView *view);
int TileXRUDMAGetQpCount(TileXRCommPtr comm, uint32_t *qpCount);
int TileXRUDMAFullmeshQuery(TileXRCommPtr comm, TileXRUDMAFullmeshHostView *view);
int TileXRGetUDMARegistryDev(TileXRCommPtr comm, GM_ADDR *registryPtr);
int TileXRGetUDMARegistryHost(TileXRCommPtr comm, const TileXRRegistryT **registry);
int TileXRSDMAAvailable(TileXRCommPtr comm, bool *available);
int TileXRGetSDMAWorkspaceDev(TileXRCommPtr comm, GM_ADDR *workspace);
void TileXRPrintDFX2Log(TileXRCommPtr comm);

// ---- additions ------------------------------------------------------------------------------

// Bring-up over a caller-supplied all-gather (a torch Store, a process group, MPI).
typedef int (*TileXRAllGatherFn)(void *ctx, const void *send, void *recv, size_t bytesPerRank);
int TileXRCommInitRankWithExchange(TileXRAllGatherFn allGather, void *ctx, int commDomain, int bufferSizeMB,
                                   int rankSize, int rank, TileXRCommPtr *comm);
// Windows in POSIX shared memory and "kernels" on CPU threads: the no-GPU plumbing mode.
int TileXRCommInitRankHostMemory(int commDomain, int bufferSizeMB, int rankSize, int rank, TileXRCommPtr *comm);
int TileXRCommInitRankHostMemoryWithExchange(TileXRAllGatherFn allGather, void *ctx, int commDomain, int bufferSizeMB,
                                             int rankSize, int rank, TileXRCommPtr *comm);
// Several ranks on ONE device inside one process (test worlds); all launches of such a world
// must go through TileXRGroupStart/End so that they become a single cooperative kernel.
int TileXRCommInitEmulated(uint32_t rankSize, int32_t device, int bufferSizeMB, TileXRCommPtr *comms);

// Calls made between Start and End on the comms of an emulated world are recorded and issued
// by End as one cooperative launch covering every rank.  Outside such a pair, a call on an
// emulated comm fails with TILEXR_ERROR_NOT_SUPPORT.
int TileXRGroupStart(void);
int TileXRGroupEnd(void);

// Device status of the last launches: 0, or a TileXRDeviceStatus left by a bounded wait.
// Synchronises nothing: call it after the stream was synchronised.
int TileXRCommGetDeviceStatus(TileXRCommPtr comm, int *status);
// Clears failure record, abort word and barrier counters after a failed launch (collective).
int TileXRCommResetStatus(TileXRCommPtr comm);
int TileXRCommSetWaitTimeoutMs(TileXRCommPtr comm, uint64_t milliseconds);
int TileXRCommHostBarrier(TileXRCommPtr comm);
int TileXRCommGetInfo(TileXRCommPtr comm, int *rank, int *rankSize, int *device, uint64_t *dataHalfBytes);

// Symmetric allocation: every rank allocates `bytes` and registers it in one collective call.
// `*peerPtrs` (host array, rankSize entries, owned by the communicator) receives the mapping
// of every rank's allocation.
int TileXRSymmAlloc(TileXRCommPtr comm, size_t bytes, void **localPtr, TileXRUDMAMemHandle *handle);
int TileXRSymmFree(TileXRCommPtr comm, TileXRUDMAMemHandle handle);
int TileXRGetPeerPointers(TileXRCommPtr comm, TileXRUDMAMemHandle handle, void **peerPtrs /*[rankSize]*/);
/* The address of [ptr, ptr + bytes) through the NVLink multicast object (a multimem store there reaches every
 * rank's copy, a multimem load-reduce sums all copies in the switch).  ptr must lie in memory of TileXRSymmAlloc
 * or in the communicator's window; *mcPtr is null when the node gave no multicast object. */
int TileXRGetMulticastPointer(TileXRCommPtr comm, const void *ptr, size_t bytes, void **mcPtr);
/* 1 when the communicator's window is bound to a multicast object (TILEXR_FLAG_NVLS is set in CommArgs). */
int TileXRNvlsAvailable(TileXRCommPtr comm);
// Finds the registered region that contains [ptr, ptr+bytes); TILEXR_ERROR_NOT_FOUND if none.
int TileXRFindRegistration(TileXRCommPtr comm, const void *ptr, size_t bytes, TileXRUDMAMemHandle *handle,
                           uint64_t *offset);

// What the device is and how it reaches its peers, detected at initialisation (read-only queries): link kind, peer
// atomics, multicast support, whether the window is bound to an NVLink multicast object.
int TileXRGetPhysicalInfo(TileXRCommPtr comm, TileXRPhysicalInfoT *info);

// At least `bytes` of device memory owned by the communicator (one buffer per communicator, grown on demand, kept until
// the communicator is destroyed): staging for operators that would otherwise allocate per call.  Calls that use it are
// ordered by the stream they run on; growing it waits for the device.
int TileXRGetOperatorScratch(TileXRCommPtr comm, size_t bytes, void **ptr);

// Host-initiated local copy on the communicator's copy-engine stream, ordered after the work
// already queued on `stream` and before work queued on it later (SDMA analogue, host side).
int TileXRLocalCopyAsync(TileXRCommPtr comm, void *dst, const void *src, size_t bytes, TileXRStream stream);

const char *TileXRGetErrorString(int status);

#ifdef __cplusplus
}
#endif

#endif // TILEXR_API_H
