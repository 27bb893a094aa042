// Symmetric device memory from the CUDA virtual-memory API, shared between the processes of one NVSwitch node
// by POSIX file descriptors, with an optional alias through an NVLink multicast object (NVLS).
//
// One collective call gives every rank: its own physical allocation, a mapping of every peer's allocation, and,
// when the GPUs and the driver allow it, one more mapping of the same bytes through a multicast object: a
// `multimem` store to that address lands in every rank's copy, a `multimem` load-reduce fetches and sums all
// copies inside the switch.  The communicator's window and the user regions of TileXRSymmAlloc are allocated this
// way; where the API, the multicast object or the descriptor exchange is refused, the callers fall back to
// cudaMalloc + CUDA IPC (no multicast alias) and the collectives to their peer-to-peer kernels.
//
// The reference's runtime owns window creation and mapping in the same place
// (src/comm/tilexr_comm.cpp:948-1022: allocate, exchange handles, map every peer).
//
// Teardown is collective as well: all ranks meet, then each unmaps the alias, unbinds its memory, unmaps the
// peers and releases.  A rank must not leave while a peer may still issue multimem accesses.
#ifndef TILEXR_VMM_H
#define TILEXR_VMM_H

#include <cstddef>
#include <cstdint>
#include <vector>

namespace TileXR {

class Exchange;

struct VmmAllocation {
    size_t bytes = 0;                   // usable size every rank asked for
    size_t mappedBytes = 0;             // rounded up to the allocation and multicast granularities
    uint8_t *local = nullptr;           // this rank's memory
    std::vector<uint8_t *> peers;       // [rankSize]; peers[rank] == local
    uint8_t *multicast = nullptr;       // alias of all ranks' copies, or null
    int device = -1;
    bool live = false;
    // driver handles (CUmemGenericAllocationHandle)
    unsigned long long memHandle = 0;
    std::vector<unsigned long long> peerHandles;
    unsigned long long mcHandle = 0;
    bool mcBound = false;
};

// What the device and driver offer.  `multicast` needs NVSwitch and a driver with the fabric support enabled.
int VmmDeviceSupport(int device, bool *vmm, bool *multicast);

// Collective over `ex`.  `tag` must be the same on all ranks and unique per call (it names the descriptor
// sockets).  On success `out` is live.  On failure every rank returns an error and holds nothing: the ranks agree
// on the outcome of each phase before they go on.
int VmmAllocate(Exchange &ex, int rank, int rankSize, int device, size_t bytes, bool wantMulticast, uint64_t tag,
                VmmAllocation *out);

// Collective when `ex` is given (orderly destroy); with `ex` null the rank just lets go of its mappings.
int VmmFree(Exchange *ex, VmmAllocation *a);

} // namespace TileXR

#endif
