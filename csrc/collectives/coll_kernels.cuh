// Argument block and geometry shared by the collective kernels and their host launcher.
//
// All collectives here are built from one mechanism that suits a uniform NVSwitch mesh: a
// rank PUSHES 256 KiB (or smaller) tiles straight into a ring of slots that it owns inside
// each destination's window and then raises a per-tile flag there; blocks of the destination
// poll those flags in their own memory and copy or reduce each tile as it lands.  Producer
// and consumer blocks run concurrently in one kernel, so transfer and local work overlap tile
// by tile and no rank ever waits at a barrier.  The reference builds the same ops from
// pull-style pipelines over its IPC windows (src/collectives/kernels/kernels/
// lcal_allgather_big_data.cce:13-191, allreduce_big_data.h:19-275, 91093/all2all_hierarchy.h);
// its ring/hierarchy/SIO variants are fabric workarounds that a one-hop mesh does not need.
#ifndef TILEXR_COLL_KERNELS_CUH
#define TILEXR_COLL_KERNELS_CUH

#include <stdint.h>

#include "tilexr_api.h"
#include "tilexr_comm_args.h"
#include "tilexr_launch.h"

namespace TileXR {

enum CollKind : int32_t {
    COLL_ALL_GATHER = 0,     // every rank contributes sliceBytes; out = concat in rank order
    COLL_ALL_TO_ALL = 1,     // in = R slices; slice p goes to rank p
    COLL_BROADCAST = 2,      // root's buffer to everybody (in == out)
    COLL_REDUCE_SCATTER = 3, // in = R slices; out = reduction of everybody's slice `rank`
    COLL_ALL_REDUCE_ONE_SHOT = 4,   // everybody reduces everything
    COLL_ALL_REDUCE_TWO_SHOT = 5,   // reduce-scatter then all-gather of reduced slices
    COLL_PROFILE_PROBE = 6,  // local copy that exercises every profiler stage
    COLL_SCATTER = 7,        // root's slice p goes to rank p (in == out, the root's own slice stays); first half of a large broadcast
};

struct CollArgs {
    const uint8_t *in;
    uint8_t *out;
    CommArgs *comm;
    void *perfTrace;
    int64_t magic;
    uint64_t sliceBytes;      // bytes per (source, destination) pair
    uint64_t sliceStride;     // distance between two slices in the user buffers (>= sliceBytes)
    uint64_t totalBytes;      // two-shot: bytes of the whole vector
    uint32_t tileBytes;       // multiple of 16
    uint32_t tiles;           // tiles per pair
    uint32_t ringTiles;       // ring slots per pair (>= 1)
    uint32_t pairStride;      // bytes between two sources' rings inside a data half
    int32_t kind;
    int32_t root;
    int32_t dtype;
    int32_t reduceOp;
    uint32_t producers;       // blocks [0, producers) push; the rest consume
    uint32_t reducers;        // two-shot: blocks [producers, producers+reducers) reduce
    uint32_t zeroCopy;        // 1: `out` is registered, peers write into it directly
    uint32_t outHandle;       // registry handle of `out` when zeroCopy
    uint64_t outOffset;       // offset of `out` inside its region
    uint32_t elemSize;
    uint32_t opType;          // TileXROpType for DFX
    // All-to-all with transpose: `in` is a [rows, R * burstBytes] matrix with row pitch pitchBytes; the slice for peer p
    // is its column block p, rows x burstBytes, sent as a contiguous block.  burstBytes == 0: plain contiguous slices.
    uint32_t burstBytes;      // multiple of 16
    uint32_t pitchBytes;
    uint64_t sliceBase;       // first byte of the slice that this launch covers
};

const KernelEntry &PushKernelEntry();          // all-gather, all-to-all, broadcast
const KernelEntry &ReduceKernelEntry();        // reduce-scatter, one-shot all-reduce
const KernelEntry &TwoShotKernelEntry();       // two-shot all-reduce
const KernelEntry &ProbeKernelEntry();

constexpr unsigned COLL_BLOCK_THREADS = 512;

// The operations that can run through the window's NVLink multicast alias (nvls_kernels.cu).
enum NvlsCollKind : int32_t { COLL_KIND_ALL_REDUCE = 0, COLL_KIND_REDUCE_SCATTER = 1, COLL_KIND_ALL_GATHER = 2, COLL_KIND_BROADCAST = 3 };
// TILEXR_SUCCESS: launched.  TILEXR_ERROR_NOT_SUPPORT: not a case for the switch, take the peer-to-peer kernels.
int NvlsWindowCollective(int kind, const void *in, void *out, int64_t count, TileXRDataType dtype, int reduceOp, int root,
                         TileXRCommPtr comm, TileXRStream stream);

} // namespace TileXR

#endif
