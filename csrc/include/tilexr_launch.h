// Kernel launch service of the core runtime, used by every operator library.
//
// A kernel is described by a KernelEntry with two entry points compiled from the same device
// body: `single` takes the argument struct by value and runs one rank; `emulated` takes a
// device array of argument structs, one per rank, and runs rank blockIdx.y, so that a whole
// emulated world (several ranks on ONE GPU) is a single cooperative launch.  Kernels whose
// blocks wait for one another, or for peers, are launched cooperatively: the launch fails
// with an error instead of deadlocking when the grid cannot be co-resident.
//
// (The reference registers device binaries and launches them by signature,
// src/collectives/host/collective_kernel.cpp:97-223; on CUDA the function pointer is enough.)
#ifndef TILEXR_LAUNCH_H
#define TILEXR_LAUNCH_H

#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
#include <functional>
#endif

#include "tilexr_api.h"

namespace TileXR {

struct KernelEntry {
    const void *single;
    const void *emulated;
    size_t argBytes;
    const char *name;
};

struct LaunchConfig {
    unsigned grid;        // blocks per rank
    unsigned block;       // threads per block
    size_t smemBytes;     // dynamic shared memory
    bool cooperative;     // blocks of the grid wait on one another
};

// Launches `kernel` for `comm`'s rank on `stream`.  On an emulated communicator the call is
// recorded and issued by TileXRGroupEnd together with the other ranks' calls.
int LaunchKernel(TileXRCommPtr comm, const KernelEntry &kernel, const void *args, const LaunchConfig &cfg,
                 TileXRStream stream);

// Number of kernels this library launched since the process started (all communicators).
uint64_t LaunchCount();
// Called by code that launches a kernel directly (local ops without a communicator).
void NoteLaunch();

// Largest grid of `kernel` that can be co-resident on the communicator's device.
// Host work (typically a small follow-up kernel launch) that has to come after the launch that `comm` issued last.  On a
// real communicator that launch is already in its stream and `fn` runs at once; a communicator of an emulated world only
// queues its launches until the group closes, and `fn` runs right after that queued launch has been issued.
int RunAfterLaunch(TileXRCommPtr comm, std::function<int()> fn);

int MaxCooperativeGrid(TileXRCommPtr comm, const KernelEntry &kernel, unsigned block, size_t smemBytes, int ranksPerDevice,
                       unsigned *maxGrid);

} // namespace TileXR

#if defined(__CUDACC__)
// Defines NAME_single / NAME_emulated around a device body `BODY(const ARGS &)` and a
// KernelEntry named NAME##Entry.
#define TILEXR_DEFINE_KERNEL(NAME, ARGS, BODY, MAX_THREADS) TILEXR_DEFINE_KERNEL_OCC(NAME, ARGS, BODY, MAX_THREADS, 1)
// Same, asking the compiler to keep MIN_BLOCKS blocks of MAX_THREADS threads resident per SM.
#define TILEXR_DEFINE_KERNEL_OCC(NAME, ARGS, BODY, MAX_THREADS, MIN_BLOCKS)                            \
    __global__ void __launch_bounds__(MAX_THREADS, MIN_BLOCKS) NAME##_single(const ARGS a) { BODY(a); } \
    __global__ void __launch_bounds__(MAX_THREADS, MIN_BLOCKS) NAME##_emulated(const ARGS *perRank)    \
    {                                                                                                  \
        const ARGS a = perRank[blockIdx.y];                                                            \
        BODY(a);                                                                                       \
    }                                                                                                  \
    static const TileXR::KernelEntry NAME##Entry = {reinterpret_cast<const void *>(&NAME##_single),    \
                                                    reinterpret_cast<const void *>(&NAME##_emulated),  \
                                                    sizeof(ARGS), #NAME};
#endif

#endif // TILEXR_LAUNCH_H
