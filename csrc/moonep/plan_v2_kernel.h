// Argument block of the second-generation MoonEP planner kernel.
#ifndef TILEXR_MOONEP_PLAN_V2_KERNEL_H
#define TILEXR_MOONEP_PLAN_V2_KERNEL_H

#include <stdint.h>

#include "plan_v2_algorithm.h"
#include "tilexr_comm_args.h"
#include "tilexr_launch.h"

namespace TileXR {

constexpr unsigned PLAN_V2_THREADS = 512;

struct PlanV2Args {
    const int32_t *topk;        // [s, k]
    const int32_t *tpe;         // [R, E]
    const int32_t *globalIds;   // [R]
    plan2::Outputs out;
    int32_t *tables;            // plan2::TableInts(dims) int32 of device memory
    CommArgs *comm;
    int64_t magic;
    plan2::Dims dims;
    uint64_t headerHash;        // dimensions, configuration and global ids as seen by the host of this rank
    uint32_t mailStride;        // bytes per sender in a window: header + E int32, rounded up to 16
    uint32_t stagedWords;       // int32 words of dynamic shared memory given to the kernel for the balancing tables, 0 = none
    // Optional tables in the form the dispatch / combine stage kernels take (all null or all set):
    int32_t *stageDst;          // [cap] raw destinations, duplicates decoded (every route carries its hidden state)
    int32_t *stageZeroFill;     // [(E + B) * 2]
    int32_t *stageDstLocal;     // [nvS] source rank * cap + route of the route that fills each row, -1 = none
    int32_t *stageStatus;       // [1] 0 = usable
    uint64_t dstLocalOff;       // window offset of the [nvS] cells the sources write
};

const KernelEntry &PlanV2KernelEntry();

} // namespace TileXR

#endif
