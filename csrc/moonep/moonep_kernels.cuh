// Argument blocks of the five MoonEP stage kernels.
#ifndef TILEXR_MOONEP_KERNELS_CUH
#define TILEXR_MOONEP_KERNELS_CUH

#include <stdint.h>

#include "moonep_plan_algorithm.h"
#include "tilexr_comm_args.h"
#include "tilexr_launch.h"

namespace TileXR {

constexpr unsigned MOONEP_THREADS = 512;
constexpr unsigned MOONEP_WARPS = MOONEP_THREADS / 32;
constexpr int MOONEP_MAX_EXPERTS = 1024;
constexpr int MOONEP_MAX_ROUTES_PER_BLOCK = 4096;
constexpr uint32_t MOONEP_COUNT_FLAG_SLOT = TILEXR_FLAGS_PER_PAIR - 1;
constexpr uint32_t MOONEP_DONE_FLAG_SLOT = TILEXR_FLAGS_PER_PAIR - 2;

// Planner scratch inside one data half of the rank's own window (offsets in bytes).
struct PlannerWindow {
    uint64_t tpeOff;         // [R][E] int32: histograms of every rank (peers write their row)
    uint64_t blockCountOff;  // [grid][E] int32
    uint64_t tablesOff;      // PlanTableInts(dims) int32
    uint64_t dstLocalOff;    // [NvS] uint64: (epoch << 32) | (srcRank * N + route), written by the sources
    uint64_t totalBytes;
};

struct PlannerArgs {
    const int32_t *topk;       // [S*K]
    int32_t *dst;              // [N]
    int32_t *cuSeqlens;        // [E+B]
    int32_t *expertsToCopy;    // [R*B]
    int32_t *zeroFillRanges;   // [(E+B)*2]
    int32_t *remoteStats;      // [2]
    int32_t *dupCounts;        // [2] or null
    int32_t *status;           // [1]
    int32_t *dstLocalOut;      // [NvS]
    CommArgs *comm;
    int64_t magic;
    PlanDims dims;
    PlannerWindow win;
    int32_t K;
    uint32_t tokensPerBlock;
};

struct MoonDispatchArgs {
    const uint8_t *hidden;       // [S, H]
    const float *weights;        // [S, K] or null
    const int32_t *dst;          // [N]
    const int32_t *zeroFill;     // [(E+B)*2]
    const int32_t *status;       // plan status, checked on entry
    uint8_t *hiddenOut;          // [NvS, H]
    float *weightsOut;           // [NvS] or null
    CommArgs *comm;
    int64_t magic;
    int32_t N, K, NvS, groups;   // groups = E + B
    uint32_t rowBytes;
    uint32_t zeroCopy;
    uint32_t outHandle, weightHandle;
    uint64_t outOffset, weightOffset;
    uint64_t weightWinOff;       // weights region inside the data half when staged
    // event trace (tilexr_moonep_trace.h), off when traceBuffer is null
    void *traceBuffer;
    uint32_t traceIteration, traceIterationCount, traceEventCapacity;
};

struct MoonCombineArgs {
    const uint8_t *hiddenNvs;    // [NvS, H]
    const float *weightsNvs;     // [NvS] or null
    const int32_t *dstLocal;     // [NvS]
    const int32_t *status;
    uint8_t *hiddenOut;          // [S, H]
    float *weightsOut;           // [S, K] or null
    CommArgs *comm;
    int64_t magic;
    int32_t S, K, N, NvS;
    uint32_t rowBytes;
    uint32_t elemKind;           // 0 fp16, 1 bf16, 2 fp32
    uint64_t weightWinOff;
};

struct MoonTensorRef {
    uint8_t *local;              // [L + B, rowBytes]
    uint64_t rowBytes;
    uint64_t offset;             // inside its registered region
    uint32_t handle;
    uint32_t valid;
};

struct MoonPrefetchArgs {
    const int32_t *expertsToCopy;   // [R, B]
    MoonTensorRef tensors[3];
    CommArgs *comm;
    int64_t magic;
    int32_t L, B;
};

struct MoonReduceGradArgs {
    const int32_t *expertsToCopy;
    MoonTensorRef tensors[3];       // fp32 gradients
    CommArgs *comm;
    int64_t magic;
    int32_t L, B;
    uint32_t clearSlots;
};

const KernelEntry &MoonPlannerKernelEntry();
const KernelEntry &MoonDispatchKernelEntry();
const KernelEntry &MoonCombineKernelEntry();
const KernelEntry &MoonPrefetchKernelEntry();
const KernelEntry &MoonReduceGradKernelEntry();

size_t MoonPlannerSmemBytes(int experts, int routesPerBlock);

} // namespace TileXR

#endif
