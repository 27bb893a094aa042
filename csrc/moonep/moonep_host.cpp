// Host side of MoonEP: ABI checks, window layout, launches, and the CPU reference plan.
// Validation follows the reference's stage router (src/moonep/host/tilexr_moonep.cpp:124-158):
// N % K == 0, E % R == 0, 1 <= B <= E/R, K <= 32, R * NvS <= 2^31.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "moonep_kernels.cuh"
#include "tilexr_log.h"
#include "tilexr_moonep.h"
#include "tilexr_moonep_trace.h"
#include "tilexr_types.h"

using namespace TileXR;

namespace {

uint64_t Align(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

long EnvLong(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

struct Ctx {
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int rank = 0, R = 0, ranksPerDevice = 1;
};

int Prepare(TileXRCommPtr comm, Ctx *c)
{
    if (comm == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    if (TileXRGetCommArgsHost(comm, &c->hostArgs) != TILEXR_SUCCESS || TileXRGetCommArgsDev(comm, &c->devArgs) != TILEXR_SUCCESS) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    if (c->hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_MOONEP_ERROR_NOT_SUPPORTED;
    c->rank = c->hostArgs->rank;
    c->R = c->hostArgs->rankSize;
    c->ranksPerDevice = (c->hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? c->R : 1;
    return TILEXR_MOONEP_SUCCESS;
}

bool ValidDims(int64_t s, int64_t k, int64_t e, int64_t b, int64_t r, int64_t padding)
{
    if (s <= 0 || k <= 0 || e <= 0 || r <= 0 || padding <= 0) return false;
    if (k > TILEXR_MOONEP_MAX_TOPK || e % r != 0 || e > MOONEP_MAX_EXPERTS) return false;
    if (b < 1 || b > e / r) return false;
    const int64_t nvs = s * k + (padding - 1) * 2 * (e / r);
    return r * nvs <= (int64_t(1) << 31);
}

PlanDims MakeDims(int64_t s, int64_t k, int64_t e, int64_t b, int64_t r, int64_t padding)
{
    PlanDims d;
    d.R = static_cast<int32_t>(r);
    d.E = static_cast<int32_t>(e);
    d.L = static_cast<int32_t>(e / r);
    d.B = static_cast<int32_t>(b);
    d.N = static_cast<int32_t>(s * k);
    d.NvS = PlanCapacity(s * k, padding, e / r);
    d.padding = static_cast<int32_t>(padding);
    return d;
}

bool TensorOk(const TileXRMoonEpTensorV1 *t, bool optional)
{
    if (t == nullptr) return optional;
    return t->structSize >= sizeof(TileXRMoonEpTensorV1) && t->data != nullptr && t->rank <= TILEXR_MOONEP_MAX_TENSOR_RANK;
}

bool PlanOk(const TileXRMoonEpPlanV1 *p)
{
    return p != nullptr && p->structSize >= sizeof(TileXRMoonEpPlanV1) && p->n > 0 && p->k > 0 && p->n % p->k == 0 && p->r > 0 &&
           p->e % p->r == 0 && p->b >= 1 && p->b <= p->e / p->r && p->k <= TILEXR_MOONEP_MAX_TOPK &&
           p->r * p->nvS <= (int64_t(1) << 31) && p->dst != nullptr && p->status != nullptr;
}

size_t ElemSize(uint32_t dtype)
{
    switch (dtype) {
        case TILEXR_MOONEP_DTYPE_FLOAT16: case TILEXR_MOONEP_DTYPE_BFLOAT16: return 2;
        case TILEXR_MOONEP_DTYPE_FLOAT32: case TILEXR_MOONEP_DTYPE_INT32: return 4;
        default: return 0;
    }
}

int CoopGrid(TileXRCommPtr comm, const Ctx &c, const KernelEntry &k, size_t smem, long want, unsigned *grid)
{
    unsigned maxGrid = 0;
    if (MaxCooperativeGrid(comm, k, MOONEP_THREADS, smem, c.ranksPerDevice, &maxGrid) != TILEXR_SUCCESS || maxGrid == 0) {
        return TILEXR_MOONEP_ERROR_INTERNAL;
    }
    *grid = static_cast<unsigned>(std::max<long>(1, std::min<long>(want, maxGrid)));
    return TILEXR_MOONEP_SUCCESS;
}

int FillTensorRef(TileXRCommPtr comm, const TileXRMoonEpTensorV1 *t, int64_t rows, MoonTensorRef *ref)
{
    std::memset(ref, 0, sizeof(*ref));
    if (t == nullptr) return TILEXR_MOONEP_SUCCESS;
    const size_t es = ElemSize(t->dtype);
    if (!TensorOk(t, false) || es == 0 || t->rank < 2 || t->shape[0] != rows) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    uint64_t rowElems = 1;
    for (uint32_t i = 1; i < t->rank; ++i) rowElems *= static_cast<uint64_t>(t->shape[i]);
    ref->local = static_cast<uint8_t *>(t->data);
    ref->rowBytes = rowElems * es;
    if (ref->rowBytes % 16 != 0) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    TileXRUDMAMemHandle handle = 0;
    uint64_t offset = 0;
    if (TileXRFindRegistration(comm, t->data, static_cast<size_t>(rows) * ref->rowBytes, &handle, &offset) != TILEXR_SUCCESS) {
        TILEXR_LOG(ERROR) << "MoonEP: weight / gradient tensors must live in registered memory (TileXRSymmAlloc)";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    ref->handle = handle;
    ref->offset = offset;
    ref->valid = 1;
    return TILEXR_MOONEP_SUCCESS;
}

PlannerWindow PlannerLayout(const PlanDims &d, unsigned grid)
{
    PlannerWindow w;
    uint64_t off = 0;
    w.tpeOff = off;
    off = Align(off + static_cast<uint64_t>(d.R) * d.E * 4, 256);
    w.blockCountOff = off;
    off = Align(off + static_cast<uint64_t>(grid) * d.E * 4, 256);
    w.tablesOff = off;
    off = Align(off + PlanTableInts(d) * 4, 256);
    w.dstLocalOff = off;
    off = Align(off + static_cast<uint64_t>(d.NvS) * 8, 256);
    w.totalBytes = off;
    return w;
}

} // namespace

extern "C" {

uint32_t TileXRMoonEpGetAbiVersion(void) { return TILEXR_MOONEP_ABI_VERSION_V2; }

int TileXRMoonEpGetCapabilitiesV1(uint64_t *nativeStages, uint64_t *stubStages)
{
    if (nativeStages == nullptr || stubStages == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    *nativeStages = TILEXR_MOONEP_STAGE_PLANNING | TILEXR_MOONEP_STAGE_DISPATCH | TILEXR_MOONEP_STAGE_PREFETCH_WEIGHT |
                    TILEXR_MOONEP_STAGE_COMBINE | TILEXR_MOONEP_STAGE_REDUCE_GRAD;
    *stubStages = 0;
    return TILEXR_MOONEP_SUCCESS;
}

int TileXRMoonEpGetCapabilitiesV2(uint64_t *nativeStages, uint64_t *stubStages)
{
    return TileXRMoonEpGetCapabilitiesV1(nativeStages, stubStages);
}

int TileXRMoonEpPlannerGetWorkspaceSizeV3(TileXRCommPtr comm, int64_t s, int64_t k, int64_t e, int64_t b, int64_t tokenPadding,
                                          uint64_t *workspaceBytes, int64_t *nvS)
{
    Ctx c;
    const int ret = Prepare(comm, &c);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    if (!ValidDims(s, k, e, b, c.R, tokenPadding) || workspaceBytes == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    const PlanDims d = MakeDims(s, k, e, b, c.R, tokenPadding);
    *workspaceBytes = Align(static_cast<uint64_t>(d.NvS) * 4, 256);   // dstLocal; the tables live in the window
    if (nvS != nullptr) *nvS = d.NvS;
    return TILEXR_MOONEP_SUCCESS;
}

int TileXRMoonEpPlannerGetDstLocalOffsetV3(TileXRCommPtr comm, int64_t s, int64_t k, int64_t e, int64_t b, int64_t tokenPadding,
                                           uint64_t *offsetBytes)
{
    Ctx c;
    const int ret = Prepare(comm, &c);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    if (!ValidDims(s, k, e, b, c.R, tokenPadding) || offsetBytes == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    *offsetBytes = 0;
    return TILEXR_MOONEP_SUCCESS;
}

int TileXRMoonEpPlanningGetWorkspaceSizeV1(TileXRCommPtr comm, int64_t s, int64_t k, int64_t e, int64_t b,
                                           int64_t tokenPadding, uint64_t *workspaceBytes, int64_t *nvS)
{
    return TileXRMoonEpPlannerGetWorkspaceSizeV3(comm, s, k, e, b, tokenPadding, workspaceBytes, nvS);
}

int TileXRMoonEpPlannerV3(const int32_t *topkExperts, const int32_t *tokensPerExpert, TileXRCommPtr comm, int64_t s,
                          int64_t k, int64_t e, int64_t b, int64_t tokenPadding, void *workspace, uint64_t workspaceBytes,
                          int32_t *dst, int32_t *cuSeqlens, int32_t *expertsToCopy, int32_t *zeroFillRanges,
                          int32_t *remoteStats, int32_t *dupCounts, int32_t *status, uint64_t waitIterations,
                          TileXRStream stream)
{
    (void)tokensPerExpert;
    (void)waitIterations;
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    if (topkExperts == nullptr || dst == nullptr || cuSeqlens == nullptr || expertsToCopy == nullptr ||
        zeroFillRanges == nullptr || remoteStats == nullptr || status == nullptr || workspace == nullptr ||
        !ValidDims(s, k, e, b, c.R, tokenPadding)) {
        TILEXR_LOG(ERROR) << "MoonEP planner: invalid arguments";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    const PlanDims d = MakeDims(s, k, e, b, c.R, tokenPadding);
    if (workspaceBytes < static_cast<uint64_t>(d.NvS) * 4) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    // tokens per block: the in-block ranking is quadratic in routes per block
    const long envBlocks = EnvLong("TILEXR_MOONEP_PLANNER_BLOCK_DIM", 64);
    unsigned grid = static_cast<unsigned>(std::max<long>(1, std::min<long>(envBlocks, (s + 7) / 8)));
    uint32_t tokensPerBlock = 0;
    size_t smem = 0;
    for (;;) {
        tokensPerBlock = static_cast<uint32_t>((s + grid - 1) / grid);
        if (static_cast<int64_t>(tokensPerBlock) * k > MOONEP_MAX_ROUTES_PER_BLOCK) {
            TILEXR_LOG(ERROR) << "MoonEP planner: too many routes per block; raise TILEXR_MOONEP_PLANNER_BLOCK_DIM";
            return TILEXR_MOONEP_ERROR_NOT_SUPPORTED;
        }
        smem = MoonPlannerSmemBytes(d.E, static_cast<int>(tokensPerBlock * k));
        unsigned g2 = 0;
        ret = CoopGrid(comm, c, MoonPlannerKernelEntry(), smem, grid, &g2);
        if (ret != TILEXR_MOONEP_SUCCESS) return ret;
        if (g2 >= grid) break;
        grid = g2;
    }
    grid = static_cast<unsigned>((s + tokensPerBlock - 1) / tokensPerBlock);
    PlannerArgs a;
    std::memset(&a, 0, sizeof(a));
    a.win = PlannerLayout(d, grid);
    if (a.win.totalBytes > c.hostArgs->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "MoonEP planner needs " << a.win.totalBytes << " window bytes per half";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    a.topk = topkExperts;
    a.dst = dst;
    a.cuSeqlens = cuSeqlens;
    a.expertsToCopy = expertsToCopy;
    a.zeroFillRanges = zeroFillRanges;
    a.remoteStats = remoteStats;
    a.dupCounts = dupCounts;
    a.status = status;
    a.dstLocalOut = static_cast<int32_t *>(workspace);
    a.comm = reinterpret_cast<CommArgs *>(c.devArgs);
    a.dims = d;
    a.K = static_cast<int32_t>(k);
    a.tokensPerBlock = tokensPerBlock;
    int64_t magic = 0;
    if (TileXRCommNextMagic(comm, &magic) != TILEXR_SUCCESS) return TILEXR_MOONEP_ERROR_INTERNAL;
    a.magic = magic;
    LaunchConfig cfg{grid, MOONEP_THREADS, smem, true};
    return LaunchKernel(comm, MoonPlannerKernelEntry(), &a, cfg, stream) == TILEXR_SUCCESS ? TILEXR_MOONEP_SUCCESS
                                                                                          : TILEXR_MOONEP_ERROR_INTERNAL;
}

int TileXRMoonEpPlanningV1(const TileXRMoonEpPlanningArgsV1 *args, TileXRStream stream)
{
    if (args == nullptr || args->structSize < sizeof(TileXRMoonEpPlanningArgsV1) || !TensorOk(args->topkExperts, false) ||
        !TensorOk(args->cuSeqlens, false) || args->plan == nullptr || args->plan->structSize < sizeof(TileXRMoonEpPlanV1)) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    const TileXRMoonEpPlanV1 *p = args->plan;
    if (p->k <= 0 || p->n % p->k != 0) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    const int64_t s = p->n / p->k;
    const int64_t perRank = p->r > 0 ? p->e / p->r : 0;
    // recover the padding from NvS = N + (padding-1) * 2 * E/R
    if (perRank <= 0 || (p->nvS - p->n) % (2 * perRank) != 0) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    const int64_t padding = (p->nvS - p->n) / (2 * perRank) + 1;
    return TileXRMoonEpPlannerV3(static_cast<const int32_t *>(args->topkExperts->data), nullptr, args->comm, s, p->k, p->e, p->b,
                                 padding, args->workspace, args->workspaceBytes, static_cast<int32_t *>(p->dst),
                                 static_cast<int32_t *>(args->cuSeqlens->data), static_cast<int32_t *>(p->expertsToCopy),
                                 static_cast<int32_t *>(p->zeroFillRanges), static_cast<int32_t *>(p->remoteStats),
                                 static_cast<int32_t *>(p->dupCounts), static_cast<int32_t *>(p->status), args->waitIterations,
                                 stream);
}

int TileXRMoonEpDispatchGetWorkspaceSizeV1(TileXRCommPtr comm, int64_t s, int64_t k, int64_t h, uint32_t hiddenDtype,
                                           uint64_t *workspaceBytes, uint64_t *workspaceAlignment)
{
    (void)comm;
    if (s <= 0 || k <= 0 || h <= 0 || ElemSize(hiddenDtype) == 0 || workspaceBytes == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    *workspaceBytes = 0;   // rows are stored into the destination tensor or the window; no extra workspace
    if (workspaceAlignment != nullptr) *workspaceAlignment = 256;
    return TILEXR_MOONEP_SUCCESS;
}

int TileXRMoonEpDispatchGetWorkspaceSizeV2(TileXRCommPtr comm, int64_t s, int64_t k, int64_t h, uint32_t hiddenDtype,
                                           uint64_t *workspaceBytes, uint64_t *workspaceAlignment)
{
    return TileXRMoonEpDispatchGetWorkspaceSizeV1(comm, s, k, h, hiddenDtype, workspaceBytes, workspaceAlignment);
}

int TileXRMoonEpDispatchV1(const TileXRMoonEpDispatchArgsV1 *args, TileXRStream stream)
{
    if (args == nullptr || args->structSize < sizeof(TileXRMoonEpDispatchArgsV1) || !PlanOk(args->plan) ||
        !TensorOk(args->hiddenSh, false) || !TensorOk(args->hiddenNvsh, false) || !TensorOk(args->routeWeightsSk, true) ||
        !TensorOk(args->routeWeightsNvs, true)) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    if ((args->routeWeightsSk == nullptr) != (args->routeWeightsNvs == nullptr)) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    if (args->flags & (TILEXR_MOONEP_FLAG_SKIP_INTER_RANK_SYNC | TILEXR_MOONEP_FLAG_ZERO_COPY)) return TILEXR_MOONEP_ERROR_NOT_SUPPORTED;
    Ctx c;
    int ret = Prepare(args->comm, &c);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    const TileXRMoonEpPlanV1 *p = args->plan;
    if (p->r != c.R || p->zeroFillRanges == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    const size_t es = ElemSize(args->hiddenSh->dtype);
    if (es == 0 || args->hiddenSh->rank != 2 || args->hiddenNvsh->rank != 2 || args->hiddenSh->dtype != args->hiddenNvsh->dtype ||
        args->hiddenSh->shape[0] * p->k != p->n || args->hiddenNvsh->shape[0] != p->nvS ||
        args->hiddenSh->shape[1] != args->hiddenNvsh->shape[1]) {
        TILEXR_LOG(ERROR) << "MoonEP dispatch: hidden tensors must be [S,H] and [NvS,H] of one dtype";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    const uint64_t rowBytes = static_cast<uint64_t>(args->hiddenSh->shape[1]) * es;
    if (rowBytes % 16 != 0) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    MoonDispatchArgs a;
    std::memset(&a, 0, sizeof(a));
    a.hidden = static_cast<const uint8_t *>(args->hiddenSh->data);
    a.weights = args->routeWeightsSk != nullptr ? static_cast<const float *>(args->routeWeightsSk->data) : nullptr;
    a.dst = static_cast<const int32_t *>(p->dst);
    a.zeroFill = static_cast<const int32_t *>(p->zeroFillRanges);
    a.status = static_cast<const int32_t *>(p->status);
    a.hiddenOut = static_cast<uint8_t *>(args->hiddenNvsh->data);
    a.weightsOut = args->routeWeightsNvs != nullptr ? static_cast<float *>(args->routeWeightsNvs->data) : nullptr;
    a.comm = reinterpret_cast<CommArgs *>(c.devArgs);
    a.N = static_cast<int32_t>(p->n);
    a.K = static_cast<int32_t>(p->k);
    a.NvS = static_cast<int32_t>(p->nvS);
    a.groups = static_cast<int32_t>(p->e + p->b);
    a.rowBytes = static_cast<uint32_t>(rowBytes);
    TileXRUDMAMemHandle h1 = 0, h2 = 0;
    uint64_t o1 = 0, o2 = 0;
    bool zeroCopy = TileXRFindRegistration(args->comm, a.hiddenOut, static_cast<size_t>(p->nvS) * rowBytes, &h1, &o1) == TILEXR_SUCCESS;
    if (zeroCopy && a.weightsOut != nullptr) {
        zeroCopy = TileXRFindRegistration(args->comm, a.weightsOut, static_cast<size_t>(p->nvS) * 4, &h2, &o2) == TILEXR_SUCCESS;
    }
    a.zeroCopy = zeroCopy ? 1u : 0u;
    a.outHandle = h1;
    a.outOffset = o1;
    a.weightHandle = h2;
    a.weightOffset = o2;
    a.weightWinOff = Align(static_cast<uint64_t>(p->nvS) * rowBytes, 256);
    unsigned grid = 0;
    ret = CoopGrid(args->comm, c, MoonDispatchKernelEntry(), 0, std::min<long>(EnvLong("TILEXR_MOONEP_DISPATCH_BLOCKS", 128), (p->n + 15) / 16), &grid);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    if (args->trace != nullptr && args->trace->buffer != nullptr) {
        // the buffer must hold the layout of tilexr_moonep_trace.h for this grid; a short buffer is refused, not overrun
        const TileXRMoonEpDispatchTraceV1 *t = args->trace;
        uint64_t recOff = 0, evOff = 0, total = 0;
        if (t->structSize < sizeof(TileXRMoonEpDispatchTraceV1) || t->iteration >= t->iterationCount ||
            TileXRMoonEpTraceLayout(t->iterationCount, grid, t->eventCapacity, &recOff, &evOff, &total) != 0 || total > t->bufferBytes) {
            TILEXR_LOG(ERROR) << "MoonEP dispatch: the trace buffer of " << t->bufferBytes << " bytes does not hold " << t->iterationCount
                              << " iterations of " << grid << " blocks with " << t->eventCapacity << " events each";
            return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
        }
        a.traceBuffer = t->buffer;
        a.traceIteration = t->iteration;
        a.traceIterationCount = t->iterationCount;
        a.traceEventCapacity = t->eventCapacity;
    }
    if (!zeroCopy && a.weightWinOff + static_cast<uint64_t>(p->nvS) * 4 > c.hostArgs->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "MoonEP dispatch: " << p->nvS << " rows of " << rowBytes << " bytes do not fit the window; allocate "
                          << "hiddenNvsh (and routeWeightsNvs) with TileXRSymmAlloc so that peers write them directly";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    int64_t magic = 0;
    if (TileXRCommNextMagic(args->comm, &magic) != TILEXR_SUCCESS) return TILEXR_MOONEP_ERROR_INTERNAL;
    a.magic = magic;
    LaunchConfig cfg{grid, MOONEP_THREADS, 0, true};
    return LaunchKernel(args->comm, MoonDispatchKernelEntry(), &a, cfg, stream) == TILEXR_SUCCESS ? TILEXR_MOONEP_SUCCESS
                                                                                                 : TILEXR_MOONEP_ERROR_INTERNAL;
}

int TileXRMoonEpDispatchV2(const TileXRMoonEpDispatchArgsV2 *args, TileXRStream stream) { return TileXRMoonEpDispatchV1(args, stream); }

static int LaunchCombine(TileXRCommPtr comm, const int32_t *dstLocal, const int32_t *status, int64_t s, int64_t k, int64_t nvS,
                         int64_t h, uint32_t dtype, const void *hiddenNvsh, void *hiddenSh, const float *weightsNvs, float *weightsSk,
                         TileXRStream stream)
{
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    const size_t es = ElemSize(dtype);
    if (dstLocal == nullptr || hiddenNvsh == nullptr || hiddenSh == nullptr || es == 0 || dtype == TILEXR_MOONEP_DTYPE_INT32 || s <= 0 ||
        k <= 0 || k > TILEXR_MOONEP_MAX_TOPK || nvS <= 0 || h <= 0 || (h * es) % 16 != 0 || s * k > TILEXR_FLAG_SLOT_SLOTS ||
        (weightsNvs == nullptr) != (weightsSk == nullptr)) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    MoonCombineArgs a;
    std::memset(&a, 0, sizeof(a));
    a.hiddenNvs = static_cast<const uint8_t *>(hiddenNvsh);
    a.weightsNvs = weightsNvs;
    a.dstLocal = dstLocal;
    a.status = status;
    a.hiddenOut = static_cast<uint8_t *>(hiddenSh);
    a.weightsOut = weightsSk;
    a.comm = reinterpret_cast<CommArgs *>(c.devArgs);
    a.S = static_cast<int32_t>(s);
    a.K = static_cast<int32_t>(k);
    a.N = static_cast<int32_t>(s * k);
    a.NvS = static_cast<int32_t>(nvS);
    a.rowBytes = static_cast<uint32_t>(h * es);
    a.elemKind = dtype == TILEXR_MOONEP_DTYPE_FLOAT32 ? 2u : dtype == TILEXR_MOONEP_DTYPE_BFLOAT16 ? 1u : 0u;
    a.weightWinOff = Align(static_cast<uint64_t>(s) * k * a.rowBytes, 256);
    if (a.weightWinOff + static_cast<uint64_t>(s) * k * 4 > c.hostArgs->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "MoonEP combine needs " << a.weightWinOff << " window bytes per half; create the communicator with a larger buffer";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    unsigned grid = 0;
    ret = CoopGrid(comm, c, MoonCombineKernelEntry(), 0, std::min<long>(EnvLong("TILEXR_MOONEP_COMBINE_BLOCKS", 148), (nvS + 15) / 16), &grid);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    int64_t magic = 0;
    if (TileXRCommNextMagic(comm, &magic) != TILEXR_SUCCESS) return TILEXR_MOONEP_ERROR_INTERNAL;
    a.magic = magic;
    LaunchConfig cfg{grid, MOONEP_THREADS, 0, true};
    return LaunchKernel(comm, MoonCombineKernelEntry(), &a, cfg, stream) == TILEXR_SUCCESS ? TILEXR_MOONEP_SUCCESS : TILEXR_MOONEP_ERROR_INTERNAL;
}

int TileXRMoonEpCombineV1(const TileXRMoonEpCombineArgsV1 *args, TileXRStream stream)
{
    if (args == nullptr || args->structSize < sizeof(TileXRMoonEpCombineArgsV1) || !PlanOk(args->plan) || args->dstLocal == nullptr ||
        !TensorOk(args->hiddenNvsh, false) || !TensorOk(args->hiddenSh, false) || !TensorOk(args->routeWeightsNvs, true) ||
        !TensorOk(args->routeWeightsSk, true)) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    if (args->flags & (TILEXR_MOONEP_FLAG_COMBINE_PUBLISH_ONLY | TILEXR_MOONEP_FLAG_COMBINE_CONSUME_ONLY |
                       TILEXR_MOONEP_FLAG_SKIP_INTER_RANK_SYNC | TILEXR_MOONEP_FLAG_ZERO_COPY)) {
        return TILEXR_MOONEP_ERROR_NOT_SUPPORTED;   // publish and consume are one kernel here
    }
    const TileXRMoonEpPlanV1 *p = args->plan;
    if (args->hiddenNvsh->rank != 2 || args->hiddenSh->rank != 2 || args->hiddenNvsh->shape[0] != p->nvS ||
        args->hiddenSh->shape[0] * p->k != p->n || args->hiddenNvsh->shape[1] != args->hiddenSh->shape[1] ||
        args->hiddenNvsh->dtype != args->hiddenSh->dtype) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    return LaunchCombine(args->comm, args->dstLocal, static_cast<const int32_t *>(p->status), p->n / p->k, p->k, p->nvS,
                         args->hiddenSh->shape[1], args->hiddenSh->dtype, args->hiddenNvsh->data, args->hiddenSh->data,
                         args->routeWeightsNvs != nullptr ? static_cast<const float *>(args->routeWeightsNvs->data) : nullptr,
                         args->routeWeightsSk != nullptr ? static_cast<float *>(args->routeWeightsSk->data) : nullptr, stream);
}

int TileXRMoonEpPrefetchWeightV1(const TileXRMoonEpPrefetchWeightArgsV1 *args, TileXRStream stream)
{
    if (args == nullptr || args->structSize < sizeof(TileXRMoonEpPrefetchWeightArgsV1) || !PlanOk(args->plan) ||
        args->plan->expertsToCopy == nullptr || (args->gate == nullptr && args->up == nullptr && args->down == nullptr)) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    Ctx c;
    int ret = Prepare(args->comm, &c);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    const TileXRMoonEpPlanV1 *p = args->plan;
    if (p->r != c.R) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    MoonPrefetchArgs a;
    std::memset(&a, 0, sizeof(a));
    a.expertsToCopy = static_cast<const int32_t *>(p->expertsToCopy);
    a.L = static_cast<int32_t>(p->e / p->r);
    a.B = static_cast<int32_t>(p->b);
    const TileXRMoonEpTensorV1 *ts[3] = {args->gate, args->up, args->down};
    for (int i = 0; i < 3; ++i) {
        ret = FillTensorRef(args->comm, ts[i], a.L + a.B, &a.tensors[i]);
        if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    }
    a.comm = reinterpret_cast<CommArgs *>(c.devArgs);
    unsigned grid = 0;
    ret = CoopGrid(args->comm, c, MoonPrefetchKernelEntry(), 0, EnvLong("TILEXR_MOONEP_PREFETCH_BLOCK_DIM", 128), &grid);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    int64_t magic = 0;
    if (TileXRCommNextMagic(args->comm, &magic) != TILEXR_SUCCESS) return TILEXR_MOONEP_ERROR_INTERNAL;
    a.magic = magic;
    LaunchConfig cfg{grid, MOONEP_THREADS, 0, true};
    return LaunchKernel(args->comm, MoonPrefetchKernelEntry(), &a, cfg, stream) == TILEXR_SUCCESS ? TILEXR_MOONEP_SUCCESS : TILEXR_MOONEP_ERROR_INTERNAL;
}

static int LaunchReduceGrad(TileXRCommPtr comm, const TileXRMoonEpPlanV1 *p, const TileXRMoonEpTensorV1 *const ts[3], TileXRStream stream)
{
    Ctx c;
    int ret = Prepare(comm, &c);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    if (!PlanOk(p) || p->expertsToCopy == nullptr || p->r != c.R) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    MoonReduceGradArgs a;
    std::memset(&a, 0, sizeof(a));
    a.expertsToCopy = static_cast<const int32_t *>(p->expertsToCopy);
    a.L = static_cast<int32_t>(p->e / p->r);
    a.B = static_cast<int32_t>(p->b);
    a.clearSlots = 1;
    bool any = false;
    for (int i = 0; i < 3; ++i) {
        if (ts[i] != nullptr && ts[i]->dtype != TILEXR_MOONEP_DTYPE_FLOAT32) {
            TILEXR_LOG(ERROR) << "MoonEP reduce-grad: gradients must be fp32";
            return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
        }
        ret = FillTensorRef(comm, ts[i], a.L + a.B, &a.tensors[i]);
        if (ret != TILEXR_MOONEP_SUCCESS) return ret;
        any = any || a.tensors[i].valid;
    }
    if (!any) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    a.comm = reinterpret_cast<CommArgs *>(c.devArgs);
    unsigned grid = 0;
    ret = CoopGrid(comm, c, MoonReduceGradKernelEntry(), 0, EnvLong("TILEXR_MOONEP_REDUCE_GRAD_BLOCK_DIM", 148), &grid);
    if (ret != TILEXR_MOONEP_SUCCESS) return ret;
    int64_t magic = 0;
    if (TileXRCommNextMagic(comm, &magic) != TILEXR_SUCCESS) return TILEXR_MOONEP_ERROR_INTERNAL;
    a.magic = magic;
    LaunchConfig cfg{grid, MOONEP_THREADS, 0, true};
    return LaunchKernel(comm, MoonReduceGradKernelEntry(), &a, cfg, stream) == TILEXR_SUCCESS ? TILEXR_MOONEP_SUCCESS : TILEXR_MOONEP_ERROR_INTERNAL;
}

int TileXRMoonEpReduceGradV1(const TileXRMoonEpReduceGradArgsV1 *args, TileXRStream stream)
{
    if (args == nullptr || args->structSize < sizeof(TileXRMoonEpReduceGradArgsV1) || args->input == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    if (args->output != nullptr && args->output->data != args->input->data) {
        TILEXR_LOG(ERROR) << "MoonEP reduce-grad accumulates in place: output must alias input";
        return TILEXR_MOONEP_ERROR_NOT_SUPPORTED;
    }
    const TileXRMoonEpTensorV1 *ts[3] = {args->input, nullptr, nullptr};
    return LaunchReduceGrad(args->comm, args->plan, ts, stream);
}

// The owner-pull path needs no staging workspace on NVLink: peers' slots are read in place.
int TileXRMoonEpReduceGradGetWorkspaceSizeV2(const TileXRMoonEpReduceGradWorkspaceQueryV2 *query,
                                             TileXRMoonEpReduceGradWorkspaceInfoV2 *info)
{
    if (query == nullptr || info == nullptr || query->structSize < sizeof(*query)) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    std::memset(info, 0, sizeof(*info));
    info->structSize = sizeof(*info);
    info->abiVersion = TILEXR_MOONEP_ABI_VERSION_V2;
    info->workspaceBytes = 0;
    info->workspaceAlignment = TILEXR_MOONEP_REDUCE_GRAD_WORKSPACE_ALIGNMENT;
    info->udmaChunkBytes = query->requestedUdmaChunkBytes != 0 ? query->requestedUdmaChunkBytes : TILEXR_MOONEP_REDUCE_GRAD_DEFAULT_CHUNK_BYTES;
    const TileXRMoonEpTensorV1 *ts[3] = {query->gate, query->up, query->down};
    for (int i = 0; i < 3; ++i) {
        if (ts[i] == nullptr) continue;
        uint64_t rowElems = 1;
        for (uint32_t d = 1; d < ts[i]->rank; ++d) rowElems *= static_cast<uint64_t>(ts[i]->shape[d]);
        info->rowBytes[i] = rowElems * 4;
        info->chunkCounts[i] = (info->rowBytes[i] + info->udmaChunkBytes - 1) / info->udmaChunkBytes;
        info->projectionQpCounts[i] = 1;
    }
    info->qpCount = 3;
    info->blockDim = static_cast<uint32_t>(EnvLong("TILEXR_MOONEP_REDUCE_GRAD_BLOCK_DIM", 148));
    return TILEXR_MOONEP_SUCCESS;
}

namespace {
struct PreparedReduceGrad {
    TileXRCommPtr comm;
};
} // namespace

int TileXRMoonEpReduceGradPrepareV2(const TileXRMoonEpReduceGradPrepareArgsV2 *args, TileXRMoonEpReduceGradPreparedV2 *prepared)
{
    if (args == nullptr || prepared == nullptr || args->comm == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    // Registration happens when the tensors are allocated (TileXRSymmAlloc); nothing else to prepare.
    *prepared = new PreparedReduceGrad{args->comm};
    return TILEXR_MOONEP_SUCCESS;
}

int TileXRMoonEpReduceGradDestroyPreparedV2(TileXRMoonEpReduceGradPreparedV2 prepared)
{
    if (prepared == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    delete static_cast<PreparedReduceGrad *>(prepared);
    return TILEXR_MOONEP_SUCCESS;
}

int TileXRMoonEpReduceGradV2(const TileXRMoonEpReduceGradArgsV2 *args, TileXRStream stream)
{
    if (args == nullptr || args->prepared == nullptr) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    const TileXRMoonEpTensorV1 *ts[3] = {args->gate, args->up, args->down};
    return LaunchReduceGrad(static_cast<PreparedReduceGrad *>(args->prepared)->comm, args->plan, ts, stream);
}

int TileXRMoonEpReferencePlan(int rank, int64_t r, int64_t s, int64_t k, int64_t e, int64_t b, int64_t tokenPadding,
                              const int32_t *allTopk, int32_t *dst, int32_t *cuSeqlens, int32_t *expertsToCopyAll,
                              int32_t *zeroFillRanges, int32_t *remoteStats, int64_t *nvS)
{
    if (allTopk == nullptr || rank < 0 || rank >= r || !ValidDims(s, k, e, b, r, tokenPadding)) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    const PlanDims d = MakeDims(s, k, e, b, r, tokenPadding);
    std::vector<int32_t> tpe(static_cast<size_t>(d.R) * d.E, 0);
    for (int src = 0; src < d.R; ++src) {
        for (int i = 0; i < d.N; ++i) {
            const int32_t x = allTopk[static_cast<size_t>(src) * d.N + i];
            if (x < 0 || x >= d.E) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
            tpe[static_cast<size_t>(src) * d.E + x] += 1;
        }
    }
    std::vector<int32_t> storage(PlanTableInts(d));
    PlanTables t;
    PlanCarve(d, storage.data(), &t);
    t.tpe = tpe.data();
    if (PlanBalance(d, t) != 0) return TILEXR_MOONEP_ERROR_INTERNAL;
    for (int x = 0; x < d.R; ++x) {
        if (PlanLayoutForDestination(d, t, x) != 0) return TILEXR_MOONEP_ERROR_INTERNAL;
    }
    PlanFinish(d, t);
    const int groups = d.E + d.B;
    if (cuSeqlens != nullptr) std::memcpy(cuSeqlens, t.cu + rank * groups, sizeof(int32_t) * groups);
    if (zeroFillRanges != nullptr) std::memcpy(zeroFillRanges, t.zeroFill + rank * groups * 2, sizeof(int32_t) * groups * 2);
    if (expertsToCopyAll != nullptr) std::memcpy(expertsToCopyAll, t.expertsToCopy, sizeof(int32_t) * d.R * d.B);
    if (remoteStats != nullptr) {
        remoteStats[0] = t.remoteStats[rank * 2];
        remoteStats[1] = t.remoteStats[rank * 2 + 1];
    }
    if (nvS != nullptr) *nvS = d.NvS;
    if (dst != nullptr) {
        std::vector<int32_t> seen(d.E, 0);
        for (int i = 0; i < d.N; ++i) {
            const int32_t x = allTopk[static_cast<size_t>(rank) * d.N + i];
            dst[i] = PlanRouteDst(d, t, rank, x, seen[x]++);
            if (dst[i] < 0) return TILEXR_MOONEP_ERROR_INTERNAL;
        }
    }
    return TILEXR_MOONEP_SUCCESS;
}

} // extern "C"
