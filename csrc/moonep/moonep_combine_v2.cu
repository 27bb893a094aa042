// MoonEP combine, second generation: the rows that one token has on this rank travel back as ONE row.
//
// The first-generation kernel (moonep_kernels.cu) sends every processed row to slot `route` of its source and the
// source adds the K rows of a token.  A token with several routes to one rank then crosses NVLink once per route.
// Here the expert rank first groups its rows by (source rank, token) and sends, per group, the fp32 sum of the
// group's rows in route order, rounded once to the row type, to the slot of the group's LOWEST route; the other
// routes of the group get a flag that says "folded" and no data.  At top-8 over 8 ranks that is 5.25 rows per token
// instead of 8.  The source waits for the K flags of a token as before and adds the rows that carry data.
//
// Grouping needs no help from the planner: a hash table keyed by source * S + token lives in the caller's workspace
// (TileXRMoonEpCombineGetWorkspaceSizeV2), is cleared and filled at the start of every launch (two meetings of the
// rank's blocks), and a work cursor hands the table's entries to the warps, so a block with many heavy groups does
// not hold the others up.  Every block leaves a profile record (tilexr_moonep_trace.h): time points, counters and
// the first wait that gave up.
//
// Numerics: a group's sum is rounded to the row type before it travels and the source adds the groups in fp32 and
// rounds again, so the result can differ from the single-rounding sum of the first generation by about one unit in
// the last place of the row type; fp32 rows differ only by the order of additions.  Route weights return bit-exact.
//
// Reference: src/moonep/combine_v2 (profile record combine_v2_profile.h:16-141, schedule
// src/moonep/common/moonep_combine_schedule.h:79-199) and the duplicate pre-reduction of
// src/moonep/combine/kernels/tilexr_moonep_combine_kernel.cpp:304-383.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/tilexr_convert.cuh"
#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "moonep_kernels.cuh"
#include "tilexr_log.h"
#include "tilexr_moonep.h"
#include "tilexr_moonep_combine_v2.h"
#include "tilexr_moonep_trace.h"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr int MOON_V2_CURSOR_WORD = 0;           // operator scratch word of the control block: two 32-bit cursors

struct MoonCombineV2Args {
    const uint8_t *hiddenNvs;    // [NvS, H]
    const float *weightsNvs;     // [NvS] or null
    const int32_t *dstLocal;     // [NvS]: srcRank * N + route, or negative
    const int32_t *status;       // plan status or null
    uint8_t *hiddenOut;          // [S, H]
    float *weightsOut;           // [S, K] or null
    CommArgs *comm;
    int64_t magic;
    int32_t S, K, N, NvS;
    uint32_t rowBytes;
    uint32_t elemKind;           // 0 fp16, 1 bf16, 2 fp32
    uint64_t weightWinOff;
    // group index in the caller's workspace: `tableSlots` entries of {key, count} and K member rows each
    int32_t *tableKeys;          // [tableSlots] source * S + token, or -1
    int32_t *tableCounts;        // [tableSlots]
    int32_t *tableMembers;       // [tableSlots, K]
    uint32_t tableSlots;         // a power of two
    TileXRMoonEpCombineProfileRecord *profile;   // [gridDim.x] or null
};

struct BlockProfile {
    TileXRMoonEpCombineProfileRecord *rec;   // non-null in thread 0 when profiling
    uint64_t metric[TILEXR_MOONEP_COMBINE_METRIC_COUNT];
};

__device__ __forceinline__ void Mark(BlockProfile &p, int point)
{
    if (p.rec != nullptr) p.rec->timePoint[point] = now_ns();
}

__device__ __forceinline__ uint32_t HashKey(uint32_t key)
{
    key ^= key >> 16;
    key *= 0x7feb352du;
    key ^= key >> 15;
    key *= 0x846ca68bu;
    key ^= key >> 16;
    return key;
}

__device__ __forceinline__ uint32_t TakeWork(uint32_t *cursor, int lane, uint32_t n)
{
    uint32_t it = 0;
    if (lane == 0) it = atomicAdd(cursor, n);
    return __shfl_sync(0xffffffffu, it, 0);
}

__device__ void MoonCombineV2Body(const MoonCombineV2Args &a)
{
    __shared__ unsigned long long sMetric[TILEXR_MOONEP_COMBINE_METRIC_COUNT];
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_COMBINE, a.S, true);
    // a plan whose planner reported a problem is not run
    {
        bool good = true;
        if (ok && threadIdx.x == 0 && a.status != nullptr && *a.status != 0) {
            RaiseFailure(w, TILEXR_DEV_BAD_ARGUMENT, a.comm->rank, 0, 0, static_cast<uint64_t>(*a.status));
            good = false;
        }
        ok = BlockBroadcastOk(good) && ok;
    }
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int R = comm->rankSize;
    const uint32_t epoch = w.epoch;
    const int lane = threadIdx.x & 31;
    const int K = a.K;
    const bool fp32Rows = a.elemKind == 2;
    const bool bf16 = a.elemKind == 1;
    const int vecs = static_cast<int>(a.rowBytes / 16);
    uint32_t *cursors = reinterpret_cast<uint32_t *>(CtrlWord(comm, rank, TILEXR_CTRL_SCRATCH_WORD + MOON_V2_CURSOR_WORD));
    BlockProfile prof{nullptr, {}};
    for (int i = threadIdx.x; i < TILEXR_MOONEP_COMBINE_METRIC_COUNT; i += blockDim.x) sMetric[i] = 0;
    if (threadIdx.x == 0 && a.profile != nullptr && blockIdx.x < TILEXR_MOONEP_COMBINE_PROFILE_MAX_BLOCKS) {
        prof.rec = a.profile + blockIdx.x;
        TileXRMoonEpCombineProfileRecord &r = *prof.rec;
        r.marker = TILEXR_MOONEP_COMBINE_PROFILE_MARKER;
        r.version = TILEXR_MOONEP_COMBINE_PROFILE_VERSION;
        r.recordBytes = sizeof(TileXRMoonEpCombineProfileRecord);
        r.rank = static_cast<uint32_t>(rank);
        r.block = blockIdx.x;
        r.blockDim = blockDim.x;
        r.gridDim = gridDim.x;
        r.timePointCount = TILEXR_MOONEP_COMBINE_TIME_COUNT;
        r.metricCount = TILEXR_MOONEP_COMBINE_METRIC_COUNT;
        r.epoch = epoch;
        for (int i = 0; i < 8; ++i) r.timePoint[i] = 0;
        for (int i = 0; i < 12; ++i) r.metric[i] = 0;
        r.failureStatus = 0;
        r.failureStep = 0;
        r.failurePeer = 0;
        r.failureReserved = 0;
        r.failureSlot = 0;
        r.failureExpected = 0;
        r.failureObserved = 0;
    }
    __syncthreads();
    Mark(prof, TILEXR_MOONEP_COMBINE_TIME_BEGIN);
    int step = TILEXR_MOONEP_COMBINE_TIME_BEGIN;

    // ---- 1. clear the index, 2. enter every row into its group ---------------------------------------------------------
    const uint32_t T = a.tableSlots;
    if (ok) {
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < T; i += gridDim.x * blockDim.x) {
            a.tableKeys[i] = -1;
            a.tableCounts[i] = 0;
        }
    }
    ok = GridBarrier(w, 0) && ok;
    Mark(prof, TILEXR_MOONEP_COMBINE_TIME_INDEX_CLEARED);
    step = ok ? TILEXR_MOONEP_COMBINE_TIME_INDEX_CLEARED : step;
    if (ok) {
        unsigned long long indexed = 0, probes = 0;
        for (int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; s < a.NvS; s += static_cast<int64_t>(gridDim.x) * blockDim.x) {
            const int32_t v = a.dstLocal[s];
            if (v < 0) continue;
            const int src = v / a.N;
            const int route = v - src * a.N;
            if (src >= R) continue;
            const int32_t key = src * a.S + route / K;
            uint32_t slot = HashKey(static_cast<uint32_t>(key)) & (T - 1);
            for (uint32_t tries = 0; tries < T; ++tries) {
                const int32_t old = atomicCAS(&a.tableKeys[slot], -1, key);
                if (old == -1 || old == key) {
                    const int pos = atomicAdd(&a.tableCounts[slot], 1);
                    if (pos < K) a.tableMembers[static_cast<uint64_t>(slot) * K + pos] = static_cast<int32_t>(s);
                    break;
                }
                slot = (slot + 1) & (T - 1);
                ++probes;
            }
            ++indexed;
        }
        atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_ROWS_INDEXED], indexed);
        atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_PROBES], probes);
    }
    ok = GridBarrier(w, 1) && ok;
    Mark(prof, TILEXR_MOONEP_COMBINE_TIME_INDEX_BUILT);
    step = ok ? TILEXR_MOONEP_COMBINE_TIME_INDEX_BUILT : step;

    // ---- 3. send one row per group ---------------------------------------------------------------------------------------
    if (ok) {
        unsigned long long groupsSent = 0, folded = 0, remote = 0;
        for (;;) {
            const uint32_t base = TakeWork(&cursors[0], lane, 32u);
            if (base >= T) break;
            const uint32_t mySlot = base + lane;
            const int myCount = mySlot < T ? min(__ldcg(&a.tableCounts[mySlot]), K) : 0;
            uint32_t todo = __ballot_sync(0xffffffffu, myCount > 0);
            while (todo != 0) {
                const int j = __ffs(todo) - 1;
                todo &= todo - 1;
                const uint32_t slot = base + j;
                const int count = __shfl_sync(0xffffffffu, myCount, j);
                // lane i keeps member i: its row here and its route at the source; then the members are put in route order
                int64_t mRow = -1;
                int mRoute = 0x7fffffff;
                int src = 0;
                if (lane < count) {
                    mRow = __ldcg(&a.tableMembers[static_cast<uint64_t>(slot) * K + lane]);
                    const int32_t v = a.dstLocal[mRow];
                    src = v / a.N;
                    mRoute = v - src * a.N;
                }
                src = __shfl_sync(0xffffffffu, src, 0);
                int order = 0;                       // number of members with a lower route
                for (int i = 0; i < count; ++i) {
                    const int ri = __shfl_sync(0xffffffffu, mRoute, i);
                    if (ri < mRoute) ++order;
                }
                // sorted[i] = lane whose member comes i-th
                int sortedLane = 0;
                for (int i = 0; i < count; ++i) {
                    const int oi = __shfl_sync(0xffffffffu, order, i);
                    if (lane < count && oi == lane) sortedLane = i;
                }
                const int64_t rowAt = __shfl_sync(0xffffffffu, mRow, sortedLane);          // lane i: row of the i-th member
                const int routeAt = __shfl_sync(0xffffffffu, mRoute, sortedLane);
                const int headRoute = __shfl_sync(0xffffffffu, routeAt, 0);
                uint8_t *peerHalf = DataHalf(comm, src, epoch);
                uint8_t *dst = peerHalf + static_cast<uint64_t>(headRoute) * a.rowBytes;
                if (count == 1) {
                    CopyLanesDeep(dst, a.hiddenNvs + __shfl_sync(0xffffffffu, rowAt, 0) * a.rowBytes, a.rowBytes, lane, 32);
                } else {
                    for (int v0 = 0; v0 < vecs; v0 += 32) {
                        const int v = v0 + lane;
                        float acc[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) acc[q] = 0.f;
                        for (int i0 = 0; i0 < count; i0 += 4) {
                            Vec16 x[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int64_t mr = __shfl_sync(0xffffffffu, rowAt, (i0 + i) & 31);
                                x[i] = Vec16{0u, 0u, 0u, 0u};
                                if (i0 + i < count && v < vecs) x[i] = ld_vec16_stream(a.hiddenNvs + mr * a.rowBytes + static_cast<int64_t>(v) * 16);
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (i0 + i >= count) continue;
                                if (fp32Rows) {
                                    acc[0] += __uint_as_float(x[i].x);
                                    acc[1] += __uint_as_float(x[i].y);
                                    acc[2] += __uint_as_float(x[i].z);
                                    acc[3] += __uint_as_float(x[i].w);
                                } else {
                                    float f[8];
                                    Unpack8(x[i], bf16, f);
#pragma unroll
                                    for (int q = 0; q < 8; ++q) acc[q] += f[q];
                                }
                            }
                        }
                        if (v < vecs) {
                            if (fp32Rows) {
                                st_vec16(dst + static_cast<int64_t>(v) * 16, Vec16{__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])});
                            } else {
                                st_vec16(dst + static_cast<int64_t>(v) * 16, Pack8(acc, bf16));
                            }
                        }
                    }
                }
                // every member's weight goes back to its own route
                if (a.weightsNvs != nullptr && lane < count) {
                    reinterpret_cast<float *>(peerHalf + a.weightWinOff)[routeAt] = a.weightsNvs[rowAt];
                }
                __syncwarp();
                // flag value 1: the slot holds a row; 2: the route was folded into the group's first slot
                if (lane < count) SetFlag(FlagSlot(comm, src, TILEXR_FLAG_SLOT_BASE + routeAt), epoch, lane == 0 ? 1u : 2u);
                if (lane == 0) {
                    ++groupsSent;
                    folded += static_cast<unsigned long long>(count - 1);
                    if (src != rank) ++remote;
                }
            }
        }
        if (lane == 0) {
            atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_GROUPS_SENT], groupsSent);
            atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_ROWS_FOLDED], folded);
            atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_REMOTE_GROUPS], remote);
            atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_BYTES_SENT], groupsSent * a.rowBytes);
        }
    }
    __syncthreads();
    Mark(prof, TILEXR_MOONEP_COMBINE_TIME_SEND_END);
    step = ok ? TILEXR_MOONEP_COMBINE_TIME_SEND_END : step;

    // ---- 4. add the rows of this rank's tokens -----------------------------------------------------------------------------
    if (ok) {
        const uint8_t *half = DataHalf(comm, rank, epoch);
        unsigned long long tokens = 0, waits = 0, waitNs = 0;
        while (w.ok()) {
            const uint32_t t = TakeWork(&cursors[1], lane, 1u);
            if (t >= static_cast<uint32_t>(a.S)) break;
            bool carries = false;
            if (lane < K) {
                const int64_t route = static_cast<int64_t>(t) * K + lane;
                const uint64_t *flag = FlagSlot(comm, rank, TILEXR_FLAG_SLOT_BASE + route);
                const uint64_t t0 = now_ns();
                if (WaitFlagGE(w, flag, 1, -1, route)) carries = FlagValue(ld_relaxed_sys_u64(flag)) == 1u;
                waitNs += now_ns() - t0;
                ++waits;
            }
            if (!__all_sync(0xffffffffu, w.ok())) {
                if (w.ok()) w.status = TILEXR_DEV_ABORTED;
                break;
            }
            const uint32_t have = __ballot_sync(0xffffffffu, carries);
            uint8_t *y = a.hiddenOut + static_cast<uint64_t>(t) * a.rowBytes;
            for (int v = lane; v < vecs; v += 32) {
                float acc[8];
                SumRowsColumn(half + static_cast<uint64_t>(t) * K * a.rowBytes, a.rowBytes, K, have, static_cast<uint64_t>(v), fp32Rows ? 2 : (bf16 ? 1 : 0), acc);
                if (fp32Rows) {
                    st_vec16(y + static_cast<int64_t>(v) * 16, Vec16{__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])});
                } else {
                    st_vec16(y + static_cast<int64_t>(v) * 16, Pack8(acc, bf16));
                }
            }
            if (lane < K && a.weightsOut != nullptr) {
                a.weightsOut[static_cast<int64_t>(t) * K + lane] = reinterpret_cast<const float *>(half + a.weightWinOff)[static_cast<int64_t>(t) * K + lane];
            }
            ++tokens;
        }
        if (lane == 0) atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_TOKENS_REDUCED], tokens);
        atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_SLOT_WAITS], waits);
        atomicAdd(&sMetric[TILEXR_MOONEP_COMBINE_METRIC_SLOT_WAIT_NS], waitNs);
        ok = w.ok();
    }
    ok = BlockBroadcastOk(ok);
    Mark(prof, TILEXR_MOONEP_COMBINE_TIME_REDUCE_END);
    if (prof.rec != nullptr) {
        for (int i = 0; i < TILEXR_MOONEP_COMBINE_METRIC_COUNT; ++i) prof.rec->metric[i] = sMetric[i];
        if (!ok) {
            // what the communicator recorded about the first wait that gave up on this rank
            prof.rec->failureStatus = static_cast<uint32_t>(comm->dfx[TILEXR_DFX_FAIL_CODE]);
            prof.rec->failureStep = static_cast<uint32_t>(step);
            prof.rec->failurePeer = static_cast<int32_t>(comm->dfx[TILEXR_DFX_FAIL_PEER]);
            prof.rec->failureSlot = comm->dfx[TILEXR_DFX_FAIL_SLOT];
            prof.rec->failureExpected = static_cast<uint64_t>(comm->dfx[TILEXR_DFX_FAIL_EXPECTED]);
            prof.rec->failureObserved = static_cast<uint64_t>(comm->dfx[TILEXR_DFX_FAIL_OBSERVED]);
        }
    }
    Mark(prof, TILEXR_MOONEP_COMBINE_TIME_END);
    KernelEpilogue(w, ok, 1);
}

TILEXR_DEFINE_KERNEL(TileXRMoonEpCombineV2Kernel, MoonCombineV2Args, MoonCombineV2Body, MOONEP_THREADS)

size_t ElemBytes(uint32_t dtype)
{
    switch (dtype) {
        case TILEXR_MOONEP_DTYPE_FLOAT16:
        case TILEXR_MOONEP_DTYPE_BFLOAT16: return 2;
        case TILEXR_MOONEP_DTYPE_FLOAT32: return 4;
        default: return 0;
    }
}

uint64_t AlignUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

uint32_t TableSlotsFor(int64_t nvS)
{
    uint32_t t = 64;
    while (t < 2 * static_cast<uint64_t>(nvS)) t <<= 1;      // load factor at most one half
    return t;
}

struct WorkspaceLayout {
    uint64_t inputOff, out0Off, out1Off, keysOff, countsOff, membersOff, profileOff, total;
    uint32_t tableSlots;
};

bool Layout(int64_t bs, int64_t h, int64_t topK, int64_t nvS, uint32_t dtype, WorkspaceLayout *l)
{
    const size_t es = ElemBytes(dtype);
    if (bs <= 0 || h <= 0 || topK <= 0 || topK > TILEXR_MOONEP_MAX_TOPK || nvS <= 0 || es == 0) return false;
    const uint64_t rowBytes = static_cast<uint64_t>(h) * es;
    l->tableSlots = TableSlotsFor(nvS);
    uint64_t off = 0;
    l->inputOff = off;
    off = AlignUp(off + static_cast<uint64_t>(nvS) * rowBytes, 256);
    l->out0Off = off;
    off = AlignUp(off + static_cast<uint64_t>(bs) * rowBytes, 256);
    l->out1Off = off;
    off = AlignUp(off + static_cast<uint64_t>(bs) * rowBytes, 256);
    l->keysOff = off;
    off = AlignUp(off + static_cast<uint64_t>(l->tableSlots) * 4, 256);
    l->countsOff = off;
    off = AlignUp(off + static_cast<uint64_t>(l->tableSlots) * 4, 256);
    l->membersOff = off;
    off = AlignUp(off + static_cast<uint64_t>(l->tableSlots) * topK * 4, 256);
    l->profileOff = off;
    off = AlignUp(off + static_cast<uint64_t>(TILEXR_MOONEP_COMBINE_PROFILE_MAX_BLOCKS) * sizeof(TileXRMoonEpCombineProfileRecord), 256);
    l->total = off;
    return true;
}

long EnvLongV2(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

int Launch(void *workspace, uint64_t workspaceBytes, const int32_t *dstLocal, const int32_t *status, TileXRCommPtr comm, int64_t bs, int64_t h,
           int64_t topK, int64_t nvS, const void *hiddenNvsh, void *hiddenSh, const float *weightsNvs, float *weightsSk, uint32_t dtype,
           TileXRStream stream)
{
    WorkspaceLayout l;
    if (comm == nullptr || workspace == nullptr || dstLocal == nullptr || hiddenNvsh == nullptr || hiddenSh == nullptr ||
        !Layout(bs, h, topK, nvS, dtype, &l) || (weightsNvs == nullptr) != (weightsSk == nullptr) || bs * topK > TILEXR_FLAG_SLOT_SLOTS ||
        (static_cast<uint64_t>(h) * ElemBytes(dtype)) % 16 != 0 || reinterpret_cast<uintptr_t>(workspace) % 16 != 0) {
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    if (workspaceBytes < l.total) {
        TILEXR_LOG(ERROR) << "MoonEP combine V2: the workspace has " << workspaceBytes << " bytes, " << l.total << " are needed";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    if (TileXRGetCommArgsHost(comm, &hostArgs) != TILEXR_SUCCESS || TileXRGetCommArgsDev(comm, &devArgs) != TILEXR_SUCCESS) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    if (hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_MOONEP_ERROR_NOT_SUPPORTED;
    if (static_cast<int64_t>(hostArgs->rankSize) * bs >= (1LL << 31)) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    MoonCombineV2Args a;
    std::memset(&a, 0, sizeof(a));
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    a.hiddenNvs = static_cast<const uint8_t *>(hiddenNvsh);
    a.weightsNvs = weightsNvs;
    a.dstLocal = dstLocal;
    a.status = status;
    a.hiddenOut = static_cast<uint8_t *>(hiddenSh);
    a.weightsOut = weightsSk;
    a.comm = reinterpret_cast<CommArgs *>(devArgs);
    a.S = static_cast<int32_t>(bs);
    a.K = static_cast<int32_t>(topK);
    a.N = static_cast<int32_t>(bs * topK);
    a.NvS = static_cast<int32_t>(nvS);
    a.rowBytes = static_cast<uint32_t>(h * ElemBytes(dtype));
    a.elemKind = dtype == TILEXR_MOONEP_DTYPE_FLOAT32 ? 2u : dtype == TILEXR_MOONEP_DTYPE_BFLOAT16 ? 1u : 0u;
    a.weightWinOff = AlignUp(static_cast<uint64_t>(bs) * topK * a.rowBytes, 256);
    if (a.weightWinOff + static_cast<uint64_t>(bs) * topK * 4 > hostArgs->dataHalfBytes) {
        TILEXR_LOG(ERROR) << "MoonEP combine V2 needs " << a.weightWinOff << " window bytes per half; create the communicator with a larger buffer";
        return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    }
    a.tableKeys = reinterpret_cast<int32_t *>(ws + l.keysOff);
    a.tableCounts = reinterpret_cast<int32_t *>(ws + l.countsOff);
    a.tableMembers = reinterpret_cast<int32_t *>(ws + l.membersOff);
    a.tableSlots = l.tableSlots;
    a.profile = EnvLongV2("TILEXR_MOONEP_COMBINE_PROFILE", 1) != 0 ? reinterpret_cast<TileXRMoonEpCombineProfileRecord *>(ws + l.profileOff) : nullptr;
    const int ranksPerDevice = (hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? hostArgs->rankSize : 1;
    unsigned maxGrid = 0;
    if (MaxCooperativeGrid(comm, TileXRMoonEpCombineV2KernelEntry, MOONEP_THREADS, 0, ranksPerDevice, &maxGrid) != TILEXR_SUCCESS || maxGrid == 0) {
        return TILEXR_MOONEP_ERROR_INTERNAL;
    }
    const long want = std::min<long>(EnvLongV2("TILEXR_MOONEP_COMBINE_BLOCKS", 148), static_cast<long>((nvS + 15) / 16));
    const unsigned grid = std::max(1u, std::min<unsigned>(static_cast<unsigned>(std::min<long>(want, TILEXR_MOONEP_COMBINE_PROFILE_MAX_BLOCKS)), maxGrid));
    int64_t magic = 0;
    if (TileXRCommNextMagic(comm, &magic) != TILEXR_SUCCESS) return TILEXR_MOONEP_ERROR_INTERNAL;
    a.magic = magic;
    LaunchConfig cfg{grid, MOONEP_THREADS, 0, true};
    return LaunchKernel(comm, TileXRMoonEpCombineV2KernelEntry, &a, cfg, stream) == TILEXR_SUCCESS ? TILEXR_MOONEP_SUCCESS : TILEXR_MOONEP_ERROR_INTERNAL;
}

} // namespace
} // namespace TileXR

using namespace TileXR;

extern "C" {

int TileXRMoonEpCombineGetWorkspaceSizeV2(int64_t bs, int64_t h, int64_t topK, int64_t nvS, uint32_t dtype, uint64_t *workspaceBytes,
                                          uint64_t *profileOffset, uint64_t *outputEpoch0Offset, uint64_t *outputEpoch1Offset)
{
    WorkspaceLayout l;
    if (workspaceBytes == nullptr || !Layout(bs, h, topK, nvS, dtype, &l)) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    *workspaceBytes = l.total;
    if (profileOffset != nullptr) *profileOffset = l.profileOff;
    if (outputEpoch0Offset != nullptr) *outputEpoch0Offset = l.out0Off;
    if (outputEpoch1Offset != nullptr) *outputEpoch1Offset = l.out1Off;
    return TILEXR_MOONEP_SUCCESS;
}

int TileXRMoonEpCombineStageV2(void *registeredWorkspace, uint64_t registeredWorkspaceBytes, const int32_t *dstLocal, TileXRCommPtr comm,
                               int64_t bs, int64_t h, int64_t topK, int64_t nvS, uint32_t aivCoreNum, const void *hiddenNvsh, void *hiddenSh,
                               const float *routeWeightsNvs, float *routeWeightsSk, uint32_t dtype, TileXRStream stream)
{
    (void)aivCoreNum;     // a block count of the reference's hardware; the grid here follows the GPU
    return Launch(registeredWorkspace, registeredWorkspaceBytes, dstLocal, nullptr, comm, bs, h, topK, nvS, hiddenNvsh, hiddenSh, routeWeightsNvs,
                  routeWeightsSk, dtype, stream);
}

int TileXRMoonEpCombineStageV2Fused(void *registeredWorkspace, uint64_t registeredWorkspaceBytes, const int32_t *dstLocal, TileXRCommPtr comm,
                                    TileXRCommPtr weightMemoryComm, int64_t bs, int64_t h, int64_t topK, int64_t nvS, uint32_t aivCoreNum,
                                    const void *hiddenNvsh, void *hiddenSh, const float *routeWeightsNvs, float *routeWeightsSk, uint32_t dtype,
                                    TileXRStream stream)
{
    // The reference moves the route weights through a second, memory-only communicator; here they ride in the same
    // kernel as the rows, so that communicator is only checked for consistency.
    if (weightMemoryComm != nullptr && weightMemoryComm != comm) {
        TileXRCommArgs *a = nullptr, *b = nullptr;
        if (TileXRGetCommArgsHost(comm, &a) != TILEXR_SUCCESS || TileXRGetCommArgsHost(weightMemoryComm, &b) != TILEXR_SUCCESS ||
            a->rankSize != b->rankSize || a->rank != b->rank) {
            return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
        }
    }
    return TileXRMoonEpCombineStageV2(registeredWorkspace, registeredWorkspaceBytes, dstLocal, comm, bs, h, topK, nvS, aivCoreNum, hiddenNvsh,
                                      hiddenSh, routeWeightsNvs, routeWeightsSk, dtype, stream);
}

int TileXRMoonEpCombineV2(void *registeredWorkspace, const int32_t *dstLocal, TileXRCommPtr comm, int64_t bs, int64_t h, int64_t topK, int64_t nvS,
                          uint32_t aivCoreNum, uint64_t *activeOutputOffset, uint32_t dtype, TileXRStream stream)
{
    // The workspace-resident form: the processed rows are the workspace's input region, the result goes to one of
    // its two output regions in turn, and the caller learns which.
    static thread_local uint64_t calls = 0;
    WorkspaceLayout l;
    if (registeredWorkspace == nullptr || activeOutputOffset == nullptr || !Layout(bs, h, topK, nvS, dtype, &l)) return TILEXR_MOONEP_ERROR_INVALID_ARGUMENT;
    uint8_t *ws = static_cast<uint8_t *>(registeredWorkspace);
    const uint64_t out = (calls++ & 1) == 0 ? l.out0Off : l.out1Off;
    const int ret = Launch(registeredWorkspace, l.total, dstLocal, nullptr, comm, bs, h, topK, nvS, ws + l.inputOff, ws + out, nullptr, nullptr, dtype, stream);
    if (ret == TILEXR_MOONEP_SUCCESS) *activeOutputOffset = out;
    (void)aivCoreNum;
    return ret;
}

} // extern "C"
