// MoonEP stage kernels for sm_100a: planner, dispatch, combine, prefetch-weight, reduce-grad.
//
// All five are cooperative kernels over NVLink peer windows with the runtime's usual rules:
// epoch-tagged flags, bounded waits that record a failure and raise the abort word, rows
// pushed to their final slot by the sender.  What the reference does with RDMA queue pairs,
// credits and staged receive scratch (src/moonep/dispatch/urma/*, combine_v2/*) is a plain
// store or load here; what it does with a host synchronisation between planning and dispatch
// (integrations/moonep_torch/tilexr_moonep/torch_api.py:1182-1192) is a device-side check of
// plan.status at the start of every later stage.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/tilexr_convert.cuh"
#include "device/tilexr_route_rank.cuh"
#include "device/tilexr_moonep_trace.cuh"
#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "moonep_kernels.cuh"
#include "tilexr_moonep.h"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

__device__ __forceinline__ uint64_t *BlockFlag(CommArgs *comm, int owner, int src, uint32_t index)
{
    return FlagSlot(comm, owner, TILEXR_FLAG_OP_BASE + static_cast<int64_t>(src) * TILEXR_FLAGS_PER_PAIR + index);
}

// Every block of every source raises flag `blockIdx` at every destination when it is done
// sending; a destination is complete when it saw all blocks of all sources.
__device__ __forceinline__ void RaiseBlockFlags(CommArgs *comm, int rank, int R, uint32_t epoch)
{
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < R) SetFlag(BlockFlag(comm, threadIdx.x, rank, blockIdx.x), epoch, 1);
}

__device__ __forceinline__ bool WaitAllBlockFlags(Waiter &w, CommArgs *comm, int rank, int R, bool ok)
{
    bool got = true;
    if (ok && static_cast<int>(threadIdx.x) < R) {
        for (uint32_t b = 0; b < gridDim.x && got; ++b) {
            got = WaitFlagGE(w, BlockFlag(comm, rank, threadIdx.x, b), 1, threadIdx.x, b);
        }
    }
    return BlockBroadcastOk(got) && ok;
}

// A kernel that writes into (or reads from) a peer's own tensors, not its window, meets the peers first: every rank
// announces that it has entered this launch (all earlier work of its stream is finished by then) and touches a peer's
// tensors only after that peer's announcement.  The window guard (the peer has finished the launch before last) says
// nothing about tensors that the peer's other kernels read or write: its expert GEMM on the rows of the previous
// dispatch, its optimizer step on the weights that a prefetch pulls, its backward GEMM into the gradient slots.
__device__ __forceinline__ bool MeetPeersOnEntry(Waiter &w, CommArgs *comm, int rank, int R, uint32_t epoch, bool ok)
{
    constexpr uint32_t READY = MOONEP_DONE_FLAG_SLOT - 1;      // far above the per-block flags of the same plane, beside the "done" flag
    if (R <= 1) return ok;
    const int t = static_cast<int>(threadIdx.x);
    if (ok && blockIdx.x == 0 && t < R && t != rank) SetFlag(BlockFlag(comm, t, rank, READY), epoch, 1);
    bool got = true;
    if (ok && t < R && t != rank) got = WaitFlagGE(w, BlockFlag(comm, rank, t, READY), 1, t, READY);
    return BlockBroadcastOk(got) && ok;
}

// A stage refuses to run on a plan whose planner reported a problem.
__device__ __forceinline__ bool PlanUsable(Waiter &w, const int32_t *status, bool ok)
{
    bool good = true;
    if (ok && threadIdx.x == 0 && status != nullptr && *status != 0) {
        RaiseFailure(w, TILEXR_DEV_BAD_ARGUMENT, w.args->rank, 0, 0, static_cast<uint64_t>(*status));
        good = false;
    }
    return BlockBroadcastOk(good) && ok;
}

// ---- planner ---------------------------------------------------------------------------------------------

__device__ void PlannerBody(const PlannerArgs &a)
{
    extern __shared__ __align__(16) uint8_t smemRaw[];
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_PLANNING, a.dims.N, true);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int R = a.dims.R, E = a.dims.E;
    const int G = gridDim.x;
    const int tid = threadIdx.x;
    const uint32_t epoch = w.epoch;
    const int routesPerBlock = static_cast<int>(a.tokensPerBlock) * a.K;
    int32_t *sExpert = reinterpret_cast<int32_t *>(smemRaw);
    int32_t *sRank = sExpert + routesPerBlock;
    int32_t *sHist = sRank + routesPerBlock;
    int32_t *sBase = sHist + E;
    uint8_t *half = DataHalf(comm, rank, epoch);
    int32_t *blockCounts = reinterpret_cast<int32_t *>(half + a.win.blockCountOff);
    int32_t *tpe = reinterpret_cast<int32_t *>(half + a.win.tpeOff);
    PlanTables t;
    PlanCarve(a.dims, reinterpret_cast<int32_t *>(half + a.win.tablesOff), &t);
    t.tpe = tpe;

    const int r0 = min(a.dims.N, static_cast<int>(blockIdx.x) * routesPerBlock);
    const int r1 = min(a.dims.N, r0 + routesPerBlock);
    const int nRoutes = r1 - r0;
    if (blockIdx.x == 0 && tid == 0) *a.status = 0;

    // 1. local histogram with a stable rank per route
    for (int e = tid; e < E; e += blockDim.x) sHist[e] = 0;
    bool valid = true;
    for (int i = tid; i < nRoutes; i += blockDim.x) {
        const int e = a.topk[r0 + i];
        sExpert[i] = e;
        if (e < 0 || e >= E) valid = false;
    }
    valid = BlockBroadcastOk(valid);
    if (!valid && tid == 0 && ok) RaiseFailure(w, TILEXR_DEV_BAD_ARGUMENT, rank, 0, 0, 0);
    ok = ok && valid;
    if (ok && tid < 32) RankRoutesByWarp(sExpert, sRank, sHist, nRoutes, tid);
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) blockCounts[static_cast<int64_t>(blockIdx.x) * E + e] = sHist[e];
    ok = GridBarrier(w, 0) && ok;

    // 2. exchange the histograms
    if (ok && blockIdx.x == 0) {
        for (int e = tid; e < E; e += blockDim.x) {
            int c = 0;
            for (int b = 0; b < G; ++b) c += blockCounts[static_cast<int64_t>(b) * E + e];
            for (int i = 0; i < R; ++i) {
                const int peer = (rank + i) % R;
                reinterpret_cast<int32_t *>(DataHalf(comm, peer, epoch) + a.win.tpeOff)[static_cast<int64_t>(rank) * E + e] = c;
            }
        }
        __syncthreads();
        if (tid < R) SetFlag(BlockFlag(comm, tid, rank, MOONEP_COUNT_FLAG_SLOT), epoch, 1);
    }
    for (int e = tid; e < E; e += blockDim.x) {
        int c = 0;
        for (int b = 0; b < static_cast<int>(blockIdx.x); ++b) c += blockCounts[static_cast<int64_t>(b) * E + e];
        sBase[e] = c;
    }
    // 3. block 0 builds the plan tables (identical on every rank: same input, same arithmetic)
    if (blockIdx.x == 0) {
        bool got = true;
        if (ok && tid < R) got = WaitFlagGE(w, BlockFlag(comm, rank, tid, MOONEP_COUNT_FLAG_SLOT), 1, tid, MOONEP_COUNT_FLAG_SLOT);
        ok = BlockBroadcastOk(got) && ok;
        __shared__ int sPlanError;
        if (tid == 0) sPlanError = 0;
        __syncthreads();
        if (ok) {
            if (tid == 0 && PlanBalance(a.dims, t) != 0) sPlanError = 1;
            __syncthreads();
            if (tid < R && PlanLayoutForDestination(a.dims, t, tid) != 0) sPlanError = 1;
            __syncthreads();
            if (tid == 0) PlanFinish(a.dims, t);
            __syncthreads();
            const int groups = E + a.dims.B;
            for (int g = tid; g < groups; g += blockDim.x) {
                a.cuSeqlens[g] = t.cu[rank * groups + g];
                a.zeroFillRanges[g * 2] = t.zeroFill[(rank * groups + g) * 2];
                a.zeroFillRanges[g * 2 + 1] = t.zeroFill[(rank * groups + g) * 2 + 1];
            }
            for (int i = tid; i < R * a.dims.B; i += blockDim.x) a.expertsToCopy[i] = t.expertsToCopy[i];
            if (tid == 0) {
                a.remoteStats[0] = t.remoteStats[rank * 2];
                a.remoteStats[1] = t.remoteStats[rank * 2 + 1];
                if (a.dupCounts != nullptr) {
                    a.dupCounts[0] = 0;
                    a.dupCounts[1] = 0;
                }
                if (sPlanError != 0) *a.status = TILEXR_MOONEP_STATUS_LAYOUT_OVERFLOW;
            }
        }
    }
    ok = GridBarrier(w, 1) && ok;
    // every rank computed the same tables, so a layout overflow stops every rank alike
    const bool planGood = ok && *reinterpret_cast<volatile int32_t *>(a.status) == 0;

    // 4. destination of every local route; tell the destination who fills each of its slots
    if (planGood) {
        for (int i = tid; i < nRoutes; i += blockDim.x) {
            const int e = sExpert[i];
            const int32_t raw = PlanRouteDst(a.dims, t, rank, e, sBase[e] + sRank[i]);
            a.dst[r0 + i] = raw;
            if (raw >= 0) {
                const int dstRank = raw / a.dims.NvS;
                const int slot = raw - dstRank * a.dims.NvS;
                uint64_t *cell = reinterpret_cast<uint64_t *>(DataHalf(comm, dstRank, epoch) + a.win.dstLocalOff) + slot;
                st_relaxed_sys_u64(cell, MakeFlag(epoch, static_cast<uint32_t>(rank * a.dims.N + r0 + i)));
            }
        }
    }
    if (ok) RaiseBlockFlags(comm, rank, R, epoch);
    ok = WaitAllBlockFlags(w, comm, rank, R, ok);
    if (planGood && ok) {
        const uint64_t *cells = reinterpret_cast<const uint64_t *>(half + a.win.dstLocalOff);
        for (int s = blockIdx.x * blockDim.x + tid; s < a.dims.NvS; s += G * blockDim.x) {
            const uint64_t v = ld_relaxed_sys_u64(cells + s);
            a.dstLocalOut[s] = FlagEpoch(v) == epoch ? static_cast<int32_t>(FlagValue(v)) : -1;
        }
    }
    if (!ok && tid == 0) {
        atomicCAS(a.status, 0, TILEXR_MOONEP_STATUS_PLANNER_TIMEOUT_BASE + static_cast<int>(comm->dfx[TILEXR_DFX_FAIL_PEER]));
    }
    KernelEpilogue(w, ok);
}

// ---- dispatch ----------------------------------------------------------------------------------------------

__device__ void MoonDispatchBody(const MoonDispatchArgs &a)
{
    __shared__ unsigned int sPeerRows[TILEXR_MAX_RANK_SIZE];     // rows this block sent to each rank (for the trace)
    __shared__ int sBad;                                         // 1 + index of a route whose destination is impossible
    __shared__ unsigned int sCleared;                            // padding rows this block cleared (for the trace)
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_DISPATCH, a.N, true);
    ok = PlanUsable(w, a.status, ok);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int R = comm->rankSize;
    const uint32_t epoch = w.epoch;
    const int lane = threadIdx.x & 31;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * MOONEP_WARPS + (threadIdx.x >> 5);
    const int64_t nWarps = static_cast<int64_t>(gridDim.x) * MOONEP_WARPS;
    uint8_t *half = DataHalf(comm, rank, epoch);
    MoonTrace trace{nullptr, nullptr, 0, 0, 0, 0};
    if (threadIdx.x == 0) {
        trace = MoonTraceOpen(a.traceBuffer, a.traceIteration, a.traceIterationCount, a.traceEventCapacity, static_cast<uint32_t>(rank),
                              static_cast<uint32_t>(R), blockIdx.x, gridDim.x, epoch);
        MoonTraceBegin(trace);
        MoonTraceEnd(trace, TILEXR_MOONEP_TRACE_PLAN_CHECK, TILEXR_MOONEP_TRACE_NO_PEER, 0, 0);
        sBad = 0;
        sCleared = 0;
    }
    for (int r = threadIdx.x; r < R; r += blockDim.x) sPeerRows[r] = 0;
    __syncthreads();
    // rows that go straight into the peers' receive tensors wait for the peers to have entered this launch
    if (a.zeroCopy) ok = MeetPeersOnEntry(w, comm, rank, R, epoch, ok);

    if (ok) {
        // padding rows are cleared by their owner; they never overlap a delivered row
        MoonTraceBegin(trace);
        // (all warps of the grid share the rows of every range: the range behind the last expert holds the whole unused
        // capacity, tens of megabytes that one block alone would take longer to clear than the sends take)
        const int64_t vecsPerRow = a.rowBytes / 16;
        unsigned int mine = 0;
        for (int g = 0; g < a.groups; ++g) {
            const int64_t first = a.zeroFill[g * 2];
            const int64_t rows = a.zeroFill[g * 2 + 1];
            const Vec16 z{0, 0, 0, 0};
            for (int64_t r = gwarp; r < rows; r += nWarps) {
                uint8_t *p = a.hiddenOut + (first + r) * a.rowBytes;
                for (int64_t v = lane; v < vecsPerRow; v += 32) st_vec16(p + v * 16, z);
                if (lane == 0 && a.weightsOut != nullptr) a.weightsOut[first + r] = 0.f;
                mine += 1;
            }
        }
        if (lane == 0 && mine != 0) atomicAdd(&sCleared, mine);
        __syncthreads();
        const uint64_t cleared = sCleared;
        MoonTraceEnd(trace, TILEXR_MOONEP_TRACE_ZERO_FILL, rank, cleared * a.rowBytes, static_cast<uint32_t>(cleared));
        MoonTraceBegin(trace);
        for (int64_t i = gwarp; i < a.N; i += nWarps) {
            int32_t raw = a.dst[i];
            if (raw < 0) raw = ~raw;     // a duplicate is delivered like a primary
            const int dstRank = raw / a.NvS;
            const int64_t slot = raw - dstRank * a.NvS;
            if (dstRank >= R) {
                // a plan that names a rank outside the communicator is not skipped over: every rank learns of it
                if (lane == 0) atomicMax(&sBad, static_cast<int>(min(i, static_cast<int64_t>(0x7ffffffe))) + 1);
                continue;
            }
            const uint8_t *row = a.hidden + (i / a.K) * a.rowBytes;
            uint8_t *out;
            float *wout = nullptr;
            if (a.zeroCopy) {
                out = comm->registryPtr->regions[a.outHandle].peerBase[dstRank] + a.outOffset + slot * a.rowBytes;
                if (a.weights != nullptr) {
                    wout = reinterpret_cast<float *>(comm->registryPtr->regions[a.weightHandle].peerBase[dstRank] + a.weightOffset) + slot;
                }
            } else {
                uint8_t *peerHalf = DataHalf(comm, dstRank, epoch);
                out = peerHalf + slot * a.rowBytes;
                if (a.weights != nullptr) wout = reinterpret_cast<float *>(peerHalf + a.weightWinOff) + slot;
            }
            CopyLanesDeep(out, row, a.rowBytes, lane, 32);
            if (lane == 0) {
                if (wout != nullptr) *wout = a.weights[i];
                if (trace.capacity != 0 || a.traceBuffer != nullptr) atomicAdd(&sPeerRows[dstRank], 1u);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            if (sBad != 0) RaiseFailure(w, TILEXR_DEV_BAD_ARGUMENT, rank, sBad - 1, static_cast<uint64_t>(R), static_cast<uint64_t>(a.dst[sBad - 1]));
            if (trace.record != nullptr) {
                // one event per destination: all of them span the block's whole send phase
                const uint64_t opened = trace.openedNs;
                for (int r = 0; r < R; ++r) {
                    if (sPeerRows[r] == 0) continue;
                    trace.openedNs = opened;
                    MoonTraceEnd(trace, TILEXR_MOONEP_TRACE_ROUTE_SEND, r, static_cast<uint64_t>(sPeerRows[r]) * a.rowBytes, sPeerRows[r]);
                }
            }
        }
        ok = BlockBroadcastOk(sBad == 0);
        MoonTraceBegin(trace);
        RaiseBlockFlags(comm, rank, R, epoch);
        MoonTraceEnd(trace, TILEXR_MOONEP_TRACE_FLAG_RAISE, TILEXR_MOONEP_TRACE_NO_PEER, 0, 0);
    }
    MoonTraceBegin(trace);
    ok = WaitAllBlockFlags(w, comm, rank, R, ok);
    MoonTraceEnd(trace, TILEXR_MOONEP_TRACE_FLAG_WAIT, TILEXR_MOONEP_TRACE_NO_PEER, 0, 0);
    if (ok && !a.zeroCopy) {
        MoonTraceBegin(trace);
        // copy the delivered rows out of the window; padding rows were cleared above
        const int64_t total = static_cast<int64_t>(a.NvS);
        const int64_t perBlock = (total + gridDim.x - 1) / gridDim.x;
        const int64_t s0 = min(total, perBlock * blockIdx.x);
        const int64_t n = min(total - s0, perBlock);
        // rows inside zero-fill ranges hold stale window bytes: skip them
        for (int64_t s = s0 + (threadIdx.x >> 5); s < s0 + n; s += MOONEP_WARPS) {
            bool padding = false;
            for (int g = 0; g < a.groups && !padding; ++g) {
                const int64_t first = a.zeroFill[g * 2];
                padding = s >= first && s < first + a.zeroFill[g * 2 + 1];
            }
            if (padding) continue;
            CopyLanes(a.hiddenOut + s * a.rowBytes, half + s * a.rowBytes, a.rowBytes, lane, 32);
            if (lane == 0 && a.weightsOut != nullptr) a.weightsOut[s] = reinterpret_cast<const float *>(half + a.weightWinOff)[s];
        }
        MoonTraceEnd(trace, TILEXR_MOONEP_TRACE_OUTPUT_COPY, rank, static_cast<uint64_t>(n) * a.rowBytes, static_cast<uint32_t>(n));
    }
    MoonTraceClose(trace, static_cast<uint32_t>(w.status));
    KernelEpilogue(w, ok);
}

// ---- combine -------------------------------------------------------------------------------------------------

__device__ void MoonCombineBody(const MoonCombineArgs &a)
{
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_COMBINE, a.S, true);
    ok = PlanUsable(w, a.status, ok);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const uint32_t epoch = w.epoch;
    const int lane = threadIdx.x & 31;
    const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * MOONEP_WARPS + (threadIdx.x >> 5);
    const int64_t nWarps = static_cast<int64_t>(gridDim.x) * MOONEP_WARPS;
    const int K = a.K;

    if (ok) {
        // A warp returns four rows, then one lane orders them all with ONE system-scope fence and raises their four flags.
        // (A release store per row makes the warp wait for that row's stores to be acknowledged by the peer before it
        // may start the next row: several microseconds of an idle warp per 14 KB.)
        constexpr int ROWS_PER_FENCE = 4;
        for (int64_t base = gwarp * ROWS_PER_FENCE; base < a.NvS; base += nWarps * ROWS_PER_FENCE) {
            uint64_t *flags[ROWS_PER_FENCE];
#pragma unroll
            for (int g = 0; g < ROWS_PER_FENCE; ++g) {
                flags[g] = nullptr;
                const int64_t s = base + g;
                if (s >= a.NvS) continue;
                const int32_t v = a.dstLocal[s];
                if (v < 0) continue;
                const int src = v / a.N;
                const int64_t route = v - src * a.N;
                if (src >= comm->rankSize) continue;
                uint8_t *peerHalf = DataHalf(comm, src, epoch);
                CopyLanesDeep(peerHalf + route * a.rowBytes, a.hiddenNvs + s * a.rowBytes, a.rowBytes, lane, 32);
                if (lane == 0 && a.weightsNvs != nullptr) reinterpret_cast<float *>(peerHalf + a.weightWinOff)[route] = a.weightsNvs[s];
                flags[g] = FlagSlot(comm, src, TILEXR_FLAG_SLOT_BASE + route);
            }
            __syncwarp();
            if (lane == 0) {
                fence_acq_rel_sys();
#pragma unroll
                for (int g = 0; g < ROWS_PER_FENCE; ++g) {
                    if (flags[g] != nullptr) st_relaxed_sys_u64(flags[g], MakeFlag(epoch, 1));
                }
            }
        }
        const uint8_t *half = DataHalf(comm, rank, epoch);
        const int vecs = a.rowBytes / 16;
        for (int64_t t = gwarp; t < a.S && w.ok(); t += nWarps) {
            if (lane < K) {
                const int64_t route = t * K + lane;
                WaitFlagGE(w, FlagSlot(comm, rank, TILEXR_FLAG_SLOT_BASE + route), 1, -1, route);
            }
            if (!__all_sync(0xffffffffu, w.ok())) {
                if (w.ok()) w.status = TILEXR_DEV_ABORTED;
                break;
            }
            uint8_t *y = a.hiddenOut + t * a.rowBytes;
            for (int v = lane; v < vecs; v += 32) {
                float acc[8];
                SumRowsColumn(half + static_cast<uint64_t>(t) * K * a.rowBytes, a.rowBytes, K, 0xffffffffu, static_cast<uint64_t>(v), a.elemKind, acc);
                if (a.elemKind == 2) {
                    st_vec16(y + v * 16, Vec16{__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3])});
                } else {
                    st_vec16(y + v * 16, Pack8(acc, a.elemKind == 1));
                }
            }
            if (lane < K && a.weightsOut != nullptr) {
                a.weightsOut[t * K + lane] = reinterpret_cast<const float *>(half + a.weightWinOff)[t * K + lane];
            }
        }
        ok = w.ok();
    }
    ok = BlockBroadcastOk(ok);
    KernelEpilogue(w, ok);
}

// ---- prefetch weight ---------------------------------------------------------------------------------------------
// Slot b of this rank receives the weight rows of expert expertsToCopy[rank][b] from its owner.

__device__ void MoonPrefetchBody(const MoonPrefetchArgs &a)
{
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_PREFETCH, a.B, true);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    constexpr uint64_t CHUNK = 256 * 1024;
    // the owners' weight rows are pulled from their own tensors: not before the owner has entered this launch
    ok = MeetPeersOnEntry(w, comm, rank, comm->rankSize, w.epoch, ok);
    if (ok) {
        // work items: (tensor, slot, chunk), walked by all blocks
        uint64_t item = 0;
        for (int ti = 0; ti < 3; ++ti) {
            const MoonTensorRef &t = a.tensors[ti];
            if (!t.valid) continue;
            const uint64_t chunks = (t.rowBytes + CHUNK - 1) / CHUNK;
            for (int b = 0; b < a.B; ++b) {
                const int e = a.expertsToCopy[rank * a.B + b];
                if (e < 0) continue;
                const int owner = e / a.L;
                const int srcRow = e - owner * a.L;
                const uint8_t *src = comm->registryPtr->regions[t.handle].peerBase[owner] + t.offset + static_cast<uint64_t>(srcRow) * t.rowBytes;
                uint8_t *dst = t.local + static_cast<uint64_t>(a.L + b) * t.rowBytes;
                for (uint64_t c = 0; c < chunks; ++c, ++item) {
                    if (item % gridDim.x != blockIdx.x) continue;
                    const uint64_t off = c * CHUNK;
                    const uint64_t n = min(CHUNK, t.rowBytes - off);
                    CopyLanesDeep(dst + off, src + off, n, threadIdx.x, blockDim.x);     // eight 16-byte loads per thread in flight
                }
            }
        }
    }
    KernelEpilogue(w, ok);
}

// ---- reduce grad ---------------------------------------------------------------------------------------------------
// The owner of expert e adds, in ascending (source rank, slot) order, the gradient rows that
// other ranks accumulated in the slot where they had borrowed e.  When everybody has pulled,
// each rank clears its own slots.

__device__ void MoonReduceGradBody(const MoonReduceGradArgs &a)
{
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_REDUCE_GRAD, a.B, true);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int R = comm->rankSize;
    const uint32_t epoch = w.epoch;
    // the borrowers' gradient slots are pulled from their own tensors: not before the borrower has entered this launch
    ok = MeetPeersOnEntry(w, comm, rank, R, epoch, ok);
    // Who borrowed which of this rank's experts: per local expert the (source rank, slot) pairs in ascending order, built once
    // per block in shared memory (the table has R * B entries; scanning it per vector, as a first version did, kept the
    // kernel at a fifth of the link).
    constexpr int MAX_SOURCES = 2048, MAX_LOCAL = 256;
    __shared__ int sFirst[MAX_LOCAL + 1];
    __shared__ int sSource[MAX_SOURCES];           // source rank << 16 | slot
    const int entries = R * a.B;
    const bool tabled = a.L <= MAX_LOCAL && entries <= MAX_SOURCES;
    if (ok && tabled) {
        for (int l = threadIdx.x; l < a.L; l += blockDim.x) {
            int n = 0;
            for (int i = 0; i < entries; ++i) n += (a.expertsToCopy[i] == rank * a.L + l && i / a.B != rank) ? 1 : 0;
            sFirst[l + 1] = n;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            sFirst[0] = 0;
            for (int l = 0; l < a.L; ++l) sFirst[l + 1] += sFirst[l];
        }
        __syncthreads();
        for (int l = threadIdx.x; l < a.L; l += blockDim.x) {
            int at = sFirst[l];
            for (int i = 0; i < entries; ++i) {
                if (a.expertsToCopy[i] == rank * a.L + l && i / a.B != rank) sSource[at++] = ((i / a.B) << 16) | (i % a.B);
            }
        }
        __syncthreads();
    }
    if (ok && tabled) {
        for (int ti = 0; ti < 3; ++ti) {
            const MoonTensorRef &t = a.tensors[ti];
            if (!t.valid) continue;
            const uint64_t vecsPerRow = t.rowBytes / 16;
            uint8_t *const *peerBase = comm->registryPtr->regions[t.handle].peerBase;
            for (int l = 0; l < a.L; ++l) {
                const int s0 = sFirst[l], s1 = sFirst[l + 1];
                if (s0 == s1) continue;
                uint8_t *dst = t.local + static_cast<uint64_t>(l) * t.rowBytes;
                // four vectors per thread and step: the owner's and every borrower's copy of them are in flight together
                constexpr int U = 4;
                const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
                for (uint64_t v0 = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v0 < vecsPerRow; v0 += stride * U) {
                    float f[U][4];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const uint64_t v = min(v0 + u * stride, vecsPerRow - 1);
                        const Vec16 acc = ld_vec16(dst + v * 16);
                        f[u][0] = __uint_as_float(acc.x);
                        f[u][1] = __uint_as_float(acc.y);
                        f[u][2] = __uint_as_float(acc.z);
                        f[u][3] = __uint_as_float(acc.w);
                    }
                    for (int si = s0; si < s1; ++si) {
                        const int src = sSource[si] >> 16, slot = sSource[si] & 0xffff;
                        const uint8_t *p = peerBase[src] + t.offset + static_cast<uint64_t>(a.L + slot) * t.rowBytes;
                        Vec16 x[U];
#pragma unroll
                        for (int u = 0; u < U; ++u) x[u] = ld_vec16_stream(p + min(v0 + u * stride, vecsPerRow - 1) * 16);
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            f[u][0] += __uint_as_float(x[u].x);
                            f[u][1] += __uint_as_float(x[u].y);
                            f[u][2] += __uint_as_float(x[u].z);
                            f[u][3] += __uint_as_float(x[u].w);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const uint64_t v = v0 + u * stride;
                        if (v < vecsPerRow) {
                            st_vec16(dst + v * 16, Vec16{__float_as_uint(f[u][0]), __float_as_uint(f[u][1]), __float_as_uint(f[u][2]), __float_as_uint(f[u][3])});
                        }
                    }
                }
            }
        }
    } else if (ok) {
        // tables beyond the shared-memory lists: scan the table per vector
        for (int ti = 0; ti < 3; ++ti) {
            const MoonTensorRef &t = a.tensors[ti];
            if (!t.valid) continue;
            const uint64_t vecsPerRow = t.rowBytes / 16;
            for (int l = 0; l < a.L; ++l) {
                const int e = rank * a.L + l;
                bool any = false;
                for (int i = 0; i < entries && !any; ++i) any = a.expertsToCopy[i] == e && i / a.B != rank;
                if (!any) continue;
                uint8_t *dst = t.local + static_cast<uint64_t>(l) * t.rowBytes;
                for (uint64_t v = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecsPerRow;
                     v += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
                    Vec16 acc = ld_vec16(dst + v * 16);
                    float f[4] = {__uint_as_float(acc.x), __uint_as_float(acc.y), __uint_as_float(acc.z), __uint_as_float(acc.w)};
                    for (int i = 0; i < entries; ++i) {
                        if (a.expertsToCopy[i] != e) continue;
                        const int src = i / a.B;
                        const int b = i - src * a.B;
                        if (src == rank) continue;
                        const uint8_t *p = comm->registryPtr->regions[t.handle].peerBase[src] + t.offset +
                                           static_cast<uint64_t>(a.L + b) * t.rowBytes + v * 16;
                        const Vec16 x = ld_vec16_stream(p);
                        f[0] += __uint_as_float(x.x);
                        f[1] += __uint_as_float(x.y);
                        f[2] += __uint_as_float(x.z);
                        f[3] += __uint_as_float(x.w);
                    }
                    st_vec16(dst + v * 16, Vec16{__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])});
                }
            }
        }
    }
    ok = GridBarrier(w, 0) && ok;
    if (a.clearSlots) {
        // tell every peer that this rank has finished reading their slots
        if (ok && blockIdx.x == 0 && static_cast<int>(threadIdx.x) < R) {
            SetFlag(BlockFlag(comm, threadIdx.x, rank, MOONEP_DONE_FLAG_SLOT), epoch, 1);
        }
        bool got = true;
        if (ok && static_cast<int>(threadIdx.x) < R) {
            got = WaitFlagGE(w, BlockFlag(comm, rank, threadIdx.x, MOONEP_DONE_FLAG_SLOT), 1, threadIdx.x, MOONEP_DONE_FLAG_SLOT);
        }
        ok = BlockBroadcastOk(got) && ok;
        if (ok) {
            for (int ti = 0; ti < 3; ++ti) {
                const MoonTensorRef &t = a.tensors[ti];
                if (!t.valid) continue;
                uint8_t *p = t.local + static_cast<uint64_t>(a.L) * t.rowBytes;
                const uint64_t vecs = static_cast<uint64_t>(a.B) * t.rowBytes / 16;
                const Vec16 z{0, 0, 0, 0};
                for (uint64_t v = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs;
                     v += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
                    st_vec16(p + v * 16, z);
                }
            }
        }
    }
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRMoonEpPlannerKernel, PlannerArgs, PlannerBody, MOONEP_THREADS)
TILEXR_DEFINE_KERNEL(TileXRMoonEpDispatchKernel, MoonDispatchArgs, MoonDispatchBody, MOONEP_THREADS)
TILEXR_DEFINE_KERNEL(TileXRMoonEpCombineKernel, MoonCombineArgs, MoonCombineBody, MOONEP_THREADS)
TILEXR_DEFINE_KERNEL(TileXRMoonEpPrefetchKernel, MoonPrefetchArgs, MoonPrefetchBody, MOONEP_THREADS)
TILEXR_DEFINE_KERNEL(TileXRMoonEpReduceGradKernel, MoonReduceGradArgs, MoonReduceGradBody, MOONEP_THREADS)

} // namespace

const KernelEntry &MoonPlannerKernelEntry() { return TileXRMoonEpPlannerKernelEntry; }
const KernelEntry &MoonDispatchKernelEntry() { return TileXRMoonEpDispatchKernelEntry; }
const KernelEntry &MoonCombineKernelEntry() { return TileXRMoonEpCombineKernelEntry; }
const KernelEntry &MoonPrefetchKernelEntry() { return TileXRMoonEpPrefetchKernelEntry; }
const KernelEntry &MoonReduceGradKernelEntry() { return TileXRMoonEpReduceGradKernelEntry; }

size_t MoonPlannerSmemBytes(int experts, int routesPerBlock)
{
    return static_cast<size_t>(routesPerBlock) * 8 + static_cast<size_t>(experts) * 8;
}

} // namespace TileXR
