// Expert-parallel dispatch and combine for sm_100a, plus the local hot ops around them
// (routing top-k, block-scaled fp8 quantisation, MXFP8, RMSNorm).
//
// Dispatch, one cooperative kernel per rank:
//   1. every block takes a contiguous range of tokens, routes them (top-k over the gate logits,
//      or reads the given expert ids and masks), and ranks its routes per expert in (token, k)
//      order; per-block expert counts go to a scratch table;
//   2. blocks also add their counts to the rank's totals; the block that finishes last pushes the totals
//      to every peer as epoch-tagged 16-byte units (an all-gather of R x E integers without fence or
//      flag), and a block goes on as soon as the blocks before it have written their counts (no grid
//      barrier).  With everybody's counts each rank computes, for itself as a sender, the exact row at
//      which each of its routes lands in the destination's expert-major / source-major layout: rows are
//      placed at their FINAL position by the sender, the receiver never sorts or compacts;
//   3. a warp per token quantises the row once (fp8 e4m3, one fp32 scale per 128 elements, kept
//      in registers) and stores it to each destination together with its scales and the assist
//      tuple; when the block is done it raises one flag per destination;
//   4. the receiver waits for the flags of every sender block and copies rows, scales and
//      tuples from its window to the output tensors (rows are skipped when the output tensor
//      is registered and was written directly).
// The reference reaches the same layout with worst-case regions per (source, expert) and a
// receiver-side compaction (src/ep/kernels/tilexr_ep_dispatch_memory_kernel.h:666-708,
// 903-1140, 1190-1317); at 4096 tokens x 8 routes that needs gigabytes of window, hence the
// count-first placement here.
//
// Combine: a warp per received row pushes it to slot (token, k) of the source's window and
// raises that slot's flag; a warp per token waits for its K flags and accumulates
// weight_k * row_k in fp32 in k order, then rounds once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>
#include <cuda_runtime_api.h>

#include "device/tilexr_data_as_flag.cuh"
#include "device/tilexr_perf_trace.cuh"
#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "device/tilexr_convert.cuh"
#include "ep_kernels.cuh"
#include "tilexr_ep.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr float FP8_E4M3_MAX = 448.0f;
constexpr float FP8_AMAX_FLOOR = 1e-4f;

__device__ __forceinline__ float WarpMax(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float WarpSum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint32_t Fp8x4(float a, float b, float c, float d)
{
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ uint32_t Fp8x4E5m2(float a, float b, float c, float d)
{
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E5M2);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E5M2);
    return lo | (hi << 16);
}

// ---- routing: one warp scores one token and picks its top-k -------------------------------------------
// Lane l owns experts l, l+32, ...  Selection is by score (+ optional bias), ties go to the
// lower expert id; the gate weight is the unbiased score, optionally renormalised over the
// selected experts and multiplied by `routedScale`.
template <int PER_LANE>
__device__ __forceinline__ void RouteTokenN(const float *logits, const float *bias, int numExperts, int topK, int scoreFunc,
                                            int renormalize, float routedScale, int lane, int32_t *idsOut, float *weightsOut)
{
    float score[PER_LANE];
    float sel[PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        const int e = j * 32 + lane;
        score[j] = e < numExperts ? logits[e] : -INFINITY;
        mx = fmaxf(mx, score[j]);
    }
    if (scoreFunc == TileXREp::TILEXR_EP_SCORE_SOFTMAX) {
        mx = WarpMax(mx);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            const int e = j * 32 + lane;
            score[j] = e < numExperts ? expf(score[j] - mx) : 0.f;
            sum += score[j];
        }
        sum = WarpSum(sum);
        const float inv = 1.0f / sum;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) score[j] *= inv;
    } else {
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            const int e = j * 32 + lane;
            score[j] = e < numExperts ? 1.0f / (1.0f + expf(-score[j])) : 0.f;
        }
    }
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        const int e = j * 32 + lane;
        sel[j] = e < numExperts ? score[j] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
    }
    float myWeight = 0.f;   // lane k keeps the k-th pick
    int myId = -1;
    float total = 0.f;
    for (int k = 0; k < topK; ++k) {
        float best = -INFINITY;
        int bestE = 0x7fffffff;
        float bestScore = 0.f;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            const int e = j * 32 + lane;
            if (sel[j] > best) {   // ascending e within a lane: first maximum wins the tie
                best = sel[j];
                bestE = e;
                bestScore = score[j];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, bestE, o);
            const float os = __shfl_xor_sync(0xffffffffu, bestScore, o);
            if (ob > best || (ob == best && oe < bestE)) {
                best = ob;
                bestE = oe;
                bestScore = os;
            }
        }
        if ((bestE & 31) == lane) {
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j) {
                if (j == (bestE >> 5)) sel[j] = -INFINITY;
            }
        }
        if (lane == k) {
            myWeight = bestScore;
            myId = bestE;
        }
        total += bestScore;
    }
    if (lane < topK) {
        float w = myWeight;
        if (renormalize) w = w / total;
        w *= routedScale;
        idsOut[lane] = myId;
        weightsOut[lane] = w;
    }
}

// The per-lane score table is sized for the expert count, so that 256 experts keep 8 scores per lane in
// registers instead of the 32 that the largest supported count needs.
__device__ __forceinline__ void RouteToken(const float *logits, const float *bias, int numExperts, int topK, int scoreFunc,
                                           int renormalize, float routedScale, int lane, int32_t *idsOut, float *weightsOut)
{
    if (numExperts <= 256) {
        RouteTokenN<8>(logits, bias, numExperts, topK, scoreFunc, renormalize, routedScale, lane, idsOut, weightsOut);
    } else if (numExperts <= 512) {
        RouteTokenN<16>(logits, bias, numExperts, topK, scoreFunc, renormalize, routedScale, lane, idsOut, weightsOut);
    } else {
        RouteTokenN<EP_MAX_EXPERTS / 32>(logits, bias, numExperts, topK, scoreFunc, renormalize, routedScale, lane, idsOut,
                                         weightsOut);
    }
}

__global__ void __launch_bounds__(256) RoutingTopKKernel(const RoutingArgs a)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32;
    const int lane = threadIdx.x & 31;
    if (warp >= a.bs) return;
    RouteToken(a.gateLogits + static_cast<int64_t>(warp) * a.numExperts, a.selectionBias, a.numExperts, a.topK, a.scoreFunc,
               a.renormalize, a.routedScale, lane, a.topkIdsOut + static_cast<int64_t>(warp) * a.topK,
               a.topkWeightsOut + static_cast<int64_t>(warp) * a.topK);
}

// ---- dispatch ---------------------------------------------------------------------------------------------

struct DispatchSmem {
    int32_t *routeExpert;   // [routesPerBlock]  expert id or -1
    int32_t *routeRank;     // [routesPerBlock]  rank among the block's routes to the same expert
    int32_t *hist;          // [E] routes of this block per expert
    int32_t *blockBase;     // [E] routes of earlier blocks per expert
    int32_t *total;         // [E] routes of all sources per expert
    int32_t *dstRow;        // [E] first row, at the owner, of (expert, this source)
    float *scaleStage;      // [EP_WARPS][64]
};

__device__ __forceinline__ DispatchSmem CarveSmem(uint8_t *base, int numExperts, int routesPerBlock)
{
    DispatchSmem s;
    s.routeExpert = reinterpret_cast<int32_t *>(base);
    s.routeRank = s.routeExpert + routesPerBlock;
    s.hist = s.routeRank + routesPerBlock;
    s.blockBase = s.hist + numExperts;
    s.total = s.blockBase + numExperts;
    s.dstRow = s.total + numExperts;
    s.scaleStage = reinterpret_cast<float *>(s.dstRow + numExperts);
    return s;
}

// out[e] = sum over blocks b in [0, nb) of counts[b * E + e], by all threads of the block.  With E a multiple
// of four a thread adds 16-byte vectors of several rows, so the chain of dependent loads is nb / (threads /
// (E / 4)) long instead of nb.
__device__ void SumBlockCounts(const int32_t *counts, int E, int nb, int32_t *out, int tid, int nThreads)
{
    for (int e = tid; e < E; e += nThreads) out[e] = 0;
    __syncthreads();
    if ((E & 3) == 0) {
        const int vecPerRow = E / 4;
        const int rowsPar = max(1, nThreads / vecPerRow);
        for (int idx = tid; idx < vecPerRow * rowsPar; idx += nThreads) {
            const int col = idx % vecPerRow;
            int4 acc = make_int4(0, 0, 0, 0);
#pragma unroll 4
            for (int b = idx / vecPerRow; b < nb; b += rowsPar) {
                const int4 v = *reinterpret_cast<const int4 *>(counts + static_cast<int64_t>(b) * E + col * 4);
                acc.x += v.x;
                acc.y += v.y;
                acc.z += v.z;
                acc.w += v.w;
            }
            atomicAdd(&out[col * 4 + 0], acc.x);
            atomicAdd(&out[col * 4 + 1], acc.y);
            atomicAdd(&out[col * 4 + 2], acc.z);
            atomicAdd(&out[col * 4 + 3], acc.w);
        }
    } else {
        for (int e = tid; e < E; e += nThreads) {
            int c = 0;
            for (int b = 0; b < nb; ++b) c += counts[static_cast<int64_t>(b) * E + e];
            out[e] = c;
        }
    }
    __syncthreads();
}

// Stage names of the profiler as the EP kernels use them: chunk_total = routing and counting (dispatch) or
// nothing (combine); chunk_barrier = wait for the earlier blocks' counts; post_sync = count exchange and row placement;
// local_input_to_ipc = rows pushed to their destinations; flag_poll_wait = waiting for arrivals;
// peer_ipc_to_output = window to output (dispatch) or the weighted reduction (combine).
__device__ void EpDispatchBody(const EpDispatchArgs &a)
{
    extern __shared__ __align__(16) uint8_t smemRaw[];
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_EP_DISPATCH, a.bs, true);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int R = comm->rankSize;
    const int E = a.numExperts;          // routed experts (what the router chooses from)
    const int C = a.numCols;             // columns of the count tables: shared ranks first, then the routed experts
    const int K = a.topK;
    const int KR = K + a.topo.sharedExperts;   // routes per token: top-k and one per shared expert
    const int G = gridDim.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const uint32_t epoch = w.epoch;
    const int routesPerBlock = static_cast<int>(a.tokensPerBlock) * KR;
    // the tables also serve as scratch for the final scan over (local expert, source): moePerRank * R numbers
    DispatchSmem sm = CarveSmem(smemRaw, max(C, a.topo.moePerRank * R), routesPerBlock);
    uint8_t *myHalf = DataHalf(comm, rank, epoch);
    PerfScope perf = PerfInit(tid == 0 ? a.perfTrace : nullptr, static_cast<uint32_t>(rank), blockIdx.x);
    PerfStageBegin(perf, TILEXR_PERF_KERNEL_TOTAL);
    PerfStageBegin(perf, TILEXR_PERF_CHUNK_TOTAL);
    int32_t *blockCounts = reinterpret_cast<int32_t *>(myHalf + a.win.blockCountOff);
    // operator scratch of the rank's control block (tilexr_comm_args.h): a count of the blocks that have finished
    // counting and the rank's totals per column, both back to zero when the launch ends; and one word per
    // block that holds the epoch of the launch whose histogram the block has written (never cleared)
    uint32_t *doneBlocks = reinterpret_cast<uint32_t *>(CtrlWord(comm, rank, TILEXR_CTRL_SCRATCH_WORD + EP_SCRATCH_DONE_WORD));
    uint32_t *totals = reinterpret_cast<uint32_t *>(CtrlWord(comm, rank, TILEXR_CTRL_SCRATCH_WORD + EP_SCRATCH_TOTALS_WORD));
    uint32_t *histReady = reinterpret_cast<uint32_t *>(CtrlWord(comm, rank, TILEXR_CTRL_SCRATCH_WORD + EP_SCRATCH_READY_WORD));
    int32_t *srcBlocks = reinterpret_cast<int32_t *>(sm.scaleStage);       // [R] blocks of each source that raise a flag
    const int units = (C + 1 + 2) / 3;           // 16-byte units of one source's counts: C counts and its block count
    const uint8_t *llMine = LlHalf(comm, rank, epoch);
    __shared__ int sIsLast;

    const int t0 = min(a.bs, static_cast<int>(blockIdx.x * a.tokensPerBlock));
    const int t1 = min(a.bs, t0 + static_cast<int>(a.tokensPerBlock));
    const int nTok = t1 - t0;
    const int nRoutes = nTok * KR;

    // ---- 1. route, rank, count (routeExpert holds the COLUMN of a route, -1 when inactive) ---------------
    for (int e = tid; e < C; e += blockDim.x) sm.hist[e] = 0;
    for (int i = warp; i < nTok; i += EP_WARPS) {
        const int t = t0 + i;
        if (a.gateLogits != nullptr) {
            RouteToken(a.gateLogits + static_cast<int64_t>(t) * E, a.selectionBias, E, K, a.scoreFunc, a.renormalize,
                       a.routedScale, lane, a.topkIdsOut + static_cast<int64_t>(t) * K,
                       a.topkWeightsOut + static_cast<int64_t>(t) * K);
            __syncwarp();
        }
        if (lane < K) {
            const int32_t *ids = a.gateLogits != nullptr ? a.topkIdsOut : a.expertIds;
            int e = ids[static_cast<int64_t>(t) * K + lane];
            if (e < 0 || e >= E) e = -1;
            if (a.maskType == TileXREp::TILEXR_EP_ACTIVE_MASK_TOKEN && a.activeMask[t] == 0) e = -1;
            if (a.maskType == TileXREp::TILEXR_EP_ACTIVE_MASK_EXPERT && a.activeMask[static_cast<int64_t>(t) * K + lane] == 0) e = -1;
            sm.routeExpert[i * KR + lane] = e >= 0 ? a.topo.sharedRanks + e : -1;
            if (a.gateLogits == nullptr && a.topkIdsOut != nullptr) a.topkIdsOut[static_cast<int64_t>(t) * K + lane] = e;
        } else if (lane < KR) {
            // every active token also goes to its copy of each shared expert
            const bool active = !(a.maskType == TileXREp::TILEXR_EP_ACTIVE_MASK_TOKEN && a.activeMask[t] == 0);
            sm.routeExpert[i * KR + lane] = active ? EpSharedCol(a.topo, rank, lane - K) : -1;
        }
    }
    __syncthreads();
    // Rank of each route among the block's routes to the same column, in (token, k) order: one warp walks the
    // routes 32 at a time; lanes with the same column find one another with a match and the last of them
    // moves the column's running count on.
    if (warp == 0) {
        for (int base = 0; base < nRoutes; base += 32) {
            const int i = base + lane;
            const int e = i < nRoutes ? sm.routeExpert[i] : -1;
            const uint32_t same = __match_any_sync(0xffffffffu, e);
            int r = 0;
            if (e >= 0) r = sm.hist[e] + __popc(same & ((1u << lane) - 1u));
            __syncwarp();
            if (e >= 0 && (same & ~((2u << lane) - 1u)) == 0) sm.hist[e] += __popc(same);
            __syncwarp();
            if (i < nRoutes) sm.routeRank[i] = r;
        }
    }
    __syncthreads();
    for (int e = tid; e < C; e += blockDim.x) {
        const int hcount = sm.hist[e];
        blockCounts[static_cast<int64_t>(blockIdx.x) * C + e] = hcount;
        if (hcount != 0) atomicAdd(&totals[e], static_cast<uint32_t>(hcount));
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        st_release_gpu_u32(&histReady[blockIdx.x], epoch);
        sIsLast = atom_add_acq_rel_gpu_u32(doneBlocks, 1u) == static_cast<uint32_t>(G) - 1u ? 1 : 0;
    }
    __syncthreads();
    PerfStageEnd(perf, TILEXR_PERF_CHUNK_TOTAL);
    PerfStageBegin(perf, TILEXR_PERF_POST_SYNC);

    // ---- 2. publish this rank's counts, learn everybody's ----------------------------------------------
    // The block that finishes counting last has the rank's totals in front of it and sends them to every
    // peer as self-validating 16-byte units (three counts and the epoch): no fence, no flag, one NVLink
    // crossing.  Nobody waits at a barrier: a block only needs the histograms of the blocks before it.
    if (ok && sIsLast != 0) {
        for (int u = tid; u < units; u += blockDim.x) {
            uint32_t v[3];
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const int idx = u * 3 + q;
                v[q] = idx < C ? __ldcg(&totals[idx]) : (idx == C ? static_cast<uint32_t>(G) : 0u);
            }
            for (int i = 0; i < R; ++i) {
                const int peer = (rank + i) % R;
                Ll16SendUnit(LlHalf(comm, peer, epoch) + (static_cast<uint64_t>(rank) * units + u) * LL16_UNIT_BYTES, v[0], v[1], v[2], epoch);
            }
        }
    }
    PerfStageBegin(perf, TILEXR_PERF_CHUNK_BARRIER);
    {
        bool got = true;
        for (int b = tid; ok && got && b < static_cast<int>(blockIdx.x); b += blockDim.x) {
            uint32_t polls = 0;
            while (ld_acquire_gpu_u32(&histReady[b]) != epoch) {
                if ((++polls & 63u) == 0) {
                    const uint64_t t = now_ns();
                    if (w.deadline == 0) {
                        w.deadline = t + w.args->waitTimeoutNs;
                    } else if (t > w.deadline || AbortRaised(w)) {
                        RaiseFailure(w, TILEXR_DEV_GRID_BARRIER_TIMEOUT, rank, b, epoch, histReady[b]);
                        got = false;
                        break;
                    }
                }
                spin_pause();
            }
        }
        ok = BlockBroadcastOk(got) && ok;
    }
    PerfStageEnd(perf, TILEXR_PERF_CHUNK_BARRIER);
    SumBlockCounts(blockCounts, C, ok ? static_cast<int>(blockIdx.x) : 0, sm.blockBase, tid, blockDim.x);
    for (int e = tid; e < C; e += blockDim.x) {
        sm.total[e] = 0;
        sm.hist[e] = 0;       // from here on: routes of lower ranks to column e
    }
    __syncthreads();
    {
        bool got = true;
        for (int u = tid; ok && got && u < R * units; u += blockDim.x) {
            const int s = u / units;
            const int j = u - s * units;
            Vec16 v;
            got = Ll16WaitUnit(w, llMine + static_cast<uint64_t>(u) * LL16_UNIT_BYTES, s, u, &v);
            if (!got) break;
            const uint32_t vals[3] = {v.x, v.y, v.z};
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const int idx = j * 3 + q;
                if (idx < C) {
                    if (vals[q] != 0) {
                        atomicAdd(&sm.total[idx], static_cast<int32_t>(vals[q]));
                        if (s < rank) atomicAdd(&sm.hist[idx], static_cast<int32_t>(vals[q]));
                    }
                } else if (idx == C) {
                    srcBlocks[s] = static_cast<int32_t>(vals[q]);
                }
            }
        }
        ok = BlockBroadcastOk(got) && ok;
    }
    if (ok) {
        for (int e = tid; e < C; e += blockDim.x) {
            const int first = EpRankFirstCol(a.topo, EpColRank(a.topo, e));
            int row = sm.hist[e];
            for (int p = first; p < e; ++p) row += sm.total[p];
            sm.dstRow[e] = row;
        }
        // Every rank sees the same counts, so every rank reaches the same verdict on overflow.
        bool fits = true;
        if (tid < R) {
            int64_t rows = 0;
            const int firstCol = EpRankFirstCol(a.topo, tid);
            for (int e = firstCol; e < firstCol + EpRankCols(a.topo, tid); ++e) rows += sm.total[e];
            fits = rows <= static_cast<int64_t>(a.maxRecvRows);
            if (!fits) RaiseFailure(w, TILEXR_DEV_BAD_ARGUMENT, tid, 0, a.maxRecvRows, static_cast<uint64_t>(rows));
        }
        ok = BlockBroadcastOk(fits);
    }

    PerfStageEnd(perf, TILEXR_PERF_POST_SYNC);

    // ---- 3. send ----------------------------------------------------------------------------------------
    PerfStageBegin(perf, TILEXR_PERF_LOCAL_INPUT_TO_IPC);
    if (ok) {
        const bool bf16 = a.isBf16 != 0;
        const bool mx = a.quantMode == TileXREp::TILEXR_EP_QUANT_MXFP8_E4M3 || a.quantMode == TileXREp::TILEXR_EP_QUANT_MXFP8_E5M2;
        const bool mxE5m2 = a.quantMode == TileXREp::TILEXR_EP_QUANT_MXFP8_E5M2;
        const bool quant = mx || a.quantMode == TileXREp::TILEXR_EP_QUANT_FP8_1X128;
        const bool int8Dynamic = a.quantMode == TileXREp::TILEXR_EP_QUANT_DYNAMIC_INT8;
        const bool int8Mode = int8Dynamic || a.quantMode == TileXREp::TILEXR_EP_QUANT_STATIC_INT8;
        const int chunks = a.h / 16;             // 16 elements per lane and iteration (fp8 paths)
        const int iters = (chunks + 31) / 32;
        // A block with few tokens (small batches) cuts every token into column ranges for several warps.
        const int parts = nTok > 0 ? max(1, min(min(8, iters), static_cast<int>(EP_WARPS) / nTok)) : 1;
        for (int item = warp; item < nTok * parts; item += EP_WARPS) {
            const int i = item / parts;
            const int part = item % parts;
            const int t = t0 + i;
            const uint8_t *row = a.x + static_cast<int64_t>(t) * a.h * a.elemSize;
            // lane k owns route k of this token: where its row, scales and tuple go
            unsigned long long myPayload = 0, myHalf = 0;
            uint32_t myRow = 0;
            int myExpert = -1;
            if (lane < KR) {
                const int e = sm.routeExpert[i * KR + lane];
                if (e >= 0) {
                    const int dst = EpColRank(a.topo, e);
                    myRow = static_cast<uint32_t>(sm.dstRow[e] + sm.blockBase[e] + sm.routeRank[i * KR + lane]);
                    uint8_t *half = DataHalf(comm, dst, epoch);
                    uint8_t *payload = a.zeroCopy
                                           ? comm->registryPtr->regions[a.outHandle].peerBase[dst] + a.outOffset +
                                                 static_cast<uint64_t>(myRow) * a.win.rowBytes
                                           : half + a.win.payloadOff + static_cast<uint64_t>(myRow) * a.win.rowBytes;
                    myPayload = reinterpret_cast<unsigned long long>(payload);
                    myHalf = reinterpret_cast<unsigned long long>(half);
                    myExpert = e;
                }
            }
            if (lane < KR && a.routeRowsOut != nullptr && part == 0) {
                a.routeRowsOut[static_cast<int64_t>(t) * KR + lane] = myExpert >= 0 ? static_cast<int32_t>(myRow) : -1;
            }
            const uint32_t routes = __ballot_sync(0xffffffffu, myExpert >= 0);
            if (routes == 0) continue;
            // Routes of this token to one remote rank form a group: the lowest k (the head) carries the
            // payload, the others only their tuple, and every member links to the next one.
            const int myDst = myExpert >= 0 ? EpColRank(a.topo, myExpert) : -1;
            uint32_t myLink = 0;
            if (a.dedup != 0) {
                bool follower = false;
                for (int j = 0; j < KR; ++j) {
                    const int dj = __shfl_sync(0xffffffffu, myDst, j);
                    const uint32_t rj = __shfl_sync(0xffffffffu, myRow, j);
                    if (dj >= 0 && dj == myDst && myDst != rank) {
                        if (j < lane) follower = true;
                        else if (j > lane && myLink == 0) myLink = rj + 1;
                    }
                }
                if (follower) myLink |= EP_LINK_FOLLOWER;
            }
            const uint32_t payloadRoutes = __ballot_sync(0xffffffffu, myExpert >= 0 && (myLink & EP_LINK_FOLLOWER) == 0);
            if (int8Mode) {
                // int8 with optional per-expert smoothing scales: every route is quantised for its own expert.
                // dynamic: one pass for the row's amax (scale = amax / 127, stored beside the row), one to convert;
                // static: the caller's scales already map into int8 range.
                uint32_t m = payloadRoutes;
                while (m != 0) {
                    const int k = __ffs(m) - 1;
                    m &= m - 1;
                    uint8_t *p = reinterpret_cast<uint8_t *>(__shfl_sync(0xffffffffu, myPayload, k));
                    uint8_t *half = reinterpret_cast<uint8_t *>(__shfl_sync(0xffffffffu, myHalf, k));
                    const uint32_t rr = __shfl_sync(0xffffffffu, myRow, k);
                    const int e = __shfl_sync(0xffffffffu, myExpert, k);
                    const float *sc = (a.quantScales != nullptr && e >= a.topo.sharedRanks)
                                          ? a.quantScales + static_cast<int64_t>(e - a.topo.sharedRanks) * a.h : nullptr;
                    float inv = 1.0f;
                    if (int8Dynamic) {
                        float amax = 0.f;
                        for (int it = 0; it < iters; ++it) {
                            const int c = it * 32 + lane;
                            if (c < chunks) {
                                float f[16];
                                Unpack8(ld_vec16(row + static_cast<int64_t>(c) * 32), bf16, f);
                                Unpack8(ld_vec16(row + static_cast<int64_t>(c) * 32 + 16), bf16, f + 8);
#pragma unroll
                                for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(sc != nullptr ? f[j] * sc[c * 16 + j] : f[j]));
                            }
                        }
                        amax = WarpMax(amax);
                        if (amax > 0.f) inv = 127.0f / amax;
                        if (part == 0 && lane == 0) {
                            st_vec16(half + a.win.scalesOff + static_cast<uint64_t>(rr) * a.win.scaleRowBytes,
                                     Vec16{__float_as_uint(amax > 0.f ? amax / 127.0f : 1.0f), 0u, 0u, 0u});
                        }
                    }
                    for (int it = part; it < iters; it += parts) {
                        const int c = it * 32 + lane;
                        if (c >= chunks) continue;
                        float f[16];
                        Unpack8(ld_vec16(row + static_cast<int64_t>(c) * 32), bf16, f);
                        Unpack8(ld_vec16(row + static_cast<int64_t>(c) * 32 + 16), bf16, f + 8);
                        uint32_t wds[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float v = (sc != nullptr ? f[j] * sc[c * 16 + j] : f[j]) * inv;
                            const int q = max(-128, min(127, __float2int_rn(v)));
                            wds[j >> 2] |= static_cast<uint32_t>(q & 0xff) << (8 * (j & 3));
                        }
                        st_vec16(p + static_cast<int64_t>(c) * 16, Vec16{wds[0], wds[1], wds[2], wds[3]});
                    }
                }
            } else if (quant) {
                // each 512-element chunk is quantised once and stored to every destination right away:
                // nothing row-sized lives in registers, so two blocks fit on an SM
#pragma unroll 2
                for (int it = part; it < iters; it += parts) {
                    const int c = it * 32 + lane;
                    float f[16];
                    if (c < chunks) {
                        Unpack8(ld_vec16(row + static_cast<int64_t>(c) * 32), bf16, f);
                        Unpack8(ld_vec16(row + static_cast<int64_t>(c) * 32 + 16), bf16, f + 8);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) f[j] = 0.f;
                    }
                    float amax = 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
                    if (mx) {
                        // MXFP8: 32 elements = 2 lanes share the exponent 2^(floor(log2 amax) - emax); this
                        // iteration's 16 exponent bytes are 16 bytes of the scale row
                        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                        const int emax = mxE5m2 ? 15 : 8;
                        int ex = -127;
                        if (amax > 0.f) {
                            const uint32_t biased = (__float_as_uint(amax) >> 23) & 0xffu;
                            ex = (biased == 0 ? -126 : static_cast<int>(biased) - 127) - emax;
                        }
                        ex = max(-127, min(127, ex));
                        const float inv = exp2f(static_cast<float>(-ex));
                        uint32_t word = (lane & 1) == 0 ? static_cast<uint32_t>(ex + 127) << (8 * ((lane >> 1) & 3)) : 0u;
                        word |= __shfl_xor_sync(0xffffffffu, word, 2);
                        word |= __shfl_xor_sync(0xffffffffu, word, 4);
                        Vec16 sv;
                        sv.x = __shfl_sync(0xffffffffu, word, 0);
                        sv.y = __shfl_sync(0xffffffffu, word, 8);
                        sv.z = __shfl_sync(0xffffffffu, word, 16);
                        sv.w = __shfl_sync(0xffffffffu, word, 24);
                        if ((payloadRoutes >> lane) & 1u) {
                            st_vec16(reinterpret_cast<uint8_t *>(myHalf) + a.win.scalesOff +
                                         static_cast<uint64_t>(myRow) * a.win.scaleRowBytes + it * 16,
                                     sv);
                        }
                        Vec16 q;
                        if (mxE5m2) {
                            q.x = Fp8x4E5m2(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                            q.y = Fp8x4E5m2(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                            q.z = Fp8x4E5m2(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
                            q.w = Fp8x4E5m2(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
                        } else {
                            q.x = Fp8x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                            q.y = Fp8x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                            q.z = Fp8x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
                            q.w = Fp8x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
                        }
                        uint32_t m = payloadRoutes;
                        while (m != 0) {
                            const int k = __ffs(m) - 1;
                            m &= m - 1;
                            uint8_t *p = reinterpret_cast<uint8_t *>(__shfl_sync(0xffffffffu, myPayload, k));
                            if (c < chunks) st_vec16(p + static_cast<int64_t>(c) * 16, q);
                        }
                        continue;
                    }
                    // 128 elements = 8 consecutive lanes
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                    amax = fmaxf(amax, FP8_AMAX_FLOOR);
                    const float inv = FP8_E4M3_MAX / amax;
                    // the four scales of this iteration are 16 bytes of the scale row: lane k stores them for route k
                    const float scale = amax / FP8_E4M3_MAX;
                    Vec16 sv;
                    sv.x = __float_as_uint(__shfl_sync(0xffffffffu, scale, 0));
                    sv.y = __float_as_uint(__shfl_sync(0xffffffffu, scale, 8));
                    sv.z = __float_as_uint(__shfl_sync(0xffffffffu, scale, 16));
                    sv.w = __float_as_uint(__shfl_sync(0xffffffffu, scale, 24));
                    if ((payloadRoutes >> lane) & 1u) {
                        st_vec16(reinterpret_cast<uint8_t *>(myHalf) + a.win.scalesOff +
                                     static_cast<uint64_t>(myRow) * a.win.scaleRowBytes + it * 16,
                                 sv);
                    }
                    Vec16 q;
                    q.x = Fp8x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                    q.y = Fp8x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                    q.z = Fp8x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
                    q.w = Fp8x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
                    uint32_t m = payloadRoutes;
                    while (m != 0) {
                        const int k = __ffs(m) - 1;
                        m &= m - 1;
                        uint8_t *p = reinterpret_cast<uint8_t *>(__shfl_sync(0xffffffffu, myPayload, k));
                        if (c < chunks) st_vec16(p + static_cast<int64_t>(c) * 16, q);
                    }
                }
            } else {
                const uint64_t perPart = ((a.win.rowBytes + parts - 1) / parts + 511) & ~511ull;
                const uint64_t b0 = min(static_cast<uint64_t>(a.win.rowBytes), perPart * part);
                const uint64_t nBytes = min(static_cast<uint64_t>(a.win.rowBytes) - b0, perPart);
                uint32_t m = payloadRoutes;
                while (m != 0) {
                    const int k = __ffs(m) - 1;
                    m &= m - 1;
                    uint8_t *p = reinterpret_cast<uint8_t *>(__shfl_sync(0xffffffffu, myPayload, k));
                    if (nBytes > 0) CopyLanes(p + b0, row + b0, nBytes, lane, 32);
                }
            }
            if (myExpert >= 0 && part == 0) {
                st_vec16(reinterpret_cast<uint8_t *>(myHalf) + a.win.assistOff + static_cast<uint64_t>(myRow) * 16,
                         Vec16{static_cast<uint32_t>(rank), static_cast<uint32_t>(t), static_cast<uint32_t>(lane),
                               static_cast<uint32_t>(lane < K ? myExpert - a.topo.sharedRanks : lane - K)});   // routed expert id, or shared expert id
                const int64_t route = static_cast<int64_t>(t) * K + lane;
                const float wgt = lane >= K ? 1.0f
                                  : a.gateLogits != nullptr ? a.topkWeightsOut[route]
                                                            : (a.expertScales != nullptr ? a.expertScales[route] : 1.0f);
                *reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(myHalf) + a.win.extOff + static_cast<uint64_t>(myRow) * 8) =
                    make_uint2(myLink, __float_as_uint(wgt));
            }
            __syncwarp();
        }
    }
    __syncthreads();
    if (ok && tid < R) {
        SetFlag(FlagSlot(comm, tid, TILEXR_FLAG_OP_BASE + static_cast<int64_t>(rank) * TILEXR_FLAGS_PER_PAIR + blockIdx.x), epoch, 1);
    }
    PerfStageEnd(perf, TILEXR_PERF_LOCAL_INPUT_TO_IPC, static_cast<uint64_t>(nRoutes) * a.win.rowBytes);

    // ---- 4. receive ---------------------------------------------------------------------------------------
    PerfStageBegin(perf, TILEXR_PERF_FLAG_POLL_WAIT);
    {
        // every thread polls its share of the (source, block) flags; a source's block count came with its counts
        bool got = true;
        if (ok) {
            for (int s = 0; s < R && got; ++s) {
                const int64_t base = TILEXR_FLAG_OP_BASE + static_cast<int64_t>(s) * TILEXR_FLAGS_PER_PAIR;
                const int blocksOfS = min(srcBlocks[s], static_cast<int>(EP_COUNT_FLAG_SLOT));
                for (int b = tid; b < blocksOfS && got; b += blockDim.x) {
                    got = WaitFlagGE(w, FlagSlot(comm, rank, base + b), 1, s, base + b);
                }
            }
        }
        ok = BlockBroadcastOk(got) && ok;
    }
    PerfStageEnd(perf, TILEXR_PERF_FLAG_POLL_WAIT);
    PerfStageBegin(perf, TILEXR_PERF_PEER_IPC_TO_OUTPUT);
    if (ok) {
        const int firstLocal = EpRankFirstCol(a.topo, rank);
        const int localCols = EpRankCols(a.topo, rank);
        int64_t rows = 0;
        for (int e = firstLocal; e < firstLocal + localCols; ++e) rows += sm.total[e];
        // Rows are dealt out to blocks in chunks of one row per thread.  Per chunk: (a) a thread per row copies
        // the tuple, link and weight and notes the head rows that have followers; (b) a thread per 16 bytes
        // copies the scales of the rows that arrived with a payload; (c) without zero-copy a warp per row moves
        // the payload out of the window; (d) warps take the noted head rows in turn and fill their followers.
        const bool quantOut = a.win.scaleRowBytes != 0 && a.dynamicScalesOut != nullptr;
        const bool scalarScale = a.quantMode == TileXREp::TILEXR_EP_QUANT_DYNAMIC_INT8;     // one fp32 per row in the output
        const uint8_t *winPayload = myHalf + a.win.payloadOff;
        const uint8_t *winScales = myHalf + a.win.scalesOff;
        const uint8_t *winExt = myHalf + a.win.extOff;
        __shared__ int32_t sHead[EP_BLOCK_THREADS];
        __shared__ int sHeadCount;
        const int scaleVecsPerRow = static_cast<int>(a.win.scaleRowBytes / 16);
        // a chunk is as small as it takes to give every block rows (32 at least), and one row per thread at most
        const int64_t chunk = min(static_cast<int64_t>(EP_BLOCK_THREADS), max(static_cast<int64_t>(32), static_cast<int64_t>(((rows + G - 1) / G + 31) & ~static_cast<int64_t>(31))));
        for (int64_t base = static_cast<int64_t>(blockIdx.x) * chunk; base < rows; base += static_cast<int64_t>(G) * chunk) {
            const int chunkRows = static_cast<int>(min(chunk, rows - base));
            if (tid == 0) sHeadCount = 0;
            __syncthreads();
            if (tid < chunkRows) {
                const int64_t r = base + tid;
                const uint2 ext = *reinterpret_cast<const uint2 *>(winExt + r * 8);
                st_vec16(reinterpret_cast<uint8_t *>(a.assistOut) + r * 16, ld_vec16(myHalf + a.win.assistOff + r * 16));
                if (a.assistExtOut != nullptr) *reinterpret_cast<uint2 *>(a.assistExtOut + r * 2) = ext;
                if (a.expandScalesOut != nullptr) a.expandScalesOut[r] = __uint_as_float(ext.y);
                if (a.dedup != 0 && (ext.x & EP_LINK_FOLLOWER) == 0 && (ext.x & EP_LINK_NEXT_MASK) != 0) {
                    sHead[atomicAdd(&sHeadCount, 1)] = tid;
                }
            }
            if (quantOut) {
                for (int idx = tid; idx < chunkRows * scaleVecsPerRow; idx += EP_BLOCK_THREADS) {
                    const int64_t r = base + idx / scaleVecsPerRow;
                    const int v = idx % scaleVecsPerRow;
                    if ((reinterpret_cast<const uint2 *>(winExt + r * 8)->x & EP_LINK_FOLLOWER) != 0) continue;
                    if (scalarScale) {
                        a.dynamicScalesOut[r] = *reinterpret_cast<const float *>(winScales + r * a.win.scaleRowBytes);
                        continue;
                    }
                    st_vec16(reinterpret_cast<uint8_t *>(a.dynamicScalesOut) + r * a.win.scaleRowBytes + v * 16,
                             ld_vec16(winScales + r * a.win.scaleRowBytes + v * 16));
                }
            }
            if (!a.zeroCopy) {
                for (int i = warp; i < chunkRows; i += EP_WARPS) {
                    const int64_t r = base + i;
                    if ((reinterpret_cast<const uint2 *>(winExt + r * 8)->x & EP_LINK_FOLLOWER) != 0) continue;
                    CopyLanes(a.expandXOut + r * a.win.rowBytes, winPayload + r * a.win.rowBytes, a.win.rowBytes, lane, 32);
                }
            }
            __syncthreads();
            const int heads = sHeadCount;
            for (int u = warp; u < heads; u += EP_WARPS) {
                const int64_t r = base + sHead[u];
                const uint8_t *src = a.zeroCopy ? a.expandXOut + r * a.win.rowBytes : winPayload + r * a.win.rowBytes;
                // lane j keeps follower j of the chain; the head row is then read once and stored to all of them
                int64_t myFollower = -1;
                int followers = 0;
                uint32_t next = reinterpret_cast<const uint2 *>(winExt + r * 8)->x & EP_LINK_NEXT_MASK;
                for (int hop = 0; next != 0 && hop < KR; ++hop) {
                    const int64_t f = static_cast<int64_t>(next) - 1;
                    if (f >= static_cast<int64_t>(a.maxRecvRows)) break;
                    if (lane == followers) myFollower = f;
                    ++followers;
                    next = reinterpret_cast<const uint2 *>(winExt + f * 8)->x & EP_LINK_NEXT_MASK;
                }
                const int rowVecs16 = static_cast<int>(a.win.rowBytes / 16);
                for (int v0 = 0; v0 < rowVecs16; v0 += 128) {
                    Vec16 q[4];
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const int v = v0 + k4 * 32 + lane;
                        if (v < rowVecs16) q[k4] = ld_vec16_stream(src + static_cast<int64_t>(v) * 16);
                    }
                    for (int j = 0; j < followers; ++j) {
                        uint8_t *dst = a.expandXOut + __shfl_sync(0xffffffffu, myFollower, j) * a.win.rowBytes;
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4) {
                            const int v = v0 + k4 * 32 + lane;
                            if (v < rowVecs16) st_vec16(dst + static_cast<int64_t>(v) * 16, q[k4]);
                        }
                    }
                }
                // a row whose length is not a multiple of 16 bytes keeps its tail
                for (uint32_t bidx = static_cast<uint32_t>(rowVecs16) * 16 + lane; bidx < a.win.rowBytes; bidx += 32) {
                    for (int j = 0; j < followers; ++j) {
                        (a.expandXOut + __shfl_sync(0xffffffffu, myFollower, j) * a.win.rowBytes)[bidx] = src[bidx];
                    }
                }
                for (int j = 0; j < followers; ++j) {
                    const int64_t f = __shfl_sync(0xffffffffu, myFollower, j);
                    if (quantOut && scalarScale) {
                        if (lane == 0) a.dynamicScalesOut[f] = *reinterpret_cast<const float *>(winScales + r * a.win.scaleRowBytes);
                    } else if (quantOut) {
                        CopyLanes(reinterpret_cast<uint8_t *>(a.dynamicScalesOut) + f * a.win.scaleRowBytes,
                                  winScales + r * a.win.scaleRowBytes, a.win.scaleRowBytes, lane, 32);
                    }
                }
            }
            __syncthreads();
        }
        if (blockIdx.x == 0) {
            // cumulative counts in (local expert, source) order: an inclusive scan of E_local * R numbers
            const int n = localCols * R;
            __syncthreads();
            for (int i = tid; i < n; i += blockDim.x) {
                // count of source i % R for local column i / R, out of that source's units (all seen to be complete above)
                const int idx = firstLocal + i / R;
                sm.hist[i] = static_cast<int32_t>(reinterpret_cast<const uint32_t *>(
                    llMine + (static_cast<uint64_t>(i % R) * units + idx / 3) * LL16_UNIT_BYTES)[idx % 3]);
            }
            __syncthreads();
            if (warp == 0) {
                int carry = 0;
                for (int base = 0; base < n; base += 32) {
                    int v = base + lane < n ? sm.hist[base + lane] : 0;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int u = __shfl_up_sync(0xffffffffu, v, o);
                        if (lane >= o) v += u;
                    }
                    v += carry;
                    if (base + lane < n) sm.hist[base + lane] = v;
                    carry = __shfl_sync(0xffffffffu, v, 31);
                }
            }
            __syncthreads();
            for (int i = tid; i < n; i += blockDim.x) a.sendCountsOut[i] = sm.hist[i];
            for (int le = tid; le < localCols; le += blockDim.x) {
                a.expertTokenNumsOut[le] = a.tokenNumsType == TileXREp::TILEXR_EP_TOKEN_NUMS_COUNT
                                               ? static_cast<int64_t>(sm.total[firstLocal + le])
                                               : static_cast<int64_t>(sm.hist[le * R + R - 1]);
            }
            if (tid == 0 && a.recvTotalOut != nullptr) *a.recvTotalOut = n > 0 ? sm.hist[n - 1] : 0;
        }
    }
    PerfStageEnd(perf, TILEXR_PERF_PEER_IPC_TO_OUTPUT);
    PerfStageEnd(perf, TILEXR_PERF_KERNEL_TOTAL);
    KernelEpilogue(w, ok, EP_SCRATCH_TOTALS_WORD + (C + 1) / 2);
}

// ---- combine -----------------------------------------------------------------------------------------------
//
// Work is handed out by two cursors in the rank's control block, so that no warp idles while another still has
// a queue (rows differ a lot: local rows are skipped, followers are folded into their head, heads sum a chain).
//
//   send items    (bucket, chunk of rows, column part): the warp reads the tuples of the chunk's rows, keeps the
//                 rows that must travel and whose token lies in `bucket`, and sends that column part of each.
//                 Buckets are ranges of the SOURCE's token index, walked in increasing order by every rank, so a
//                 token's slots arrive from all ranks at about the same time and in token order;
//   reduce items  (token, column part) in increasing token order: wait for the part's slot flags, sum.
//
// The last `reducerBlocks` blocks take reduce items from the start, the others first send and then join: the
// reduction of the early buckets overlaps the transfer of the later ones, and after the last row has landed
// only the last bucket is left to sum.  Every (row, part) has a flag of its own, raised by the sending warp.

__device__ __forceinline__ uint32_t TakeItem(uint32_t *cursor, int lane)
{
    uint32_t it = 0;
    if (lane == 0) it = atomicAdd(cursor, 1u);
    return __shfl_sync(0xffffffffu, it, 0);
}

// Sends column part `part` of row `r` to slot `slot` of rank `src` and raises the part's flag there.  A head row
// of a group is replaced by the gate-weighted fp32 sum of the group's rows (one rounding).  Called by a whole warp.
__device__ __forceinline__ void CombineSendPart(const EpCombineArgs &a, CommArgs *comm, uint32_t epoch, int64_t r, int64_t rows,
                                                int src, int64_t slot, uint32_t link, uint32_t weightBits, uint32_t part, int lane)
{
    const bool bf16 = a.isBf16 != 0;
    const int KR = a.topK + a.topo.sharedExperts;
    const int rowVecs = a.rowBytes / 16;
    const int vBegin = static_cast<int>(part) * static_cast<int>(a.partVecs);
    const int vEnd = min(rowVecs, vBegin + static_cast<int>(a.partVecs));
    uint8_t *dst = DataHalf(comm, src, epoch) + slot * a.rowBytes;
    if ((link & EP_LINK_NEXT_MASK) == 0) {
        // eight 16-byte vectors in flight per lane: under an all-to-all of eight ranks a store takes several
        // microseconds to be acknowledged, and the warps on an SM must cover that with bytes in flight
        const uint8_t *src = a.expertOut + r * a.rowBytes;
        int v = vBegin + lane;
        for (; v + 7 * 32 < vEnd; v += 8 * 32) {
            Vec16 q[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) q[u] = ld_vec16_stream(src + static_cast<int64_t>(v + u * 32) * 16);
#pragma unroll
            for (int u = 0; u < 8; ++u) st_vec16(dst + static_cast<int64_t>(v + u * 32) * 16, q[u]);
        }
        // the rest of the row (fewer than eight vectors per lane) in rounds of four with the missing ones switched off;
        // one vector at a time it would cost a round trip each
        for (; v < vEnd; v += 4 * 32) {
            Vec16 q[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (v + u * 32 < vEnd) q[u] = ld_vec16_stream(src + static_cast<int64_t>(v + u * 32) * 16);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (v + u * 32 < vEnd) st_vec16(dst + static_cast<int64_t>(v + u * 32) * 16, q[u]);
            }
        }
    } else {
        // The rows of this token on this rank, in k order, times their gate weights: lane i keeps member i of
        // the chain, then every 16-byte column is summed in fp32 and rounded once.
        int64_t memberRow = -1;
        float memberW = 0.f;
        int members = 0;
        int64_t cur = r;
        uint2 e2 = make_uint2(link, weightBits);
        while (members < KR) {
            if (lane == members) {
                memberRow = cur;
                memberW = __uint_as_float(e2.y);
            }
            ++members;
            const uint32_t next = e2.x & EP_LINK_NEXT_MASK;
            if (next == 0 || static_cast<int64_t>(next) - 1 >= rows) break;
            cur = static_cast<int64_t>(next) - 1;
            e2 = *reinterpret_cast<const uint2 *>(a.assistExt + cur * 2);
        }
        for (int v0 = vBegin; v0 < vEnd; v0 += 32) {
            const int v = v0 + lane;
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
            // the columns of four members are fetched together, then added in k order
            for (int i0 = 0; i0 < members; i0 += 4) {
                Vec16 q[4];
                float mw[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int64_t mr = __shfl_sync(0xffffffffu, memberRow, (i0 + i) & 31);
                    mw[i] = __shfl_sync(0xffffffffu, memberW, (i0 + i) & 31);
                    q[i] = Vec16{0u, 0u, 0u, 0u};
                    if (i0 + i < members && v < vEnd) q[i] = ld_vec16_stream(a.expertOut + mr * a.rowBytes + v * 16);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (i0 + i < members) {
                        float f[8];
                        Unpack8(q[i], bf16, f);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] = fmaf(mw[i], f[j], acc[j]);
                    }
                }
            }
            if (v < vEnd) st_vec16(dst + v * 16, Pack8(acc, bf16));
        }
    }
    // every lane's stores of this part are ordered before the flag by the warp barrier and the release
    __syncwarp();
    if (lane == 0) SetFlag(FlagSlot(comm, src, TILEXR_FLAG_SLOT_BASE + slot * a.parts + part), epoch, 1);
}

__device__ void EpCombineBody(const EpCombineArgs &a)
{
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_EP_COMBINE, a.bs, true);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int K = a.topK;
    const int KR = K + a.topo.sharedExperts;     // slots per token: top-k routes and one per shared expert
    const int lane = threadIdx.x & 31;
    const uint32_t epoch = w.epoch;
    const bool bf16 = a.isBf16 != 0;
    const uint32_t P = a.parts;
    const int rowVecs = a.rowBytes / 16;
    const int partVecs = a.partVecs;
    uint32_t *cursors = reinterpret_cast<uint32_t *>(CtrlWord(comm, rank, TILEXR_CTRL_SCRATCH_WORD));
    PerfScope perf = PerfInit(threadIdx.x == 0 ? a.perfTrace : nullptr, static_cast<uint32_t>(rank), blockIdx.x);
    PerfStageBegin(perf, TILEXR_PERF_KERNEL_TOTAL);

    if (ok) {
        const int64_t rows = a.sendCounts[a.sendCountEntries - 1];
        // Rows of this rank's own tokens stay where they are when the reducer knows their row (direct), and the
        // followers of a group are summed into their head's row.
        const bool direct = a.routeRows != nullptr && a.expertIds != nullptr;
        const bool sender = a.noSend == 0 && blockIdx.x + a.reducerBlocks < gridDim.x;
        // What a lane learns about row r: does it travel, where to, which bucket of the source's tokens.
        auto classify = [&](int64_t r, int &src, int64_t &slot, uint2 &ext, uint32_t &bucket) -> bool {
            const Vec16 tuple = ld_vec16(a.assist + r * 4);
            src = static_cast<int>(tuple.x);
            slot = static_cast<int64_t>(tuple.y) * KR + tuple.z;
            bucket = min(tuple.y / a.bucketTokens, a.buckets - 1u);
            bool send = src >= 0 && src < comm->rankSize && tuple.y < static_cast<uint32_t>(a.bs) && tuple.z < static_cast<uint32_t>(KR);
            if (direct && src == rank) send = false;
            if (send && a.dedup != 0) {
                ext = *reinterpret_cast<const uint2 *>(a.assistExt + r * 2);
                if ((ext.x & EP_LINK_FOLLOWER) != 0) send = false;
            }
            return send;
        };
        const uint32_t senders = gridDim.x - a.reducerBlocks;
        const bool sorted = a.buckets > 1 && rows <= static_cast<int64_t>(a.listCap);
        if (sender && sorted) {
            PerfStageBegin(perf, TILEXR_PERF_LOCAL_INPUT_TO_IPC);
            // Rows in a (local expert, source) segment are in token order, so consecutive rows share a bucket:
            // the rows that travel are first sorted by bucket into lists (positions by atomics, order within a
            // bucket does not matter), then one cursor walks the lists bucket after bucket, a row part per item.
            uint32_t *bucketCount = cursors + 2 * EP_SCRATCH_BUCKET_WORD;
            int32_t *lists = reinterpret_cast<int32_t *>(DataHalf(comm, rank, epoch) + a.listOff);
            const int64_t gw = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
            const int64_t nw = static_cast<int64_t>(senders) * (blockDim.x >> 5);
            for (int64_t base = gw * 32; base < rows; base += nw * 32) {
                const int64_t r = base + lane;
                int src = -1;
                int64_t slot = 0;
                uint2 ext = make_uint2(0u, 0u);
                uint32_t bucket = 0;
                const bool send = r < rows && classify(r, src, slot, ext, bucket);
                uint32_t left = __ballot_sync(0xffffffffu, send);
                while (left != 0) {
                    const uint32_t bb = __shfl_sync(0xffffffffu, bucket, __ffs(left) - 1);
                    const uint32_t m = __ballot_sync(0xffffffffu, send && bucket == bb);
                    uint32_t pos = 0;
                    if (lane == 0) pos = atomicAdd(&bucketCount[bb], static_cast<uint32_t>(__popc(m)));
                    pos = __shfl_sync(0xffffffffu, pos, 0);
                    if (send && bucket == bb) lists[static_cast<uint64_t>(bb) * a.listCap + pos + __popc(m & ((1u << lane) - 1u))] = static_cast<int32_t>(r);
                    left &= ~m;
                }
            }
            __syncthreads();
            {
                bool got = true;
                if (threadIdx.x == 0) {
                    __threadfence();
                    got = GridBarrierThread0(w, 1, senders);
                }
                ok = BlockBroadcastOk(got);
            }
            if (ok) {
                uint32_t incl = lane < static_cast<int>(a.buckets) ? __ldcg(&bucketCount[lane]) : 0u;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t u = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += u;
                }
                const uint32_t nItems = __shfl_sync(0xffffffffu, incl, 31) * P;
                for (;;) {
                    const uint32_t it = TakeItem(&cursors[0], lane);
                    if (it >= nItems) break;
                    const uint32_t i = it / P;
                    const uint32_t part = it - i * P;
                    const int b = __popc(__ballot_sync(0xffffffffu, lane < static_cast<int>(a.buckets) && incl <= i));
                    const uint32_t before = b > 0 ? __shfl_sync(0xffffffffu, incl, b - 1) : 0u;
                    const int64_t r = __ldcg(&lists[static_cast<uint64_t>(b) * a.listCap + (i - before)]);
                    const Vec16 tuple = ld_vec16(a.assist + r * 4);
                    uint2 ext = make_uint2(0u, 0u);
                    if (a.dedup != 0) ext = *reinterpret_cast<const uint2 *>(a.assistExt + r * 2);
                    CombineSendPart(a, comm, epoch, r, rows, static_cast<int>(tuple.x), static_cast<int64_t>(tuple.y) * KR + tuple.z, ext.x,
                                    ext.y, part, lane);
                }
            }
            PerfStageEnd(perf, TILEXR_PERF_LOCAL_INPUT_TO_IPC);
        } else if (sender) {
            PerfStageBegin(perf, TILEXR_PERF_LOCAL_INPUT_TO_IPC);
            // Unsorted: items are (chunk of rows, column part) in row order.
            const uint32_t c = a.chunkRows;
            const uint32_t nChunks = static_cast<uint32_t>((rows + c - 1) / c);
            const uint32_t nItems = nChunks * P;
            for (;;) {
                const uint32_t it = TakeItem(&cursors[0], lane);
                if (it >= nItems) break;
                const uint32_t chunk = it / P;
                const uint32_t part = it - chunk * P;
                const int64_t r = static_cast<int64_t>(chunk) * c + lane;
                int src = -1;
                int64_t slot = 0;
                uint2 ext = make_uint2(0u, 0u);
                uint32_t bucket = 0;
                const bool send = lane < static_cast<int>(c) && r < rows && classify(r, src, slot, ext, bucket);
                uint32_t m = __ballot_sync(0xffffffffu, send);
                while (m != 0) {
                    const int j = __ffs(m) - 1;
                    m &= m - 1;
                    const int64_t rj = static_cast<int64_t>(chunk) * c + j;
                    CombineSendPart(a, comm, epoch, rj, rows, __shfl_sync(0xffffffffu, src, j), __shfl_sync(0xffffffffu, slot, j),
                                    __shfl_sync(0xffffffffu, ext.x, j), __shfl_sync(0xffffffffu, ext.y, j), part, lane);
                }
            }
            PerfStageEnd(perf, TILEXR_PERF_LOCAL_INPUT_TO_IPC);
        }
        PerfStageBegin(perf, TILEXR_PERF_PEER_IPC_TO_OUTPUT);
        // ---- reduce this rank's tokens ------------------------------------------------------------------------
        const uint8_t *half = DataHalf(comm, rank, epoch);
        const uint32_t nReduce = static_cast<uint32_t>(a.bs) * P;
        while (w.ok()) {
            const uint32_t it = TakeItem(&cursors[1], lane);
            if (it >= nReduce) break;
            const int64_t t = it / P;
            const uint32_t part = it - static_cast<uint32_t>(t) * P;
            const int vBegin = static_cast<int>(part) * partVecs;
            const int vEnd = min(rowVecs, vBegin + partVecs);
            int e = -1;
            float wk = 0.f;
            unsigned long long myRowPtr = 0;
            // `e` is the COLUMN of the route (shared ranks first, then routed experts), -1 when inactive
            if (lane < K) {
                e = a.expertIds != nullptr ? a.expertIds[t * K + lane] : 0;
                if (e >= a.numExperts) e = -1;
                if (a.maskType == TileXREp::TILEXR_EP_ACTIVE_MASK_TOKEN && a.activeMask[t] == 0) e = -1;
                if (a.maskType == TileXREp::TILEXR_EP_ACTIVE_MASK_EXPERT && a.activeMask[t * K + lane] == 0) e = -1;
                if (e >= 0) e += a.topo.sharedRanks;
                wk = a.expertScales != nullptr ? a.expertScales[t * K + lane] : 1.0f;
            } else if (lane < KR) {
                // the shared experts' outputs are added with weight one
                const bool activeTok = !(a.maskType == TileXREp::TILEXR_EP_ACTIVE_MASK_TOKEN && a.activeMask[t] == 0);
                e = activeTok ? EpSharedCol(a.topo, rank, lane - K) : -1;
                wk = 1.0f;
            }
            const int myDst = e >= 0 ? EpColRank(a.topo, e) : -1;
            if (a.dedup != 0) {
                // routes to one remote rank come back as one weighted sum in the slot of the lowest k
                bool lower = false, higher = false;
                for (int j = 0; j < KR; ++j) {
                    const int dj = __shfl_sync(0xffffffffu, myDst, j);
                    if (dj >= 0 && dj == myDst && myDst != rank) {
                        if (j < lane) lower = true;
                        else if (j > lane) higher = true;
                    }
                }
                if (lower) e = -1;
                else if (higher) wk = 1.0f;
            }
            if (lane < KR && e >= 0) {
                const int64_t slot = t * KR + lane;
                const int64_t localRow = direct && myDst == rank ? a.routeRows[slot] : -1;
                if (localRow >= 0 && localRow < rows) {
                    myRowPtr = reinterpret_cast<unsigned long long>(a.expertOut + localRow * a.rowBytes);
                } else {
                    myRowPtr = reinterpret_cast<unsigned long long>(half + slot * a.rowBytes);
                    WaitFlagGE(w, FlagSlot(comm, rank, TILEXR_FLAG_SLOT_BASE + slot * P + part), 1, myDst, slot);
                }
            }
            const bool good = __all_sync(0xffffffffu, w.ok());
            if (!good) {
                if (w.ok()) w.status = TILEXR_DEV_ABORTED;
                break;
            }
            const uint32_t active = __ballot_sync(0xffffffffu, e >= 0);
            uint8_t *y = a.yOut + t * a.rowBytes;
            // RU 16-byte columns per lane and row: a warp reads RU * 512 contiguous bytes of a row in one go (DRAM
            // pages are used well although up to KR rows are walked together), and accumulates route by route
            // in k order.
            constexpr int RU = 2;
            for (int v0 = vBegin; v0 < vEnd; v0 += 32 * RU) {  // warp-uniform trip count: the loop body shuffles
                float acc[RU][8];
#pragma unroll
                for (int u = 0; u < RU; ++u) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
                }
                for (int k = 0; k < KR; ++k) {
                    if (((active >> k) & 1u) == 0) continue;
                    const uint8_t *src = reinterpret_cast<const uint8_t *>(__shfl_sync(0xffffffffu, myRowPtr, k));
                    const float wgt = __shfl_sync(0xffffffffu, wk, k);
                    Vec16 q[RU];
#pragma unroll
                    for (int u = 0; u < RU; ++u) {
                        const int v = v0 + u * 32 + lane;
                        q[u] = Vec16{0u, 0u, 0u, 0u};
                        if (v < vEnd) q[u] = ld_vec16_stream(src + v * 16);
                    }
#pragma unroll
                    for (int u = 0; u < RU; ++u) {
                        float f[8];
                        Unpack8(q[u], bf16, f);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[u][i] = fmaf(wgt, f[i], acc[u][i]);
                    }
                }
#pragma unroll
                for (int u = 0; u < RU; ++u) {
                    const int v = v0 + u * 32 + lane;
                    if (v >= vEnd) continue;
                    if (a.sharedExpertX != nullptr) {
                        float f[8];
                        Unpack8(ld_vec16(a.sharedExpertX + t * a.rowBytes + v * 16), bf16, f);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[u][j] += f[j];
                    }
                    st_vec16(y + v * 16, Pack8(acc[u], bf16));
                }
            }
        }
        ok = w.ok();
        PerfStageEnd(perf, TILEXR_PERF_PEER_IPC_TO_OUTPUT);
    }
    ok = BlockBroadcastOk(ok);
    PerfStageEnd(perf, TILEXR_PERF_KERNEL_TOTAL);
    KernelEpilogue(w, ok, EP_SCRATCH_TOTALS_WORD);      // the cursors and the bucket counts
}

TILEXR_DEFINE_KERNEL_OCC(TileXREpDispatchKernel, EpDispatchArgs, EpDispatchBody, EP_BLOCK_THREADS, 2)
TILEXR_DEFINE_KERNEL_OCC(TileXREpCombineKernel, EpCombineArgs, EpCombineBody, EP_BLOCK_THREADS, 2)

// ---- stand-alone quantisation and norm kernels ---------------------------------------------------------------

// One warp per row; lane handles 16 elements per iteration, a 128-element block is 8 lanes.
__global__ void __launch_bounds__(256) Fp8Quant1x128Kernel(const uint8_t *x, int64_t rows, int h, int bf16, uint8_t *y, float *scales)
{
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int chunks = h / 16;
    const uint8_t *src = x + row * h * 2;
    for (int c0 = 0; c0 < chunks; c0 += 32) {
        const int c = c0 + lane;
        float f[16];
        if (c < chunks) {
            Unpack8(ld_vec16(src + static_cast<int64_t>(c) * 32), bf16 != 0, f);
            Unpack8(ld_vec16(src + static_cast<int64_t>(c) * 32 + 16), bf16 != 0, f + 8);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) f[j] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        amax = fmaxf(amax, FP8_AMAX_FLOOR);
        const float inv = FP8_E4M3_MAX / amax;
        if (c < chunks) {
            if ((lane & 7) == 0) scales[row * (h / 128) + c / 8] = amax / FP8_E4M3_MAX;
            Vec16 q;
            q.x = Fp8x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
            q.y = Fp8x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
            q.z = Fp8x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
            q.w = Fp8x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
            st_vec16(y + row * h + static_cast<int64_t>(c) * 16, q);
        }
    }
}

__global__ void __launch_bounds__(256) Fp8Dequant1x128Kernel(const uint8_t *y, const float *scales, int64_t rows, int h, int bf16, uint8_t *x)
{
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // one thread per 8 elements
    const int per = h / 8;
    if (idx >= rows * per) return;
    const int64_t row = idx / per;
    const int c = static_cast<int>(idx % per);
    const uint2 raw = *reinterpret_cast<const uint2 *>(y + row * h + static_cast<int64_t>(c) * 8);
    const float s = scales[row * (h / 128) + c / 16];
    float f[8];
    const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * j)) & 0xffffu), __NV_E4M3);
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&h2));
            f[i * 4 + j * 2] = f2.x * s;
            f[i * 4 + j * 2 + 1] = f2.y * s;
        }
    }
    st_vec16(x + (row * h + static_cast<int64_t>(c) * 8) * 2, Pack8(f, bf16 != 0));
}

// MXFP8: 32-element blocks share an E8M0 exponent 2^(floor(log2(amax)) - emax), emax = 8 for
// e4m3 and 15 for e5m2; elements are x / 2^exp rounded to nearest even with saturation.
__global__ void __launch_bounds__(256) Mxfp8QuantKernel(const uint8_t *x, int64_t rows, int h, int bf16, int e5m2, uint8_t *y, uint8_t *scales)
{
    const int blocksPerRow = (h + 31) / 32;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // one thread per 32-element block
    if (idx >= rows * blocksPerRow) return;
    const int64_t row = idx / blocksPerRow;
    const int b = static_cast<int>(idx % blocksPerRow);
    const int n = min(32, h - b * 32);
    float f[32];
    float amax = 0.f;
    for (int j = 0; j < 32; ++j) {
        float v = 0.f;
        if (j < n) {
            const uint16_t raw = *reinterpret_cast<const uint16_t *>(x + (row * h + b * 32 + j) * 2);
            v = bf16 ? __uint_as_float(static_cast<uint32_t>(raw) << 16) : __half2float(*reinterpret_cast<const __half *>(&raw));
        }
        f[j] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    const int emax = e5m2 ? 15 : 8;
    int exp = 0;
    if (amax > 0.f) {
        exp = static_cast<int>((__float_as_uint(amax) >> 23) & 0xff) - 127 - emax;   // floor(log2(amax)) - emax
        if ((__float_as_uint(amax) >> 23) == 0) exp = -126 - emax;                    // subnormal input
    } else {
        exp = -127;
    }
    exp = max(-127, min(127, exp));
    scales[row * blocksPerRow + b] = static_cast<uint8_t>(exp + 127);
    const float inv = exp2f(static_cast<float>(-exp));
    for (int j = 0; j < n; ++j) {
        const float v = f[j] * inv;
        const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3);
        y[row * h + b * 32 + j] = q;
    }
}

__global__ void __launch_bounds__(256) Mxfp8DequantKernel(const uint8_t *y, const uint8_t *scales, int64_t rows, int h, int e5m2, int bf16, uint8_t *x)
{
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * h) return;
    const int64_t row = idx / h;
    const int col = static_cast<int>(idx % h);
    const int blocksPerRow = (h + 31) / 32;
    const float s = exp2f(static_cast<float>(static_cast<int>(scales[row * blocksPerRow + col / 32]) - 127));
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(y[idx], e5m2 ? __NV_E5M2 : __NV_E4M3);
    const float v = __half2float(*reinterpret_cast<const __half *>(&hr)) * s;
    if (bf16) {
        const __nv_bfloat16 o = __float2bfloat16_rn(v);
        *reinterpret_cast<__nv_bfloat16 *>(x + idx * 2) = o;
    } else {
        *reinterpret_cast<__half *>(x + idx * 2) = __float2half_rn(v);
    }
}

// One block per row.  The row stays in registers between the two passes.
__global__ void __launch_bounds__(256) RmsNormKernel(const uint8_t *x, uint8_t *residual, const uint8_t *gamma, float eps, int h, int bf16, uint8_t *y)
{
    __shared__ float partial[8];
    const int64_t row = blockIdx.x;
    const int vecs = h / 8;
    constexpr int MAX_VECS = 8;   // 256 threads x 8 vectors x 8 elements = 16384 columns
    float vals[MAX_VECS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VECS; ++i) {
        const int v = i * 256 + threadIdx.x;
        if (v < vecs) {
            Unpack8(ld_vec16(x + (row * h + static_cast<int64_t>(v) * 8) * 2), bf16 != 0, vals[i]);
            if (residual != nullptr) {
                float r[8];
                Unpack8(ld_vec16(residual + (row * h + static_cast<int64_t>(v) * 8) * 2), bf16 != 0, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
                // the sum, rounded to the storage type, is both the new residual and the norm input
                const Vec16 packed = Pack8(vals[i], bf16 != 0);
                st_vec16(residual + (row * h + static_cast<int64_t>(v) * 8) * 2, packed);
                Unpack8(packed, bf16 != 0, vals[i]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
    }
    ss = WarpSum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += partial[i];
    const float rstd = rsqrtf(tot / static_cast<float>(h) + eps);
#pragma unroll
    for (int i = 0; i < MAX_VECS; ++i) {
        const int v = i * 256 + threadIdx.x;
        if (v < vecs) {
            float g[8];
            Unpack8(ld_vec16(gamma + static_cast<int64_t>(v) * 16), bf16 != 0, g);
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * g[j];
            st_vec16(y + (row * h + static_cast<int64_t>(v) * 8) * 2, Pack8(o, bf16 != 0));
        }
    }
}

int CheckLaunch(const char *what)
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "[TileXR] %s launch failed: %s\n", what, cudaGetErrorString(e));
        return TILEXR_ERROR_RUNTIME;
    }
    NoteLaunch();
    return TILEXR_SUCCESS;
}

} // namespace

const KernelEntry &EpDispatchKernelEntry() { return TileXREpDispatchKernelEntry; }
const KernelEntry &EpCombineKernelEntry() { return TileXREpCombineKernelEntry; }

size_t EpDispatchSmemBytes(int numExperts, int routesPerBlock)
{
    return static_cast<size_t>(routesPerBlock) * 8 + static_cast<size_t>(numExperts) * 16 + EP_WARPS * 64 * sizeof(float);
}

int LaunchRoutingTopK(const RoutingArgs &args, void *stream)
{
    const int warpsPerBlock = 8;
    const unsigned grid = static_cast<unsigned>((args.bs + warpsPerBlock - 1) / warpsPerBlock);
    RoutingTopKKernel<<<grid, warpsPerBlock * 32, 0, static_cast<cudaStream_t>(stream)>>>(args);
    return CheckLaunch("routing top-k");
}

int LaunchFp8Quant1x128(const void *x, int64_t rows, int64_t h, bool bf16, void *y, float *scales, void *stream)
{
    const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
    Fp8Quant1x128Kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t *>(x), rows, static_cast<int>(h),
                                                                              bf16 ? 1 : 0, static_cast<uint8_t *>(y), scales);
    return CheckLaunch("fp8 quant");
}

int LaunchFp8Dequant1x128(const void *y, const float *scales, int64_t rows, int64_t h, bool bf16, void *x, void *stream)
{
    const int64_t n = rows * (h / 8);
    const unsigned grid = static_cast<unsigned>((n + 255) / 256);
    Fp8Dequant1x128Kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t *>(y), scales, rows,
                                                                                static_cast<int>(h), bf16 ? 1 : 0, static_cast<uint8_t *>(x));
    return CheckLaunch("fp8 dequant");
}

int LaunchMxfp8Quant(const void *x, int64_t rows, int64_t h, bool bf16, bool e5m2, void *y, uint8_t *scales, void *stream)
{
    const int64_t n = rows * ((h + 31) / 32);
    const unsigned grid = static_cast<unsigned>((n + 255) / 256);
    Mxfp8QuantKernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t *>(x), rows, static_cast<int>(h),
                                                                           bf16 ? 1 : 0, e5m2 ? 1 : 0, static_cast<uint8_t *>(y), scales);
    return CheckLaunch("mxfp8 quant");
}

int LaunchMxfp8Dequant(const void *y, const uint8_t *scales, int64_t rows, int64_t h, bool e5m2, bool bf16, void *x, void *stream)
{
    const int64_t n = rows * h;
    const unsigned grid = static_cast<unsigned>((n + 255) / 256);
    Mxfp8DequantKernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t *>(y), scales, rows,
                                                                             static_cast<int>(h), e5m2 ? 1 : 0, bf16 ? 1 : 0,
                                                                             static_cast<uint8_t *>(x));
    return CheckLaunch("mxfp8 dequant");
}

int LaunchRmsNorm(const void *x, void *residual, const void *gamma, float eps, int64_t rows, int64_t h, bool bf16, void *y, void *stream)
{
    RmsNormKernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(x), static_cast<uint8_t *>(residual), static_cast<const uint8_t *>(gamma), eps,
        static_cast<int>(h), bf16 ? 1 : 0, static_cast<uint8_t *>(y));
    return CheckLaunch("rmsnorm");
}

} // namespace TileXR
