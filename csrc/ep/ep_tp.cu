// Expert parallelism combined with tensor parallelism (tpWorldSize T > 1).
//
// The R ranks form R / T expert groups of T consecutive ranks; the ranks of a group hold the SAME experts, each a
// 1/T slice of their weights, so every rank of a group needs every row routed to the group's experts, and the
// group's T partial outputs of a row have to be summed.  The reference does this in two hops (an EP exchange among
// the ranks of one lane, then each rank appends what its group peers received: src/ep/kernels/
// tilexr_ep_dispatch_kernel.cpp:663-697 and :805-827) and leaves the partial sums to the caller.  Behind an NVSwitch every
// rank reaches every other rank at full speed, so here the source writes its row to all T ranks of the group directly,
// and combine adds the T partial outputs on the way back:
//
//   dispatch   route (token, k) to expert e becomes T routes (token, k * T + l), l = 0..T-1, to the "lane experts"
//              (e, l); lane expert (e, l) lives on rank group(e) * T + l and has the local index of e.  The fused
//              dispatch kernel runs on these K * T routes and E * T experts unchanged: rows arrive sorted by local
//              expert, then source rank, then (token, slot), ready for a grouped GEMM.  tpRecvCountsOut[l] is the
//              number of rows that came from ranks of lane l.
//   combine    y[token] = sum over k of w[k] * (sum over l of partial(k, l)): the fused combine kernel with K * T
//              slots per token and each weight repeated T times.
//
// The two kernels here only rewrite the small per-route arrays; they run on the caller's stream in front of the
// fused kernels (and behind dispatch, for the lane counts).
#include <cuda_runtime_api.h>
#include <stdint.h>

#include "ep_kernels.cuh"

namespace TileXR {

namespace {

__global__ void EpTpExpandKernel(const int32_t *ids, const float *weights, const uint8_t *routeMask, int64_t routes, int T, int experts,
                                 int perGroup, int32_t *idsOut, float *weightsOut, uint8_t *routeMaskOut)
{
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;       // one (route, lane) pair
    if (i >= routes * T) return;
    const int64_t route = i / T;
    const int lane = static_cast<int>(i % T);
    if (idsOut != nullptr) {
        const int e = ids[route];
        idsOut[i] = (e >= 0 && e < experts) ? ((e / perGroup) * T + lane) * perGroup + e % perGroup : -1;
    }
    if (weightsOut != nullptr) weightsOut[i] = weights[route];
    if (routeMaskOut != nullptr) routeMaskOut[i] = routeMask[route];
}

// sendCounts holds the running row count in (local expert, source rank) order.
__global__ void EpTpLaneCountsKernel(const int32_t *sendCounts, int entries, int R, int T, int32_t *tpRecvCounts)
{
    __shared__ int sLane[TILEXR_MAX_RANK_SIZE];
    for (int l = threadIdx.x; l < T; l += blockDim.x) sLane[l] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
        const int rows = sendCounts[i] - (i > 0 ? sendCounts[i - 1] : 0);
        if (rows > 0) atomicAdd(&sLane[(i % R) % T], rows);
    }
    __syncthreads();
    for (int l = threadIdx.x; l < T; l += blockDim.x) tpRecvCounts[l] = sLane[l];
}

} // namespace

int EpTpExpand(const int32_t *ids, const float *weights, const uint8_t *routeMask, int64_t routes, int T, int experts, int perGroup,
               int32_t *idsOut, float *weightsOut, uint8_t *routeMaskOut, cudaStream_t stream)
{
    const int64_t n = routes * T;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
    EpTpExpandKernel<<<blocks, 256, 0, stream>>>(ids, weights, routeMask, routes, T, experts, perGroup, idsOut, weightsOut, routeMaskOut);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int EpTpLaneCounts(const int32_t *sendCounts, int entries, int R, int T, int32_t *tpRecvCounts, cudaStream_t stream)
{
    EpTpLaneCountsKernel<<<1, 256, 0, stream>>>(sendCounts, entries, R, T, tpRecvCounts);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

} // namespace TileXR
