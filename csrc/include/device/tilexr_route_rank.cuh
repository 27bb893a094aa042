// Stable rank of each route among a block's routes to the same expert, and the per-expert count, in time linear in
// the number of routes.
#ifndef TILEXR_ROUTE_RANK_CUH
#define TILEXR_ROUTE_RANK_CUH

#include <stdint.h>

namespace tilexr {

// One warp (all 32 lanes call) walks `experts[0, n)` 32 routes at a time.  Lanes that hold the same expert find one
// another with match.any; each takes `hist[e]` plus the number of such lanes below it as its rank, then the lowest of
// them adds the group to `hist[e]`.  `hist` must be zeroed (or hold the counts of earlier routes) and, like
// `experts` and `rank`, live in shared memory that the other warps leave alone until the block's next barrier.
// Routes with a negative expert get rank 0 and are not counted.
__device__ __forceinline__ void RankRoutesByWarp(const int32_t *experts, int32_t *rank, int32_t *hist, int n, int lane)
{
    const unsigned below = (1u << lane) - 1u;
    for (int base = 0; base < n; base += 32) {
        const int i = base + lane;
        const int e = i < n ? experts[i] : -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (i < n) rank[i] = e >= 0 ? hist[e] + __popc(same & below) : 0;
        __syncwarp();
        if (e >= 0 && (same & below) == 0) hist[e] += __popc(same);
        __syncwarp();
    }
}

// The same ranks for `experts` in global memory: the expert ids of four steps are fetched before the first of them is
// ranked, so that the four loads are in flight together (one step's load would otherwise sit in front of every step).
__device__ __forceinline__ void RankRoutesByWarpDeep(const int32_t *experts, int32_t *rank, int32_t *hist, int n, int lane)
{
    const unsigned below = (1u << lane) - 1u;
    for (int base = 0; base < n; base += 128) {
        int e4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + u * 32 + lane;
            e4[u] = i < n ? experts[i] : -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + u * 32 + lane;
            if (base + u * 32 >= n) break;      // warp-uniform
            const int e = e4[u];
            const unsigned same = __match_any_sync(0xffffffffu, e);
            if (i < n) rank[i] = e >= 0 ? hist[e] + __popc(same & below) : 0;
            __syncwarp();
            if (e >= 0 && (same & below) == 0) hist[e] += __popc(same);
            __syncwarp();
        }
    }
}

} // namespace tilexr

#endif
