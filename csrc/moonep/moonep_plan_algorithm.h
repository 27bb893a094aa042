// The MoonEP balance plan as plain integer arithmetic on caller-provided tables.  One source
// for the CPU reference and for the planner kernel (the reference keeps its planner algorithm
// in a host+device header for the same reason: src/moonep/planner_v2/common/ep_plan_algorithm.h).
//
// Input is the histogram tpe[src][expert] of every rank.  The plan, in the order computed
// (specification: reference tools/moonep/planner_reference.py:104-310):
//   1. prefix of every expert's count over source ranks, and the expert's global count;
//   2. balance[home] = rows routed to home's experts - N; repeatedly the rank with the largest
//      surplus (first on ties) hands the rank with the largest deficit exactly what it lacks;
//   3. every home fills its quotas: the destination with the largest remaining quota takes from
//      the home's expert with the most remaining rows;
//   4. per destination: remote experts with rows there, sorted by (rows, id) descending; the
//      first B get prefetch slots.  Groups 0..E-1 (unselected experts) then E..E+B-1 (slots)
//      are laid out back to back, each padded to `padding` rows; cuSeqlens = padded ends;
//      the gap of each group (and the tail up to NvS for the last) is a zero-fill range;
//   5. prefix of every expert's allocation over destinations;
//   6. a route that is the g-th occurrence of its expert in global source order goes to the
//      first destination whose allocation prefix exceeds g.
#ifndef TILEXR_MOONEP_PLAN_ALGORITHM_H
#define TILEXR_MOONEP_PLAN_ALGORITHM_H

#include <stdint.h>

#if defined(__CUDACC__)
#define TXR_PLAN_FN __host__ __device__ inline
#else
#define TXR_PLAN_FN inline
#endif

namespace TileXR {

struct PlanDims {
    int32_t R;        // ranks
    int32_t E;        // experts
    int32_t L;        // experts per rank
    int32_t B;        // prefetch slots per rank
    int32_t N;        // routes per rank = S*K
    int32_t NvS;      // row capacity per rank
    int32_t padding;  // token padding
};

// All tables are int32 and live wherever the caller puts them (host vector, device window).
struct PlanTables {
    const int32_t *tpe;       // [R][E] input
    int32_t *tpePrefix;       // [R][E] inclusive prefix over sources
    int32_t *global;          // [E]
    int32_t *balance;         // [R]
    int32_t *moves;           // [R][R] moves[surplus][deficit]
    int32_t *alloc;           // [E][R]
    int32_t *allocPrefix;     // [E][R]
    int32_t *remaining;       // [R][L]
    int32_t *expertOffsets;   // [R][E] first row of expert e at destination d
    int32_t *cu;              // [R][E+B]
    int32_t *zeroFill;        // [R][E+B][2]
    int32_t *expertsToCopy;   // [R][B]
    int32_t *remoteStats;     // [R][2]
    int32_t *remoteList;      // [R][E] scratch
    int32_t *selected;        // [R][E] scratch
};

TXR_PLAN_FN uint64_t PlanTableInts(const PlanDims &d)
{
    const uint64_t R = d.R, E = d.E, L = d.L, B = d.B;
    return R * E /*tpePrefix*/ + E + R + R * R + E * R * 2 + R * L + R * E + R * (E + B) + R * (E + B) * 2 + R * B + R * 2 +
           R * E * 2;
}

// Carves the tables (everything except `tpe`) out of one int32 array of PlanTableInts entries.
TXR_PLAN_FN void PlanCarve(const PlanDims &d, int32_t *base, PlanTables *t)
{
    const int64_t R = d.R, E = d.E, L = d.L, B = d.B;
    int32_t *p = base;
    t->tpePrefix = p; p += R * E;
    t->global = p; p += E;
    t->balance = p; p += R;
    t->moves = p; p += R * R;
    t->alloc = p; p += E * R;
    t->allocPrefix = p; p += E * R;
    t->remaining = p; p += R * L;
    t->expertOffsets = p; p += R * E;
    t->cu = p; p += R * (E + B);
    t->zeroFill = p; p += R * (E + B) * 2;
    t->expertsToCopy = p; p += R * B;
    t->remoteStats = p; p += R * 2;
    t->remoteList = p; p += R * E;
    t->selected = p; p += R * E;
}

TXR_PLAN_FN int32_t PlanCapacity(int64_t n, int64_t padding, int64_t expertsPerRank)
{
    return static_cast<int32_t>(n + (padding - 1) * 2 * expertsPerRank);
}

// Steps 1-3, serial.
TXR_PLAN_FN int PlanBalance(const PlanDims &d, PlanTables &t)
{
    const int R = d.R, E = d.E, L = d.L;
    for (int e = 0; e < E; ++e) {
        int32_t c = 0;
        for (int s = 0; s < R; ++s) {
            c += t.tpe[s * E + e];
            t.tpePrefix[s * E + e] = c;
        }
        t.global[e] = c;
    }
    for (int h = 0; h < R; ++h) {
        int32_t sum = 0;
        for (int l = 0; l < L; ++l) sum += t.global[h * L + l];
        t.balance[h] = sum - d.N;
        for (int x = 0; x < R; ++x) t.moves[h * R + x] = 0;
    }
    for (int guard = 0; guard <= R; ++guard) {
        int surplus = 0, deficit = 0;
        for (int i = 1; i < R; ++i) {
            if (t.balance[i] > t.balance[surplus]) surplus = i;   // first maximum
            if (t.balance[i] < t.balance[deficit]) deficit = i;   // first minimum
        }
        if (t.balance[surplus] <= 0 || t.balance[deficit] >= 0) break;
        const int32_t count = -t.balance[deficit];
        t.moves[surplus * R + deficit] = count;
        t.balance[surplus] -= count;
        t.balance[deficit] = 0;
    }
    for (int e = 0; e < E; ++e) {
        for (int x = 0; x < R; ++x) t.alloc[e * R + x] = 0;
        t.alloc[e * R + e / L] = t.global[e];
    }
    for (int h = 0; h < R; ++h) {
        int32_t *remaining = t.remaining + h * L;
        int32_t *quotas = t.moves + h * R;     // consumed in place; moves are not needed afterwards
        for (int l = 0; l < L; ++l) remaining[l] = t.global[h * L + l];
        for (;;) {
            int dst = 0;
            for (int i = 1; i < R; ++i) {
                if (quotas[i] > quotas[dst]) dst = i;
            }
            if (quotas[dst] <= 0) break;
            int le = 0;
            for (int l = 1; l < L; ++l) {
                if (remaining[l] > remaining[le]) le = l;
            }
            if (remaining[le] <= 0) return -1;   // cannot happen for a consistent histogram
            const int32_t count = remaining[le] < quotas[dst] ? remaining[le] : quotas[dst];
            const int e = h * L + le;
            t.alloc[e * R + dst] += count;
            t.alloc[e * R + h] -= count;
            remaining[le] -= count;
            quotas[dst] -= count;
        }
    }
    for (int x = 0; x < R; ++x) {
        t.remoteStats[x * 2] = 0;
        t.remoteStats[x * 2 + 1] = 0;
    }
    return 0;
}

// Step 4 for one destination; independent across destinations except remoteStats[.][1],
// which PlanFinish derives afterwards.  Returns non-zero when the padded layout exceeds NvS.
TXR_PLAN_FN int PlanLayoutForDestination(const PlanDims &d, PlanTables &t, int dst)
{
    const int R = d.R, E = d.E, L = d.L, B = d.B;
    int32_t *remote = t.remoteList + dst * E;
    int32_t *selected = t.selected + dst * E;
    int32_t *slots = t.expertsToCopy + dst * B;
    int n = 0;
    for (int e = 0; e < E; ++e) {
        selected[e] = 0;
        t.expertOffsets[dst * E + e] = 0;
        const bool local = e >= dst * L && e < (dst + 1) * L;
        if (!local && t.alloc[e * R + dst] > 0) {
            // insertion sort, descending by (rows, id)
            const int32_t rows = t.alloc[e * R + dst];
            int pos = n;
            while (pos > 0) {
                const int32_t other = remote[pos - 1];
                const int32_t otherRows = t.alloc[other * R + dst];
                if (otherRows > rows || (otherRows == rows && other > e)) break;
                remote[pos] = other;
                --pos;
            }
            remote[pos] = e;
            ++n;
        }
    }
    t.remoteStats[dst * 2] = n;
    for (int b = 0; b < B; ++b) {
        slots[b] = b < n ? remote[b] : -1;
        if (b < n) selected[remote[b]] = 1;
    }
    int32_t end = 0;
    for (int g = 0; g < E + B; ++g) {
        int32_t count = 0;
        int expert = -1;
        if (g < E) {
            if (!selected[g]) {
                expert = g;
                count = t.alloc[g * R + dst];
            }
        } else {
            expert = slots[g - E];
            if (expert >= 0) count = t.alloc[expert * R + dst];
        }
        if (count > 0) t.expertOffsets[dst * E + expert] = end;
        const int32_t padded = count > 0 ? (count + d.padding - 1) / d.padding * d.padding : 0;
        const int32_t realEnd = end + count;
        const int32_t paddedEnd = end + padded;
        const int32_t zeroEnd = (g + 1 == E + B) ? d.NvS : paddedEnd;
        t.zeroFill[(dst * (E + B) + g) * 2] = zeroEnd > realEnd ? realEnd : 0;
        t.zeroFill[(dst * (E + B) + g) * 2 + 1] = zeroEnd > realEnd ? zeroEnd - realEnd : 0;
        end = paddedEnd;
        t.cu[dst * (E + B) + g] = paddedEnd;
    }
    return end > d.NvS ? 1 : 0;
}

// Step 5 and the "times my experts are copied" statistic.
TXR_PLAN_FN void PlanFinish(const PlanDims &d, PlanTables &t)
{
    const int R = d.R, E = d.E, L = d.L, B = d.B;
    for (int e = 0; e < E; ++e) {
        int32_t c = 0;
        for (int x = 0; x < R; ++x) {
            c += t.alloc[e * R + x];
            t.allocPrefix[e * R + x] = c;
        }
    }
    for (int x = 0; x < R; ++x) {
        for (int b = 0; b < B; ++b) {
            const int32_t e = t.expertsToCopy[x * B + b];
            if (e >= 0) t.remoteStats[(e / L) * 2 + 1] += 1;
        }
    }
}

// Step 6: destination row of the route that is occurrence `occurrence` (among this rank's
// routes, in token-major order) of `expert`.  Returns -1 when the tables are inconsistent.
TXR_PLAN_FN int32_t PlanRouteDst(const PlanDims &d, const PlanTables &t, int rank, int expert, int32_t occurrence)
{
    const int R = d.R, E = d.E;
    const int32_t g = (rank == 0 ? 0 : t.tpePrefix[(rank - 1) * E + expert]) + occurrence;
    int dst = 0;
    while (dst < R && t.allocPrefix[expert * R + dst] <= g) ++dst;
    if (dst >= R) return -1;
    const int32_t previous = dst == 0 ? 0 : t.allocPrefix[expert * R + dst - 1];
    return dst * d.NvS + t.expertOffsets[dst * E + expert] + g - previous;
}

} // namespace TileXR

#endif // TILEXR_MOONEP_PLAN_ALGORITHM_H
