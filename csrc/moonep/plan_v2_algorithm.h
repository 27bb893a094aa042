// Second-generation MoonEP plan as integer arithmetic on caller-provided tables: one source for the CPU oracle
// (TileXRMoeEpPlanV2Reference) and for the planner kernel.  The public contract is in tilexr_ep_plan.h.
//
// The work is cut so that the kernel can run the inherently sequential part on one thread and the per-route part
// on all of them:
//   PlanValidate      arguments, histogram of the rank's own routes against its row of the table
//   PlanBalance       loads, affinity lists, moves inside servers, moves across servers, remainders, layouts
//   PlanOrdinal*      position of every route among the rank's routes to the same expert
//   PlanRouteDst      one route -> destination row (any thread)
//   PlanMarkDuplicates one token -> ~raw for repeated destination ranks (any thread)
//   PlanFinish        status words
//
// Algorithm (specification: reference src/moonep/planner_v2/common/ep_plan_algorithm_impl.h:186-591):
//   load[home] = routes to home's experts.  Inside each server, ranks are ordered by load (descending; ties by
//   global id, then index); the list is cut where two neighbours no longer fit one capacity together; the i-th
//   overloaded rank left of the cut (nearest the cut first) gives min(surplus, deficit) to the i-th underloaded rank
//   right of it.  Across servers, the least loaded min(#underloaded, #active / 2) ranks receive, lowest first; each
//   walks its affinity list (sources by XOR distance of global ids) over at most three senders and takes from the
//   first one that is still free this round.  A move hands over home's experts in order of remaining share
//   (descending; ties lower id): the receiver needs a free weight slot unless it already holds the expert, and the
//   tokens are drawn from source ranks in the receiver's affinity order, optionally limited per (source, receiver)
//   pair.  Every draw is a segment {expert, src, dst, first ordinal at src, first row at dst, count}; only the
//   rank's own segments are kept.  What nobody moved goes home.
#ifndef TILEXR_MOONEP_PLAN_V2_ALGORITHM_H
#define TILEXR_MOONEP_PLAN_V2_ALGORITHM_H

#include <stdint.h>

#include "tilexr_ep_plan.h"

#if defined(__CUDACC__)
#define TXR_PLAN2_FN __host__ __device__ inline
#else
#define TXR_PLAN2_FN inline
#endif

namespace TileXR {
namespace plan2 {

struct Dims {
    int32_t rank, R, E, L, B, S, K;
    int32_t cap;          // S * K
    int32_t nvS;
    int32_t padding;
    int32_t routeLimit;   // 0 = none
    int32_t segCapacity;
};

struct Segment {
    int32_t expert, src, dst, srcBegin, dstBegin, count;
};

struct Inputs {
    const int32_t *topk;       // [cap]
    const int32_t *tpe;        // [R][E]
    const int32_t *globalIds;  // [R]
};

struct Outputs {
    int32_t *dst;              // [cap]
    int32_t *cuSeqlens;        // [E + B]
    int32_t *expertsToCopy;    // [B]
    int32_t *remoteStats;      // [2]
    int32_t *remoteExperts;    // [R][B] or null
    uint64_t *expertTargets;   // [L][ceil(R/64)] or null (both or neither)
    int32_t *status;           // [8]
};

// Everything lives in one int32 array of TableInts(d) entries.
struct Tables {
    int32_t *load;         // [R]
    int32_t *slotsUsed;    // [R]
    int32_t *listA;        // [R] active
    int32_t *listB;        // [R] senders
    int32_t *listC;        // [R] receivers
    int32_t *listD;        // [R] taken this round
    int32_t *remaining;    // [R][E] routes of (src, expert) nobody has placed yet
    int32_t *alloc;        // [R][E] routes of expert e computed on rank d
    int32_t *srcCursor;    // [R][E]
    int32_t *dstCursor;    // [R][E]
    int32_t *base;         // [R][E] first row of expert e on rank d
    int32_t *slots;        // [R][B]
    int32_t *pairTokens;   // [R][R]
    int32_t *affinity;     // [R][R]
    int32_t *expertList;   // [E] scratch: histogram, then expert orders
    int32_t *ordinal;      // [cap]
    Segment *segments;     // [segCapacity]
};

struct Progress {
    int32_t localSegments, expertMoves, intraRounds, interRounds, maxRemote, localEnd;
    int32_t slotBlock, supplyBlock, pairBlock;
    int32_t fatal;         // TileXRMoonEPPlanStatus
    int32_t balanced;
    int32_t layoutStatus;
};

TXR_PLAN2_FN int32_t Min32(int32_t a, int32_t b) { return a < b ? a : b; }
TXR_PLAN2_FN int64_t At(const Dims &d, int32_t r, int32_t e) { return static_cast<int64_t>(r) * d.E + e; }

TXR_PLAN2_FN uint64_t TableInts(const Dims &d)
{
    const uint64_t R = d.R, E = d.E, B = d.B;
    return 6 * R + 5 * R * E + R * B + 2 * R * R + E + static_cast<uint64_t>(d.cap) +
           static_cast<uint64_t>(d.segCapacity) * (sizeof(Segment) / sizeof(int32_t));
}

TXR_PLAN2_FN void Carve(const Dims &d, int32_t *p, Tables *t)
{
    const int64_t R = d.R, E = d.E, B = d.B;
    t->load = p; p += R;
    t->slotsUsed = p; p += R;
    t->listA = p; p += R;
    t->listB = p; p += R;
    t->listC = p; p += R;
    t->listD = p; p += R;
    t->remaining = p; p += R * E;
    t->alloc = p; p += R * E;
    t->srcCursor = p; p += R * E;
    t->dstCursor = p; p += R * E;
    t->base = p; p += R * E;
    t->slots = p; p += R * B;
    t->pairTokens = p; p += R * R;
    t->affinity = p; p += R * R;
    t->expertList = p; p += E;
    t->ordinal = p; p += d.cap;
    t->segments = reinterpret_cast<Segment *>(p);
}

// How many of its own segments a rank can record.  A rank owns one segment per (expert, draw from its routes) plus
// one per expert for the routes that stay home; the capacity below is generous for balanced and skewed routings
// alike, and a plan that needs more ends with PLAN_ERROR_MOVE_RECORD_OVERFLOW on that rank.  The kernel and the
// oracle use the same number, so an overflow is the same on both.
TXR_PLAN2_FN int32_t DefaultSegmentCapacity(int32_t R, int32_t E)
{
    const int64_t v = static_cast<int64_t>(E) * 4 + static_cast<int64_t>(R) * 64;
    return v > 0x3fffffff ? 0x3fffffff : static_cast<int32_t>(v);
}

// ---- validation ---------------------------------------------------------------------------------------------------
TXR_PLAN2_FN int32_t ValidateConfig(int32_t rank, int64_t R, int64_t S, int64_t K, int64_t E, const TileXRMoonEPPlanConfig &c)
{
    if (R <= 0 || R > 128 || rank < 0 || rank >= R || S <= 0 || K <= 0 || K > 32 || E <= 0 || E > 0x7fffffff || E % R != 0 ||
        S > 0x7fffffff / K) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    const int64_t cap = S * K;
    if (c.rankTokenCapacity != cap || c.prefetchSlots <= 0 || c.prefetchSlots > 0x7fffffff || c.nvS < cap || c.nvS > 0x7fffffff ||
        c.tokenPadding <= 0 || c.tokenRouteLimitPerPair < 0 || c.tokenRouteLimitPerPair > cap ||
        c.cardsPerServer != TILEXR_MOONEP_PLAN_CARDS_PER_SERVER || c.cardsPerCabinet != TILEXR_MOONEP_PLAN_CARDS_PER_CABINET ||
        c.crossCandidateCount != TILEXR_MOONEP_PLAN_CROSS_CANDIDATES || R * c.nvS > 0x7fffffff) {
        return PLAN_ERROR_CONFIG_MISMATCH;
    }
    return PLAN_OK;
}

TXR_PLAN2_FN Dims MakeDims(int32_t rank, int64_t R, int64_t S, int64_t K, int64_t E, const TileXRMoonEPPlanConfig &c)
{
    Dims d;
    d.rank = rank;
    d.R = static_cast<int32_t>(R);
    d.E = static_cast<int32_t>(E);
    d.L = static_cast<int32_t>(E / R);
    d.B = static_cast<int32_t>(c.prefetchSlots);
    d.S = static_cast<int32_t>(S);
    d.K = static_cast<int32_t>(K);
    d.cap = static_cast<int32_t>(S * K);
    d.nvS = static_cast<int32_t>(c.nvS);
    d.padding = static_cast<int32_t>(c.tokenPadding > 0x7fffffff ? 0x7fffffff : c.tokenPadding);
    d.routeLimit = static_cast<int32_t>(c.tokenRouteLimitPerPair);
    d.segCapacity = DefaultSegmentCapacity(d.R, d.E);
    return d;
}

// Global ids distinct and non-negative, expert ids in range, counts non-negative (else CONFIG_MISMATCH); the rank's own
// row equals the histogram of its routes and every row sums to cap (else TPE_MISMATCH).  Everything is looked at and a
// configuration problem wins, so that a parallel check reaches the same verdict.
TXR_PLAN2_FN int32_t PlanValidate(const Dims &d, const Inputs &in, Tables &t)
{
    bool config = false, histogram = false;
    for (int32_t a = 0; a < d.R; ++a) {
        if (in.globalIds[a] < 0) config = true;
        for (int32_t b = 0; b < a; ++b) {
            if (in.globalIds[a] == in.globalIds[b]) config = true;
        }
    }
    for (int32_t e = 0; e < d.E; ++e) t.expertList[e] = 0;
    for (int32_t i = 0; i < d.cap; ++i) {
        const int32_t e = in.topk[i];
        if (e < 0 || e >= d.E) {
            config = true;
        } else {
            ++t.expertList[e];
        }
    }
    for (int32_t src = 0; src < d.R; ++src) {
        int64_t sum = 0;
        for (int32_t e = 0; e < d.E; ++e) {
            const int32_t v = in.tpe[At(d, src, e)];
            if (v < 0) config = true;
            if (src == d.rank && v != t.expertList[e]) histogram = true;
            sum += v;
        }
        if (sum != d.cap) histogram = true;
    }
    return config ? PLAN_ERROR_CONFIG_MISMATCH : histogram ? PLAN_ERROR_TPE_MISMATCH : PLAN_OK;
}

// ---- orders -------------------------------------------------------------------------------------------------------
// true when rank a comes before rank b: by load (direction given), then global id, then index.
TXR_PLAN2_FN bool RankBefore(const Tables &t, const Inputs &in, int32_t a, int32_t b, bool ascending)
{
    const int32_t la = t.load[a], lb = t.load[b];
    if (la != lb) return ascending ? la < lb : la > lb;
    const int32_t ga = in.globalIds[a], gb = in.globalIds[b];
    return ga != gb ? ga < gb : a < b;
}

TXR_PLAN2_FN void SortRanksByLoad(const Tables &t, const Inputs &in, int32_t *list, int32_t n, bool ascending)
{
    for (int32_t i = 1; i < n; ++i) {
        const int32_t v = list[i];
        int32_t j = i;
        while (j > 0 && RankBefore(t, in, v, list[j - 1], ascending)) {
            list[j] = list[j - 1];
            --j;
        }
        list[j] = v;
    }
}

// Sources as seen from `dst`: XOR distance of the global ids, then global id, then index.
TXR_PLAN2_FN bool CloserTo(const Inputs &in, int32_t dst, int32_t a, int32_t b)
{
    const uint32_t gd = static_cast<uint32_t>(in.globalIds[dst]);
    const uint32_t ga = static_cast<uint32_t>(in.globalIds[a]), gb = static_cast<uint32_t>(in.globalIds[b]);
    const uint32_t da = ga ^ gd, db = gb ^ gd;
    if (da != db) return da < db;
    return ga != gb ? ga < gb : a < b;
}

TXR_PLAN2_FN void BuildAffinity(const Dims &d, const Inputs &in, Tables &t)
{
    for (int32_t dst = 0; dst < d.R; ++dst) {
        int32_t *row = t.affinity + static_cast<int64_t>(dst) * d.R;
        for (int32_t i = 0; i < d.R; ++i) {
            int32_t j = i;
            while (j > 0 && CloserTo(in, dst, i, row[j - 1])) {
                row[j] = row[j - 1];
                --j;
            }
            row[j] = i;
        }
    }
}

// ---- moves --------------------------------------------------------------------------------------------------------
TXR_PLAN2_FN bool RecordSegment(const Dims &d, Tables &t, Progress &g, int32_t expert, int32_t src, int32_t dst, int32_t srcBegin,
                                int32_t dstBegin, int32_t count)
{
    if (src != d.rank) return true;
    if (g.localSegments >= d.segCapacity) {
        g.fatal = PLAN_ERROR_MOVE_RECORD_OVERFLOW;
        return false;
    }
    Segment &m = t.segments[g.localSegments++];
    m.expert = expert;
    m.src = src;
    m.dst = dst;
    m.srcBegin = srcBegin;
    m.dstBegin = dstBegin;
    m.count = count;
    return true;
}

TXR_PLAN2_FN bool HoldsExpert(const Dims &d, const Tables &t, int32_t dst, int32_t expert)
{
    const int32_t *row = t.slots + static_cast<int64_t>(dst) * d.B;
    for (int32_t i = 0; i < t.slotsUsed[dst]; ++i) {
        if (row[i] == expert) return true;
    }
    return false;
}

// Draws up to `want` routes of `expert` for `dst` from the sources in dst's affinity order.  Returns what it got.
TXR_PLAN2_FN int32_t DrawTokens(const Dims &d, Tables &t, Progress &g, int32_t expert, int32_t dst, int32_t want)
{
    const int32_t *order = t.affinity + static_cast<int64_t>(dst) * d.R;
    const int64_t dstCell = At(d, dst, expert);
    int32_t got = 0;
    for (int32_t i = 0; i < d.R && got < want; ++i) {
        const int32_t src = order[i];
        const int64_t cell = At(d, src, expert);
        int32_t room = want - got;
        if (d.routeLimit != 0) {
            const int32_t left = d.routeLimit - t.pairTokens[static_cast<int64_t>(src) * d.R + dst];
            room = Min32(room, left < 0 ? 0 : left);
        }
        const int32_t take = Min32(t.remaining[cell], room);
        if (take <= 0) continue;
        if (!RecordSegment(d, t, g, expert, src, dst, t.srcCursor[cell], t.dstCursor[dstCell], take)) return -1;
        t.remaining[cell] -= take;
        t.srcCursor[cell] += take;
        t.dstCursor[dstCell] += take;
        if (d.routeLimit != 0) t.pairTokens[static_cast<int64_t>(src) * d.R + dst] += take;
        got += take;
    }
    return got;
}

// Why a draw fell short: a pair limit stands in the way of remaining supply, or there is no supply left.
TXR_PLAN2_FN void NoteShortfall(const Dims &d, const Tables &t, Progress &g, int32_t expert, int32_t dst)
{
    int64_t supply = 0;
    bool limited = false;
    for (int32_t src = 0; src < d.R; ++src) {
        const int32_t left = t.remaining[At(d, src, expert)];
        supply += left;
        if (d.routeLimit != 0 && left > 0 && t.pairTokens[static_cast<int64_t>(src) * d.R + dst] >= d.routeLimit) limited = true;
    }
    if (limited) {
        g.pairBlock = 1;
    } else if (supply == 0) {
        g.supplyBlock = 1;
    }
}

// Moves up to `requested` routes of home's experts to dst; returns the number moved.
TXR_PLAN2_FN int32_t MoveShare(const Dims &d, Tables &t, Progress &g, int32_t home, int32_t dst, int32_t requested)
{
    if (requested <= 0 || home == dst || g.fatal != PLAN_OK) return 0;
    // home's experts with a share left are visited largest share first, lower id on ties.  Usually the first one or two
    // cover the request, so the next expert is selected when it is needed (one pass over home's L experts) instead of
    // sorting all of them first; the shares of the experts not yet visited do not change in between, so the order is
    // that of the sorted list.  expertList[0, L) marks the visited ones.
    const int32_t first = home * d.L;
    for (int32_t i = 0; i < d.L; ++i) t.expertList[i] = 0;
    int32_t open = requested;
    bool usable = false;
    while (open > 0) {
        int32_t expert = -1, share = 0;
        for (int32_t i = 0; i < d.L; ++i) {
            const int32_t v = t.alloc[At(d, home, first + i)];
            if (v > share && t.expertList[i] == 0) {
                expert = first + i;
                share = v;
            }
        }
        if (expert < 0) break;
        t.expertList[expert - first] = 1;
        const bool held = HoldsExpert(d, t, dst, expert);
        if (!held && t.slotsUsed[dst] >= d.B) {
            g.slotBlock = 1;
            continue;
        }
        usable = true;
        const int32_t want = Min32(share, open);
        const int32_t got = DrawTokens(d, t, g, expert, dst, want);
        if (got < 0) return 0;
        if (got > 0) {
            if (!held) t.slots[static_cast<int64_t>(dst) * d.B + t.slotsUsed[dst]++] = expert;
            t.alloc[At(d, home, expert)] -= got;
            t.alloc[At(d, dst, expert)] += got;
            t.load[home] -= got;
            t.load[dst] += got;
            open -= got;
            ++g.expertMoves;
        }
        if (got < want) NoteShortfall(d, t, g, expert, dst);
    }
    if (open > 0 && !usable) g.pairBlock = 1;
    return requested - open;
}

// ---- balancing inside servers ---------------------------------------------------------------------------------------
TXR_PLAN2_FN void BalanceWithinServers(const Dims &d, const Inputs &in, Tables &t, Progress &g)
{
    int32_t lastServer = -1;
    for (;;) {
        // next server id in ascending order
        int32_t server = 0x7fffffff;
        for (int32_t r = 0; r < d.R; ++r) {
            const int32_t key = in.globalIds[r] / TILEXR_MOONEP_PLAN_CARDS_PER_SERVER;
            if (key > lastServer && key < server) server = key;
        }
        if (server == 0x7fffffff) return;
        lastServer = server;
        for (;;) {
            int32_t n = 0;
            for (int32_t r = 0; r < d.R; ++r) {
                if (in.globalIds[r] / TILEXR_MOONEP_PLAN_CARDS_PER_SERVER == server && t.load[r] != d.cap) t.listA[n++] = r;
            }
            SortRanksByLoad(t, in, t.listA, n, false);
            if (n < 2 || t.load[t.listA[0]] + t.load[t.listA[1]] < d.cap || t.load[t.listA[n - 1]] > d.cap) break;
            int32_t cut = n / 2;
            while (cut > 0 && t.load[t.listA[cut - 1]] + t.load[t.listA[cut]] <= d.cap) --cut;
            if (cut == 0) break;
            int32_t ns = 0, nr = 0;
            for (int32_t i = cut - 1; i >= 0; --i) {
                if (t.load[t.listA[i]] > d.cap) t.listB[ns++] = t.listA[i];
            }
            for (int32_t i = cut; i < n; ++i) {
                if (t.load[t.listA[i]] < d.cap) t.listC[nr++] = t.listA[i];
            }
            int32_t moved = 0;
            for (int32_t i = 0; i < Min32(ns, nr); ++i) {
                const int32_t want = Min32(t.load[t.listB[i]] - d.cap, d.cap - t.load[t.listC[i]]);
                if (want > 0) moved += MoveShare(d, t, g, t.listB[i], t.listC[i], want);
                if (g.fatal != PLAN_OK) return;
            }
            if (moved == 0) {
                g.pairBlock = 1;
                break;
            }
            ++g.intraRounds;
        }
    }
}

// ---- balancing across servers -----------------------------------------------------------------------------------------
TXR_PLAN2_FN void BalanceAcrossServers(const Dims &d, const Inputs &in, Tables &t, Progress &g)
{
    for (;;) {
        int32_t n = 0, under = 0;
        for (int32_t r = 0; r < d.R; ++r) {
            if (t.load[r] == d.cap) continue;
            t.listA[n++] = r;
            if (t.load[r] < d.cap) ++under;
        }
        if (n < 2 || under == 0 || under == n) return;
        SortRanksByLoad(t, in, t.listA, n, false);
        const int32_t nr = Min32(under, n / 2);
        if (nr <= 0) return;
        const int32_t ns = n - nr;
        for (int32_t i = 0; i < ns; ++i) t.listB[i] = t.listA[i];
        for (int32_t i = 0; i < nr; ++i) t.listC[i] = t.listA[ns + i];
        SortRanksByLoad(t, in, t.listC, nr, true);
        for (int32_t r = 0; r < d.R; ++r) t.listD[r] = 0;
        int32_t moved = 0;
        for (int32_t i = 0; i < nr; ++i) {
            const int32_t dst = t.listC[i];
            const int32_t *order = t.affinity + static_cast<int64_t>(dst) * d.R;
            int32_t candidates = 0;
            for (int32_t a = 0; a < d.R && candidates < TILEXR_MOONEP_PLAN_CROSS_CANDIDATES; ++a) {
                const int32_t src = order[a];
                bool sender = false;
                for (int32_t q = 0; q < ns; ++q) sender = sender || t.listB[q] == src;
                if (!sender) continue;
                ++candidates;
                if (t.listD[src]) continue;
                const int32_t want = Min32(t.load[src] - d.cap, d.cap - t.load[dst]);
                if (want <= 0) continue;
                const int32_t got = MoveShare(d, t, g, src, dst, want);
                if (g.fatal != PLAN_OK) return;
                if (got > 0) {
                    moved += got;
                    t.listD[src] = 1;
                    break;
                }
            }
        }
        if (moved == 0) {
            g.pairBlock = 1;
            return;
        }
        ++g.interRounds;
    }
}

// What nobody moved is computed at home.  The routes of one expert: every source's remainder goes to the expert's home
// rank, in source order.  Returns true when this rank is one of the sources; *seg is then its segment, which the caller
// appends to the list (in expert order).  Experts touch disjoint cells, so they can be handled in parallel.
TXR_PLAN2_FN bool RemainderOfExpert(const Dims &d, Tables &t, int32_t e, Segment *seg)
{
    const int32_t home = e / d.L;
    const int64_t homeCell = At(d, home, e);
    int32_t cursor = t.dstCursor[homeCell];
    bool mine = false;
    for (int32_t src = 0; src < d.R; ++src) {
        const int64_t cell = At(d, src, e);
        const int32_t n = t.remaining[cell];
        if (n <= 0) continue;
        if (src == d.rank) {
            seg->expert = e;
            seg->src = src;
            seg->dst = home;
            seg->srcBegin = t.srcCursor[cell];
            seg->dstBegin = cursor;
            seg->count = n;
            mine = true;
        }
        t.remaining[cell] = 0;
        t.srcCursor[cell] += n;
        cursor += n;
    }
    t.dstCursor[homeCell] = cursor;
    return mine;
}

// true when RemainderOfExpert(e) will return a segment of this rank (asked before it runs)
TXR_PLAN2_FN bool RemainderIsMine(const Dims &d, const Tables &t, int32_t e) { return t.remaining[At(d, d.rank, e)] > 0; }

TXR_PLAN2_FN void SendRemaindersHome(const Dims &d, Tables &t, Progress &g)
{
    for (int32_t e = 0; e < d.E; ++e) {
        Segment seg;
        if (!RemainderOfExpert(d, t, e, &seg)) continue;
        if (g.localSegments >= d.segCapacity) {
            g.fatal = PLAN_ERROR_MOVE_RECORD_OVERFLOW;
            return;
        }
        t.segments[g.localSegments++] = seg;
    }
}

// ---- layouts --------------------------------------------------------------------------------------------------------
// Per destination: its foreign experts ordered by share (descending, lower id first) take the weight slots; rows are
// laid out as the experts computed from home weights (groups 0..E-1, foreign ones empty) followed by the slots
// (groups E..E+B-1), every group padded.  Cut into a clearing step, a step per destination that fills the slots and a
// step per destination that lays out the rows, so that the kernel can spread each step over its threads; between the
// steps the per-destination results (t.listA: slots used, t.listB: slots whose expert lives here, t.listC: status) are
// folded by one thread.
#if defined(__CUDA_ARCH__)
#define TXR_PLAN2_OR64(ptr, value) atomicOr(reinterpret_cast<unsigned long long *>(ptr), static_cast<unsigned long long>(value))
#else
#define TXR_PLAN2_OR64(ptr, value) (*(ptr) |= (value))
#endif

TXR_PLAN2_FN void LayoutClear(const Dims &d, const Outputs &out, Tables &t, int32_t first, int32_t stride)
{
    const int32_t groups = d.E + d.B;
    const int32_t words = (d.R + 63) / 64;
    for (int64_t i = first; i < static_cast<int64_t>(d.R) * d.B; i += stride) t.slots[i] = -1;
    for (int32_t i = first; i < d.B; i += stride) out.expertsToCopy[i] = -1;
    if (out.remoteExperts != nullptr) {
        for (int64_t i = first; i < static_cast<int64_t>(d.R) * d.B; i += stride) out.remoteExperts[i] = -1;
        for (int64_t i = first; i < static_cast<int64_t>(d.L) * words; i += stride) out.expertTargets[i] = 0;
    }
    for (int32_t i = first; i < groups; i += stride) out.cuSeqlens[i] = 0;
}

TXR_PLAN2_FN void LayoutSlotsOfDst(const Dims &d, const Outputs &out, Tables &t, int32_t dst)
{
    const int32_t words = (d.R + 63) / 64;
    int32_t *row = t.slots + static_cast<int64_t>(dst) * d.B;
    int32_t n = 0;
    t.listA[dst] = 0;
    t.listB[dst] = 0;
    t.listC[dst] = PLAN_OK;
    for (int32_t e = 0; e < d.E; ++e) {
        const int32_t share = t.alloc[At(d, dst, e)];
        if (share <= 0 || e / d.L == dst) continue;
        if (n >= d.B) {
            t.listC[dst] = PLAN_PARTIAL_PREFETCH_SLOT_EXHAUSTED;
            return;
        }
        int32_t j = n++;
        while (j > 0) {
            const int32_t prevShare = t.alloc[At(d, dst, row[j - 1])];
            if (!(share > prevShare || (share == prevShare && e < row[j - 1]))) break;
            row[j] = row[j - 1];
            --j;
        }
        row[j] = e;
    }
    int32_t mine = 0;
    for (int32_t i = 0; i < d.B; ++i) {
        const int32_t e = row[i];
        if (dst == d.rank) out.expertsToCopy[i] = e;
        if (out.remoteExperts != nullptr) out.remoteExperts[static_cast<int64_t>(dst) * d.B + i] = e;
        if (e >= 0 && e / d.L == d.rank) {
            ++mine;
            if (out.expertTargets != nullptr) {
                TXR_PLAN2_OR64(&out.expertTargets[static_cast<int64_t>(e - d.rank * d.L) * words + dst / 64], 1ull << (dst % 64));
            }
        }
    }
    t.listA[dst] = n;
    t.listB[dst] = mine;
}

// Folds the slot step; returns its status.
TXR_PLAN2_FN int32_t LayoutFoldSlots(const Dims &d, const Outputs &out, const Tables &t, Progress &g)
{
    int32_t status = PLAN_OK, mine = 0;
    g.maxRemote = 0;
    g.localEnd = 0;
    for (int32_t dst = 0; dst < d.R; ++dst) {
        if (t.listC[dst] != PLAN_OK) status = t.listC[dst];
        if (t.listA[dst] > g.maxRemote) g.maxRemote = t.listA[dst];
        mine += t.listB[dst];
    }
    out.remoteStats[0] = t.listA[d.rank];
    out.remoteStats[1] = mine;
    return status;
}

// After the slot step succeeded everywhere, a foreign expert with a share on dst sits in one of dst's slots.
TXR_PLAN2_FN void LayoutRowsOfDst(const Dims &d, const Outputs &out, Tables &t, Progress &g, int32_t dst)
{
    const int32_t groups = d.E + d.B;
    const int32_t *row = t.slots + static_cast<int64_t>(dst) * d.B;
    const int32_t homeBegin = dst * d.L, homeEnd = homeBegin + d.L;
    // count <= nvS < 2^31 and padding <= nvS, so count + padding fits 32 unsigned bits: a 32-bit division (the 64-bit one
    // is a subroutine of a hundred cycles on the GPU)
    const uint32_t pad = static_cast<uint32_t>(d.padding);
    int64_t end = 0;
    t.listC[dst] = PLAN_OK;
    for (int32_t group = 0; group < groups; ++group) {
        int32_t expert = -1;
        if (group < d.E) {
            const bool foreign = group < homeBegin || group >= homeEnd;
            if (!(foreign && t.alloc[At(d, dst, group)] > 0)) expert = group;      // else it is computed in its slot
        } else {
            expert = row[group - d.E];
        }
        int32_t count = 0;
        if (expert >= 0) {
            count = t.alloc[At(d, dst, expert)];
            t.base[At(d, dst, expert)] = static_cast<int32_t>(end);
        }
        const int64_t padded = count <= 0 ? 0 : static_cast<int64_t>((static_cast<uint32_t>(count) + pad - 1u) / pad) * pad;
        if (padded > static_cast<int64_t>(d.nvS) - end) {
            t.listC[dst] = PLAN_ERROR_LAYOUT_EXCEEDS_NVS;
            return;
        }
        end += padded;
        if (dst == d.rank) out.cuSeqlens[group] = static_cast<int32_t>(end);
    }
    if (dst == d.rank) g.localEnd = static_cast<int32_t>(end);
}

TXR_PLAN2_FN int32_t LayoutFoldRows(const Dims &d, const Tables &t)
{
    int32_t status = PLAN_OK;
    for (int32_t dst = 0; dst < d.R; ++dst) {
        if (t.listC[dst] != PLAN_OK) status = t.listC[dst];
    }
    return status;
}

TXR_PLAN2_FN int32_t BuildLayouts(const Dims &d, const Outputs &out, Tables &t, Progress &g)
{
    LayoutClear(d, out, t, 0, 1);
    for (int32_t dst = 0; dst < d.R; ++dst) LayoutSlotsOfDst(d, out, t, dst);
    int32_t status = LayoutFoldSlots(d, out, t, g);
    if (status != PLAN_OK) return status;
    for (int32_t dst = 0; dst < d.R; ++dst) LayoutRowsOfDst(d, out, t, g, dst);
    return LayoutFoldRows(d, t);
}

// Table initialisation, cut so that the kernel can spread it over its threads: every function handles the items
// first, first + stride, ... ; the caller runs A, then (after a barrier when parallel) B, then PlanBalance on one thread.
TXR_PLAN2_FN void PlanInitA(const Dims &d, const Inputs &in, Tables &t, int32_t first, int32_t stride)
{
    for (int64_t i = first; i < static_cast<int64_t>(d.R) * d.E; i += stride) {
        t.remaining[i] = in.tpe[i];
        t.alloc[i] = 0;
        t.srcCursor[i] = 0;
        t.dstCursor[i] = 0;
        t.base[i] = 0;
    }
    for (int64_t i = first; i < static_cast<int64_t>(d.R) * d.B; i += stride) t.slots[i] = -1;
    for (int64_t i = first; i < static_cast<int64_t>(d.R) * d.R; i += stride) t.pairTokens[i] = 0;
    for (int32_t r = first; r < d.R; r += stride) t.slotsUsed[r] = 0;
}

// Every expert starts at home with all of its routes; a rank's load is the sum over its home experts.
TXR_PLAN2_FN void PlanInitB(const Dims &d, const Inputs &in, Tables &t, int32_t first, int32_t stride)
{
    for (int32_t e = first; e < d.E; e += stride) {
        int32_t n = 0;
        for (int32_t src = 0; src < d.R; ++src) n += in.tpe[At(d, src, e)];
        t.alloc[At(d, e / d.L, e)] = n;
    }
}

TXR_PLAN2_FN void PlanInitC(const Dims &d, Tables &t, int32_t first, int32_t stride)
{
    for (int32_t r = first; r < d.R; r += stride) {
        int32_t n = 0;
        for (int32_t e = r * d.L; e < (r + 1) * d.L; ++e) n += t.alloc[At(d, r, e)];
        t.load[r] = n;
    }
}

TXR_PLAN2_FN void PlanInitSerial(const Dims &d, const Inputs &in, Tables &t)
{
    PlanInitA(d, in, t, 0, 1);
    PlanInitB(d, in, t, 0, 1);
    PlanInitC(d, t, 0, 1);
}

// ---- the sequential part ----------------------------------------------------------------------------------------------
// Runs on one thread, after the initialisation above.  Afterwards g.fatal / g.balanced / g.layoutStatus say whether
// destinations can be computed.
TXR_PLAN2_FN void PlanMoves(const Dims &d, const Inputs &in, Tables &t, Progress &g)
{
    g = Progress{};
    BuildAffinity(d, in, t);
    BalanceWithinServers(d, in, t, g);
    if (g.fatal == PLAN_OK) BalanceAcrossServers(d, in, t, g);
}

TXR_PLAN2_FN void PlanNoteBalanced(const Dims &d, const Tables &t, Progress &g)
{
    g.balanced = 1;
    for (int32_t r = 0; r < d.R; ++r) {
        if (t.load[r] != d.cap) g.balanced = 0;
    }
}

// The whole of it on one thread (the CPU form; the kernel runs PlanMoves on one thread and spreads the rest).
TXR_PLAN2_FN void PlanBalance(const Dims &d, const Inputs &in, const Outputs &out, Tables &t, Progress &g)
{
    PlanMoves(d, in, t, g);
    if (g.fatal == PLAN_OK) SendRemaindersHome(d, t, g);
    if (g.fatal != PLAN_OK) return;
    PlanNoteBalanced(d, t, g);
    g.layoutStatus = BuildLayouts(d, out, t, g);
}

// Destinations are computed when the layouts are valid, also for a partially balanced plan.
TXR_PLAN2_FN bool PlanHasDestinations(const Progress &g) { return g.fatal == PLAN_OK && g.layoutStatus == PLAN_OK; }

// ---- per-route part -----------------------------------------------------------------------------------------------------
// Sequential form of the ordinals (the kernel computes the same numbers with one thread per expert).
TXR_PLAN2_FN void PlanOrdinalsSerial(const Dims &d, const Inputs &in, Tables &t)
{
    for (int32_t e = 0; e < d.E; ++e) t.expertList[e] = 0;
    for (int32_t i = 0; i < d.cap; ++i) t.ordinal[i] = t.expertList[in.topk[i]]++;
}

// Ordinals of the routes to one expert, in route order.
TXR_PLAN2_FN void PlanOrdinalsOfExpert(const Dims &d, const Inputs &in, Tables &t, int32_t expert)
{
    int32_t n = 0;
    for (int32_t i = 0; i < d.cap; ++i) {
        if (in.topk[i] == expert) t.ordinal[i] = n++;
    }
}

// Raw destination of the route with this ordinal inside segment m (which covers it), or -1 when the row is out of range.
TXR_PLAN2_FN int32_t RouteRawInSegment(const Dims &d, const Tables &t, const Segment &m, int32_t ordinal)
{
    const int64_t row = static_cast<int64_t>(t.base[At(d, m.dst, m.expert)]) + m.dstBegin + (ordinal - m.srcBegin);
    const int64_t raw = static_cast<int64_t>(m.dst) * d.nvS + row;
    if (row < 0 || row >= d.nvS || raw > 0x7fffffff) return -1;
    return static_cast<int32_t>(raw);
}

// Raw destination of one route, or -1 when no segment covers it (an internal error).
TXR_PLAN2_FN int32_t PlanRouteDst(const Dims &d, const Inputs &in, const Tables &t, const Progress &g, int32_t route)
{
    const int32_t expert = in.topk[route];
    const int32_t ordinal = t.ordinal[route];
    for (int32_t i = 0; i < g.localSegments; ++i) {
        const Segment &m = t.segments[i];
        if (m.expert != expert || ordinal < m.srcBegin || ordinal >= m.srcBegin + m.count) continue;
        return RouteRawInSegment(d, t, m, ordinal);
    }
    return -1;
}

// The same through per-expert lists of the segments (head[expert] = one segment of the expert or -1, next[i] = another
// one or -1): the segments of an expert cover disjoint ordinals, so the order of a list does not matter.
TXR_PLAN2_FN int32_t PlanRouteDstListed(const Dims &d, const Tables &t, const int32_t *head, const int32_t *next, int32_t expert,
                                        int32_t ordinal)
{
    for (int32_t i = head[expert]; i >= 0; i = next[i]) {
        const Segment &m = t.segments[i];
        if (ordinal < m.srcBegin || ordinal >= m.srcBegin + m.count) continue;
        return RouteRawInSegment(d, t, m, ordinal);
    }
    return -1;
}

// A route whose token has an earlier route to the same rank only carries its weight: stored as ~raw.  `dst` holds raw
// values for the whole token when this runs.
TXR_PLAN2_FN void PlanMarkDuplicates(const Dims &d, int32_t *dst, int32_t token)
{
    int32_t *row = dst + static_cast<int64_t>(token) * d.K;
    uint32_t dup = 0;
    for (int32_t k = 1; k < d.K; ++k) {
        for (int32_t p = 0; p < k; ++p) {
            if (row[p] / d.nvS == row[k] / d.nvS) dup |= 1u << k;
        }
    }
    for (int32_t k = 1; k < d.K; ++k) {
        if (dup & (1u << k)) row[k] = ~row[k];
    }
}

// Rows of this rank that no route fills: the padding behind every group, and everything behind the last group.
// zeroFill[g] = {first row, number of rows}: the form the dispatch stage takes, which clears them.
TXR_PLAN2_FN void PlanZeroFill(const Dims &d, const Tables &t, const int32_t *cuSeqlens, int32_t *zeroFill)
{
    const int32_t *row = t.slots + static_cast<int64_t>(d.rank) * d.B;
    const int32_t groups = d.E + d.B;
    int32_t *inSlot = t.expertList;   // scratch, free once the plan is balanced
    for (int32_t e = 0; e < d.E; ++e) inSlot[e] = 0;
    for (int32_t i = 0; i < d.B; ++i) {
        if (row[i] >= 0) inSlot[row[i]] = 1;
    }
    for (int32_t g = 0; g < groups; ++g) {
        int32_t expert = -1;
        if (g < d.E) {
            if (!inSlot[g]) expert = g;
        } else {
            expert = row[g - d.E];
        }
        const int32_t begin = g == 0 ? 0 : cuSeqlens[g - 1];
        const int32_t count = expert >= 0 ? t.alloc[At(d, d.rank, expert)] : 0;
        const int32_t end = g == groups - 1 ? d.nvS : cuSeqlens[g];
        zeroFill[2 * g] = begin + count;
        zeroFill[2 * g + 1] = end - (begin + count);
    }
}

// ---- status ---------------------------------------------------------------------------------------------------------------
// `routesOk` is false when some route found no segment.
TXR_PLAN2_FN int32_t PlanFinish(const Dims &d, const Tables &t, const Progress &g, bool routesOk, int32_t *status)
{
    int32_t result;
    if (g.fatal != PLAN_OK) {
        result = g.fatal;
    } else if (!g.balanced) {
        result = g.slotBlock ? PLAN_PARTIAL_PREFETCH_SLOT_EXHAUSTED : g.supplyBlock ? PLAN_PARTIAL_TOKEN_SUPPLY : PLAN_PARTIAL_NO_FEASIBLE_PAIR;
    } else if (g.layoutStatus != PLAN_OK) {
        result = g.layoutStatus;
    } else {
        result = routesOk ? PLAN_OK : PLAN_ERROR_INTERNAL_INVARIANT;
    }
    int32_t deficit = 0;
    for (int32_t r = 0; r < d.R; ++r) {
        if (t.load[r] < d.cap) deficit += d.cap - t.load[r];
    }
    const bool laidOut = g.fatal == PLAN_OK;
    status[0] = result;
    status[1] = g.intraRounds;
    status[2] = g.interRounds;
    status[3] = deficit;
    status[4] = laidOut ? g.maxRemote : 0;
    status[5] = laidOut ? g.localEnd : 0;
    status[6] = g.expertMoves;
    status[7] = g.localSegments;
    return result;
}

} // namespace plan2
} // namespace TileXR

#endif // TILEXR_MOONEP_PLAN_V2_ALGORITHM_H
