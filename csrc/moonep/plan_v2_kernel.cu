// Planner kernel of the second-generation MoonEP plan (contract: tilexr_ep_plan.h, algorithm: plan_v2_algorithm.h).
//
// One block per rank.  The ranks do not exchange plan data: each runs the same deterministic algorithm on the same
// histogram table.  What crosses NVLink is a "mailbox" per (receiver, sender) in the receiver's window:
//   1. header hash (dimensions, configuration, global rank ids) and the sender's own histogram row, checked by the
//      receiver against its caller's table: ranks that were called with different arguments or tables find out here
//      instead of computing plans that do not fit together;
//   2. the sender's final status; every rank returns the largest code, so all ranks agree on whether the plan holds.
// The balancing part is sequential and runs on thread 0; ordinals, destinations and duplicate marks use the block.
// All waits are bounded (communicator's wait budget); a give-up is reported through the device status.
//
// Reference: src/moonep/planner_v2/kernels/tilexr_moonep_planner_kernel.cpp:232-366 (mailbox phases), 542-695.
#include "device/tilexr_rma.cuh"
#include "device/tilexr_route_rank.cuh"
#include "device/tilexr_sync.cuh"
#include "plan_v2_kernel.h"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

struct Mail {
    uint64_t hash;
    int32_t status;
    int32_t pad;
};

__device__ __forceinline__ uint8_t *MailBox(const PlanV2Args &a, int owner, int src, uint32_t epoch)
{
    return DataHalf(a.comm, owner, epoch) + static_cast<uint64_t>(src) * a.mailStride;
}

__device__ __forceinline__ uint64_t *MailFlag(const PlanV2Args &a, int owner, int src)
{
    return FlagSlot(a.comm, owner, TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(src) * TILEXR_FLAGS_PER_PAIR);
}

// Thread t raises the flag of this rank in rank t's window and waits for rank t's flag here.
__device__ __forceinline__ bool MeetRanks(Waiter &w, const PlanV2Args &a, uint32_t value)
{
    const int R = a.dims.R, rank = a.dims.rank;
    __syncthreads();
    bool ok = true;
    const int t = threadIdx.x;
    if (t < R && t != rank) {
        fence_acq_rel_sys();
        SetFlag(MailFlag(a, t, rank), w.epoch, value);
        ok = WaitFlagGE(w, MailFlag(a, rank, t), value, t, value);
    }
    return BlockBroadcastOk(ok);
}

__device__ void PlanV2Body(const PlanV2Args &a)
{
    __shared__ plan2::Progress g;
    __shared__ int sValidate;
    __shared__ int sBadRoute;
    __shared__ int sRemainders;
    __shared__ int sFinal;
    __shared__ uint64_t sHash;

    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_PLANNING, a.dims.cap, true);
    uint64_t phaseStart = now_ns();
    auto phaseDone = [&](int index) {      // thread 0 leaves the phase's duration in the DFX block (read with TileXRGetCommArgsHost)
        if (threadIdx.x == 0) {
            const uint64_t t1 = now_ns();
            a.comm->dfx[TILEXR_DFX_PLAN_PHASE_NS + index] = static_cast<int64_t>(t1 - phaseStart);
            phaseStart = t1;
        }
    };
    const plan2::Dims d = a.dims;
    const int tid = threadIdx.x, nt = blockDim.x;
    const plan2::Inputs in{a.topk, a.tpe, a.globalIds};
    plan2::Tables t;
    plan2::Carve(d, a.tables, &t);
    if (tid == 0) {
        sValidate = PLAN_OK;
        sBadRoute = 0;
        sFinal = PLAN_OK;
        // the global rank ids are device data: they join the host's hash of dimensions and configuration here
        uint64_t h = a.headerHash;
        for (int r = 0; r < d.R; ++r) {
            h ^= static_cast<uint64_t>(static_cast<uint32_t>(a.globalIds[r])) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
            h *= 0xff51afd7ed558ccdull;
        }
        sHash = h;
    }
    __syncthreads();

    // 1. mail: header and own histogram row to everybody (own window included: one code path for the check)
    if (ok) {
        for (int p = 0; p < d.R; ++p) {
            uint8_t *box = MailBox(a, p, d.rank, w.epoch);
            if (tid == 0) {
                Mail *m = reinterpret_cast<Mail *>(box);
                m->hash = sHash;
                m->status = -1;
            }
            int32_t *row = reinterpret_cast<int32_t *>(box + sizeof(Mail));
            for (int e = tid; e < d.E; e += nt) row[e] = a.tpe[plan2::At(d, d.rank, e)];
        }
        ok = MeetRanks(w, a, 1);
    }
    phaseDone(0);
    // 2. check what arrived against the caller's table
    int mismatch = 0;
    if (ok) {
        for (int i = tid; i < d.R * d.E; i += nt) {
            const int src = i / d.E, e = i - src * d.E;
            const int32_t *row = reinterpret_cast<const int32_t *>(MailBox(a, d.rank, src, w.epoch) + sizeof(Mail));
            if (row[e] != a.tpe[i]) mismatch |= 1;
        }
        if (tid < d.R && reinterpret_cast<const Mail *>(MailBox(a, d.rank, tid, w.epoch))->hash != sHash) mismatch |= 2;
    }
    mismatch = __syncthreads_or(mismatch);

    // 3. the caller's own inputs (the rules of plan2::PlanValidate, checked by the whole block), then the plan
    int bad = 0;   // bit 0: histogram problem, bit 1: configuration problem
    if (ok) {
        for (int e = tid; e < d.E; e += nt) t.expertList[e] = 0;
        for (int r = tid; r < d.R; r += nt) t.listA[r] = 0;
        if (tid < d.R) {
            if (a.globalIds[tid] < 0) bad |= 2;
            for (int b = 0; b < tid; ++b) {
                if (a.globalIds[b] == a.globalIds[tid]) bad |= 2;
            }
        }
        __syncthreads();
        for (int i = tid; i < d.cap; i += nt) {
            const int32_t e = a.topk[i];
            if (e < 0 || e >= d.E) {
                bad |= 2;
            } else {
                atomicAdd(&t.expertList[e], 1);
            }
        }
        __syncthreads();
        for (int i = tid; i < d.R * d.E; i += nt) {
            const int src = i / d.E, e = i - src * d.E;
            const int32_t v = a.tpe[i];
            if (v < 0) bad |= 2;
            if (src == d.rank && v != t.expertList[e]) bad |= 1;
            atomicAdd(&t.listA[src], v);      // a negative count is a configuration problem already
        }
        __syncthreads();
        if (tid < d.R && t.listA[tid] != d.cap) bad |= 1;
    }
    bad = __syncthreads_or(bad);
    if (ok && mismatch == 0 && bad == 0) {      // block-uniform
        plan2::PlanInitA(d, in, t, tid, nt);
        __syncthreads();
        plan2::PlanInitB(d, in, t, tid, nt);
        __syncthreads();
        plan2::PlanInitC(d, t, tid, nt);
        __syncthreads();
    }
    // The balancing is one thread walking small tables with dependent accesses: from global memory every step costs an L2
    // round trip.  When the tables fit (they do for the usual 8 ranks x 256 experts: about 90 KB), the block copies them,
    // the histogram table and the segment list into shared memory, thread 0 balances there, and the block copies the
    // result back for the per-route phase.
    extern __shared__ __align__(16) int32_t planShared[];
    const int64_t prefixWords = 6ll * d.R + 5ll * d.R * d.E + static_cast<int64_t>(d.R) * d.B + 2ll * d.R * d.R + d.E;   // load .. expertList
    const int64_t tpeWords = static_cast<int64_t>(d.R) * d.E;
    const int64_t segWords = static_cast<int64_t>(d.segCapacity) * (sizeof(plan2::Segment) / 4);
    const bool staged = a.stagedWords != 0 && prefixWords + tpeWords + segWords <= static_cast<int64_t>(a.stagedWords);
    const bool balance = ok && mismatch == 0 && bad == 0;      // block-uniform
    if (balance && staged) {
        for (int64_t i = tid; i < prefixWords; i += nt) planShared[i] = a.tables[i];
        for (int64_t i = tid; i < tpeWords; i += nt) planShared[prefixWords + i] = a.tpe[i];
    }
    __syncthreads();
    phaseDone(1);
    // the tables the balancing works on: the shared-memory copy when there is one
    plan2::Tables tb = t;
    plan2::Inputs inb = in;
    if (staged) {
        plan2::Carve(d, planShared, &tb);
        tb.ordinal = t.ordinal;                                             // not touched by the balancing
        tb.segments = reinterpret_cast<plan2::Segment *>(planShared + prefixWords + tpeWords);
        inb.tpe = planShared + prefixWords;
    }
    if (tid == 0) {
        int32_t v = (mismatch & 2) ? PLAN_ERROR_CONFIG_MISMATCH : (mismatch & 1) ? PLAN_ERROR_TPE_MISMATCH : PLAN_OK;
        if (ok && v == PLAN_OK) v = (bad & 2) ? PLAN_ERROR_CONFIG_MISMATCH : (bad & 1) ? PLAN_ERROR_TPE_MISMATCH : PLAN_OK;
        sValidate = v;
        g = plan2::Progress{};
        if (ok && v == PLAN_OK) plan2::PlanMoves(d, inb, tb, g);           // the moves between ranks: sequential by nature
    }
    __syncthreads();
    // What follows the moves has no order between experts (the remainders) or between destinations (the layouts), so the
    // block spreads it: plan2::PlanBalance is the same steps on one thread.
    if (balance && g.fatal == PLAN_OK) {                                   // block-uniform: g is shared
        for (int e = tid; e < d.E; e += nt) tb.expertList[e] = plan2::RemainderIsMine(d, tb, e) ? 1 : 0;
        __syncthreads();
        const int32_t firstSegment = g.localSegments;
        for (int e = tid; e < d.E; e += nt) {
            int32_t before = 0;                                            // this rank's remainder segments are listed in expert order
            for (int f = 0; f < e; ++f) before += tb.expertList[f];
            plan2::Segment seg;
            if (plan2::RemainderOfExpert(d, tb, e, &seg) && firstSegment + before < d.segCapacity) tb.segments[firstSegment + before] = seg;
            if (e == d.E - 1) sRemainders = before + tb.expertList[e];
        }
        __syncthreads();
        if (tid == 0) {
            if (firstSegment + sRemainders > d.segCapacity) {
                g.fatal = PLAN_ERROR_MOVE_RECORD_OVERFLOW;
                g.localSegments = d.segCapacity;
            } else {
                g.localSegments = firstSegment + sRemainders;
                plan2::PlanNoteBalanced(d, tb, g);
            }
        }
        __syncthreads();
        if (g.fatal == PLAN_OK) {
            plan2::LayoutClear(d, a.out, tb, tid, nt);
            __syncthreads();
            for (int dst = tid; dst < d.R; dst += nt) plan2::LayoutSlotsOfDst(d, a.out, tb, dst);
            __syncthreads();
            if (tid == 0) g.layoutStatus = plan2::LayoutFoldSlots(d, a.out, tb, g);
            __syncthreads();
            if (g.layoutStatus == PLAN_OK) {
                for (int dst = tid; dst < d.R; dst += nt) plan2::LayoutRowsOfDst(d, a.out, tb, g, dst);
                __syncthreads();
                if (tid == 0) g.layoutStatus = plan2::LayoutFoldRows(d, tb);
            }
        }
    }
    __syncthreads();
    if (balance && staged) {
        for (int64_t i = tid; i < prefixWords; i += nt) a.tables[i] = planShared[i];
        const int32_t *segs = planShared + prefixWords + tpeWords;
        int32_t *segsOut = reinterpret_cast<int32_t *>(t.segments);
        for (int64_t i = tid; i < segWords; i += nt) segsOut[i] = segs[i];
        __syncthreads();
    }
    phaseDone(2);
    const bool planned = ok && sValidate == PLAN_OK;
    if (planned && plan2::PlanHasDestinations(g)) {
        // Ordinal of a route among this rank's routes to the same expert, in route order, then its destination.  The
        // routes are cut into one contiguous piece per warp; every warp ranks its piece against a histogram of its own
        // (32 routes a step), the histograms are turned into per-piece offsets, and the pass that computes the
        // destinations adds the offset.  A route finds its segment through per-expert lists.  The tables of the balancing
        // that are no longer needed hold all of it: srcCursor and dstCursor (adjacent) the histograms, expertList the list
        // heads, remaining the links.
        const int pieces = min(nt / 32, 2 * d.R);
        const int pieceRoutes = ((d.cap + pieces - 1) / pieces + 31) / 32 * 32;
        int32_t *hists = tb.srcCursor;
        int32_t *head = tb.expertList;
        int32_t *next = tb.remaining;
        const bool listed = g.localSegments <= d.R * d.E;
        for (int i = tid; i < pieces * d.E; i += nt) hists[i] = 0;
        for (int e = tid; e < d.E; e += nt) head[e] = -1;
        __syncthreads();
        if (tid / 32 < pieces) {
            const int begin = (tid / 32) * pieceRoutes;
            const int n = min(pieceRoutes, d.cap - begin);
            if (n > 0) RankRoutesByWarpDeep(a.topk + begin, t.ordinal + begin, hists + (tid / 32) * d.E, n, tid % 32);
        }
        if (listed) {
            for (int i = tid; i < g.localSegments; i += nt) next[i] = atomicExch(&head[tb.segments[i].expert], i);
        }
        __syncthreads();
        for (int e = tid; e < d.E; e += nt) {
            int32_t before = 0;
            for (int w = 0; w < pieces; ++w) {
                const int32_t v = hists[w * d.E + e];
                hists[w * d.E + e] = before;
                before += v;
            }
        }
        __syncthreads();
        plan2::Tables tr = t;
        tr.base = tb.base;
        tr.segments = tb.segments;
        for (int r = tid; r < d.cap; r += nt) {
            const int32_t expert = a.topk[r];
            const int32_t ordinal = t.ordinal[r] + hists[(r / pieceRoutes) * d.E + expert];
            t.ordinal[r] = ordinal;
            const int32_t raw = listed ? plan2::PlanRouteDstListed(d, tr, head, next, expert, ordinal) : plan2::PlanRouteDst(d, in, tr, g, r);
            if (raw < 0) sBadRoute = 1;
            a.out.dst[r] = raw < 0 ? 0 : raw;
        }
        __syncthreads();
        if (sBadRoute == 0) {
            for (int tok = tid; tok < d.S; tok += nt) plan2::PlanMarkDuplicates(d, a.out.dst, tok);
        }
    } else {
        for (int r = tid; r < d.cap; r += nt) a.out.dst[r] = 0;
    }
    __syncthreads();
    phaseDone(3);
    const bool routed = planned && plan2::PlanHasDestinations(g) && sBadRoute == 0;
    if (a.stageDst != nullptr) {
        // every route tells its destination which row it fills (the combine stage walks the rows)
        for (int r = tid; r < d.cap; r += nt) {
            const int32_t enc = a.out.dst[r];
            const int32_t raw = enc >= 0 ? enc : ~enc;
            a.stageDst[r] = routed ? raw : 0;
            if (routed) {
                const int dstRank = raw / d.nvS;
                uint64_t *cell = reinterpret_cast<uint64_t *>(DataHalf(a.comm, dstRank, w.epoch) + a.dstLocalOff) + (raw - dstRank * d.nvS);
                st_relaxed_sys_u64(cell, MakeFlag(w.epoch, static_cast<uint32_t>(d.rank * d.cap + r)));
            }
        }
        if (tid == 0 && routed) plan2::PlanZeroFill(d, t, a.out.cuSeqlens, a.stageZeroFill);
    }
    if (tid == 0) {
        for (int i = 0; i < TILEXR_MOONEP_PLAN_STATUS_WORDS; ++i) a.out.status[i] = 0;
        if (planned) {
            sFinal = plan2::PlanFinish(d, t, g, sBadRoute == 0, a.out.status);
        } else {
            sFinal = ok ? sValidate : PLAN_ERROR_INTERNAL_INVARIANT;
            a.out.status[0] = sFinal;
        }
    }
    __syncthreads();

    // 4. consensus: every rank ends with the largest status code
    if (ok) {
        if (tid < d.R) reinterpret_cast<Mail *>(MailBox(a, tid, d.rank, w.epoch))->status = sFinal;
        ok = MeetRanks(w, a, 2);
        if (ok && tid == 0) {
            int32_t worst = sFinal;
            for (int src = 0; src < d.R; ++src) {
                const int32_t s = reinterpret_cast<const volatile Mail *>(MailBox(a, d.rank, src, w.epoch))->status;
                if (s > worst) worst = s;
            }
            a.out.status[0] = worst;
            sFinal = worst;
        }
    }
    __syncthreads();
    if (a.stageDst != nullptr) {
        const bool usable = ok && routed && sFinal <= PLAN_PARTIAL_TOKEN_SUPPLY;
        if (usable) {
            const uint64_t *cells = reinterpret_cast<const uint64_t *>(DataHalf(a.comm, d.rank, w.epoch) + a.dstLocalOff);
            for (int s = tid; s < d.nvS; s += nt) {
                const uint64_t v = ld_relaxed_sys_u64(cells + s);
                a.stageDstLocal[s] = FlagEpoch(v) == w.epoch ? static_cast<int32_t>(FlagValue(v)) : -1;
            }
        }
        if (tid == 0) *a.stageStatus = usable ? 0 : (sFinal != PLAN_OK ? sFinal : PLAN_ERROR_INTERNAL_INVARIANT);
    }
    phaseDone(4);
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRMoonEpPlanV2Kernel, PlanV2Args, PlanV2Body, PLAN_V2_THREADS)

} // namespace

const KernelEntry &PlanV2KernelEntry() { return TileXRMoonEpPlanV2KernelEntry; }

} // namespace TileXR
