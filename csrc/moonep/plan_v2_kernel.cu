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
    __shared__ int sFinal;
    __shared__ uint64_t sHash;

    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_MOONEP_PLANNING, a.dims.cap, true);
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
    if (tid == 0) {
        int32_t v = (mismatch & 2) ? PLAN_ERROR_CONFIG_MISMATCH : (mismatch & 1) ? PLAN_ERROR_TPE_MISMATCH : PLAN_OK;
        if (ok && v == PLAN_OK) v = (bad & 2) ? PLAN_ERROR_CONFIG_MISMATCH : (bad & 1) ? PLAN_ERROR_TPE_MISMATCH : PLAN_OK;
        sValidate = v;
        g = plan2::Progress{};
        if (ok && v == PLAN_OK) {
            if (staged) {
                plan2::Tables ts;
                plan2::Carve(d, planShared, &ts);
                ts.ordinal = t.ordinal;                                             // not touched by the balancing
                ts.segments = reinterpret_cast<plan2::Segment *>(planShared + prefixWords + tpeWords);
                const plan2::Inputs ins{a.topk, planShared + prefixWords, a.globalIds};
                plan2::PlanBalance(d, ins, a.out, ts, g);
            } else {
                plan2::PlanBalance(d, in, a.out, t, g);
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
    const bool planned = ok && sValidate == PLAN_OK;
    if (planned && plan2::PlanHasDestinations(g)) {
        for (int e = tid; e < d.E; e += nt) plan2::PlanOrdinalsOfExpert(d, in, t, e);
        __syncthreads();
        for (int r = tid; r < d.cap; r += nt) {
            const int32_t raw = plan2::PlanRouteDst(d, in, t, g, r);
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
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRMoonEpPlanV2Kernel, PlanV2Args, PlanV2Body, PLAN_V2_THREADS)

} // namespace

const KernelEntry &PlanV2KernelEntry() { return TileXRMoonEpPlanV2KernelEntry; }

} // namespace TileXR
