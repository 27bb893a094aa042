// Flag-based rendezvous between ranks and between the blocks of one rank.
//
// A flag is a 64-bit word `(epoch << 32) | value` living in the flag area of a window.
// `epoch` is the low 32 bits of the launch's magic (TileXRCommNextMagic), so flag memory is
// never cleared: a wait compares the whole word with `>=`, which a later launch's flag also
// satisfies (the producer can only be in a later launch if it finished this one).  This is
// the reference's scheme (src/include/tilexr_sync.h:17-26, 81-123) with two changes that a
// shared GPU needs: every wait has a time budget, and a wait that gives up records a failure
// and raises an abort word in every peer so that no rank keeps spinning.
#ifndef TILEXR_SYNC_CUH
#define TILEXR_SYNC_CUH

#include "tilexr_platform.cuh"
#include "../tilexr_comm_args.h"

namespace tilexr {

using TileXR::CommArgs;

TXR_HD uint64_t MakeFlag(uint32_t epoch, uint32_t value) { return (static_cast<uint64_t>(epoch) << 32) | value; }
TXR_HD uint32_t FlagEpoch(uint64_t flag) { return static_cast<uint32_t>(flag >> 32); }
TXR_HD uint32_t FlagValue(uint64_t flag) { return static_cast<uint32_t>(flag & 0xffffffffu); }

TXR_D uint64_t *FlagSlot(const CommArgs *args, int owner, int64_t slot)
{
    return reinterpret_cast<uint64_t *>(args->peerMems[owner] + TILEXR_WIN_FLAG_OFFSET) + slot;
}

TXR_D uint64_t *CtrlWord(const CommArgs *args, int owner, int64_t word)
{
    return reinterpret_cast<uint64_t *>(args->peerMems[owner] + TILEXR_WIN_CTRL_OFFSET) + word;
}

TXR_D uint8_t *DataHalf(const CommArgs *args, int owner, uint32_t epoch)
{
    return args->peerMems[owner] + TILEXR_WIN_DATA_OFFSET + static_cast<uint64_t>(epoch & 1u) * args->dataHalfBytes;
}

// Half (epoch & 1) of the low-latency plane of `owner`: written only with epoch-tagged 16-byte units
// (tilexr_data_as_flag.cuh).  The halves alternate like the data halves and fall under the same reuse guard.
TXR_D uint8_t *LlHalf(const CommArgs *args, int owner, uint32_t epoch)
{
    return args->peerMems[owner] + TILEXR_WIN_LL_OFFSET + static_cast<uint64_t>(epoch & 1u) * TILEXR_WIN_LL_HALF_BYTES;
}

// Per-thread wait state.  `status` stays TILEXR_DEV_OK until the first failure; after that
// every wait returns false at once so the caller walks to the kernel's end without touching
// more flags (the reference's failed cores also keep walking its barrier skeleton).
struct Waiter {
    CommArgs *args;
    uint32_t epoch;
    int32_t block;
    int32_t status;
    uint64_t deadline;   // absolute ns, 0 = not started

    TXR_D bool ok() const { return status == TileXR::TILEXR_DEV_OK; }
};

// The epoch of a launch tags its flags.  On a GPU communicator it is kept on the device: every launch reads
// the epoch of the rank's last finished launch from its own control block and uses the next one, and the
// last block to leave stores it back (KernelEpilogue).  A launch therefore carries no per-call host state,
// so a captured CUDA graph can replay it; all ranks stay in step because they issue the same launches.
// Host-memory communicators (CPU plumbing) take the epoch from the host's magic counter.
TXR_D Waiter MakeWaiter(CommArgs *args, int64_t magic, int block)
{
    Waiter w;
    w.args = args;
    if (args->extraFlag & TileXR::TILEXR_FLAG_HOST_MEMORY) {
        w.epoch = static_cast<uint32_t>(magic);
    } else {
        w.epoch = static_cast<uint32_t>(ld_relaxed_sys_u64(CtrlWord(args, args->rank, TILEXR_CTRL_EPOCH_WORD))) + 1u;
    }
    w.block = block;
    w.status = TileXR::TILEXR_DEV_OK;
    w.deadline = 0;
    return w;
}

// First failure wins: the record in dfx[] describes the wait that gave up first on this rank.
TXR_D void RaiseFailure(Waiter &w, int code, int peer, int64_t slot, uint64_t expected, uint64_t observed)
{
    w.status = code;
    CommArgs *a = w.args;
    uint64_t *failCode = reinterpret_cast<uint64_t *>(&a->dfx[TileXR::TILEXR_DFX_FAIL_CODE]);
    if (atom_cas_sys_u64(failCode, 0, static_cast<uint64_t>(code)) == 0) {
        a->dfx[TileXR::TILEXR_DFX_FAIL_PEER] = peer;
        a->dfx[TileXR::TILEXR_DFX_FAIL_SLOT] = slot;
        a->dfx[TileXR::TILEXR_DFX_FAIL_EXPECTED] = static_cast<int64_t>(expected);
        a->dfx[TileXR::TILEXR_DFX_FAIL_OBSERVED] = static_cast<int64_t>(observed);
        a->dfx[TileXR::TILEXR_DFX_FAIL_BLOCK] = w.block;
        a->dfx[TileXR::TILEXR_DFX_RUN_STATUS] = TILEXR_RUN_FAILED;
    }
    if (code != TileXR::TILEXR_DEV_ABORTED) {
        // Tell everyone, ourselves included.  A rank whose window is gone is not reachable
        // anyway; the store is fire-and-forget.
        for (int r = 0; r < a->rankSize; ++r) {
            st_relaxed_sys_u64(CtrlWord(a, r, TILEXR_CTRL_ABORT_WORD), MakeFlag(w.epoch, static_cast<uint32_t>(code)));
        }
        fence_acq_rel_sys();
    }
}

TXR_D bool AbortRaised(const Waiter &w)
{
    return ld_relaxed_sys_u64(CtrlWord(w.args, w.args->rank, TILEXR_CTRL_ABORT_WORD)) != 0;
}

// Spin until `*flag >= MakeFlag(epoch, value)`.  Returns false (and records why) when the
// budget CommArgs::waitTimeoutNs runs out or the abort word is raised.
// Host builds tell a protocol recorder how a wait ended (tilexr_platform.cuh); device builds compile this away.
TXR_D void TraceWaitEnd(const uint64_t *flag, uint64_t want, uint64_t seen, int peer, bool satisfied)
{
#if !TXR_ON_DEVICE
    if (HostTraceHooks *h = HostTraceSlot()) h->onFlagWait(h->ctx, flag, want, seen, peer, satisfied ? 1 : 0);
#else
    (void)flag; (void)want; (void)seen; (void)peer; (void)satisfied;
#endif
}

TXR_D bool WaitFlagGE(Waiter &w, const uint64_t *flag, uint32_t value, int peer, int64_t slot, int failCode)
{
    if (!w.ok()) return false;
    const uint64_t want = MakeFlag(w.epoch, value);
    uint64_t seen = ld_acquire_sys_u64(flag);
    if (seen >= want) {
        TraceWaitEnd(flag, want, seen, peer, true);
        return true;
    }
    uint32_t polls = 0;
    for (;;) {
        seen = ld_acquire_sys_u64(flag);
        if (seen >= want) {
            TraceWaitEnd(flag, want, seen, peer, true);
            return true;
        }
        if ((++polls & 63u) == 0) {
            if (AbortRaised(w)) {
                TraceWaitEnd(flag, want, seen, peer, false);
                RaiseFailure(w, TileXR::TILEXR_DEV_ABORTED, peer, slot, want, seen);
                return false;
            }
            const uint64_t t = now_ns();
            if (w.deadline == 0) {
                w.deadline = t + w.args->waitTimeoutNs;
            } else if (t > w.deadline) {
                TraceWaitEnd(flag, want, seen, peer, false);
                RaiseFailure(w, failCode, peer, slot, want, seen);
                return false;
            }
        }
        spin_pause();
    }
}

TXR_D bool WaitFlagGE(Waiter &w, const uint64_t *flag, uint32_t value, int peer, int64_t slot)
{
    return WaitFlagGE(w, flag, value, peer, slot, TileXR::TILEXR_DEV_WAIT_TIMEOUT);
}

TXR_D void SetFlag(uint64_t *flag, uint32_t epoch, uint32_t value)
{
    st_release_sys_u64(flag, MakeFlag(epoch, value));
}

// Non-blocking probe (reference: CheckRankInnerFlag).
TXR_D bool CheckFlagGE(const uint64_t *flag, uint32_t epoch, uint32_t value)
{
    return ld_acquire_sys_u64(flag) >= MakeFlag(epoch, value);
}

// ---- barrier among the blocks of one rank -------------------------------------------------
// Generation barrier in the rank's own control block.  It needs every block of the launch to
// be resident, so kernels that use it are launched cooperatively.  `nBlocks` blocks call it
// with the same `index` (0..15).  Call from thread 0 of a block, between two block syncs.
TXR_D bool GridBarrierThread0(Waiter &w, int index, uint32_t nBlocks)
{
    if (nBlocks <= 1) return w.ok();
    uint32_t *pair = reinterpret_cast<uint32_t *>(CtrlWord(w.args, w.args->rank, TILEXR_CTRL_GRIDBAR_WORD + index));
    uint32_t *count = pair;
    uint32_t *gen = pair + 1;
    const uint32_t g = ld_acquire_gpu_u32(gen);
    if (atom_add_acq_rel_gpu_u32(count, 1) == nBlocks - 1) {
        st_release_gpu_u32(count, 0);
        st_release_gpu_u32(gen, g + 1);
        return w.ok();
    }
    uint32_t polls = 0;
    while (ld_acquire_gpu_u32(gen) == g) {
        if ((++polls & 63u) == 0) {
            const uint64_t t = now_ns();
            if (w.deadline == 0) {
                w.deadline = t + w.args->waitTimeoutNs;
            } else if (t > w.deadline) {
                RaiseFailure(w, TileXR::TILEXR_DEV_GRID_BARRIER_TIMEOUT, w.args->rank, index, nBlocks, g);
                return false;
            }
        }
        spin_pause();
    }
    return w.ok();
}

// ---- reuse guard --------------------------------------------------------------------------
// Data half (epoch & 1) was last used by launch epoch-2.  Before writing into a peer's half
// (or letting peers read ours again) make sure that peer finished launch epoch-2: it stores
// its finished epoch into doneEpoch[itsRank] of every window at kernel end (PublishDone).
TXR_D bool WaitPeerFinished(Waiter &w, int peer, uint32_t finishedEpoch)
{
    if (!w.ok()) return false;
    const uint64_t *done = CtrlWord(w.args, w.args->rank, TILEXR_CTRL_DONE_WORD + peer);
    const uint64_t want = MakeFlag(finishedEpoch, 0);
    uint32_t polls = 0;
    for (;;) {
        const uint64_t seen = ld_acquire_sys_u64(done);
        if (seen >= want) {
            TraceWaitEnd(done, want, seen, peer, true);
            return true;
        }
        if ((++polls & 63u) == 0) {
            if (AbortRaised(w)) {
                TraceWaitEnd(done, want, seen, peer, false);
                RaiseFailure(w, TileXR::TILEXR_DEV_ABORTED, peer, TILEXR_CTRL_DONE_WORD + peer, want, seen);
                return false;
            }
            const uint64_t t = now_ns();
            if (w.deadline == 0) {
                w.deadline = t + w.args->waitTimeoutNs;
            } else if (t > w.deadline) {
                TraceWaitEnd(done, want, seen, peer, false);
                RaiseFailure(w, TileXR::TILEXR_DEV_REUSE_GUARD_TIMEOUT, peer, TILEXR_CTRL_DONE_WORD + peer, want, seen);
                return false;
            }
        }
        spin_pause();
    }
}

// Written by one thread of the rank after all of the rank's blocks have finished their
// reads and writes of this launch.
TXR_D void PublishDone(const Waiter &w)
{
    CommArgs *a = w.args;
    // One fence orders everything this rank did before all of the stores below; a release store per peer would
    // wait for the previous peer's store to be acknowledged over NVLink, rankSize - 1 round trips in a row.
    fence_acq_rel_sys();
    for (int i = 0; i < a->rankSize; ++i) {
        const int r = (a->rank + i) % a->rankSize;
        st_relaxed_sys_u64(CtrlWord(a, r, TILEXR_CTRL_DONE_WORD + a->rank), MakeFlag(w.epoch, 0));
    }
}

#if defined(__CUDACC__)

// Block-level helpers: thread 0 waits, the block learns the outcome.
__device__ __forceinline__ bool BlockBroadcastOk(bool ok)
{
    return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Everything a kernel body does first: waiter for this thread, DFX record, reuse guard.
// Returns false when the guard failed; the kernel must then skip its work.
__device__ __forceinline__ bool KernelPrologue(Waiter &w, CommArgs *args, int64_t magic, int op, int64_t count,
                                               bool guard)
{
    w = MakeWaiter(args, magic, blockIdx.x);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        args->dfx[TileXR::TILEXR_DFX_MAGIC] = w.epoch;
        args->dfx[TileXR::TILEXR_DFX_OP] = op;
        args->dfx[TileXR::TILEXR_DFX_COUNT_ARG] = count;
        args->dfx[TileXR::TILEXR_DFX_RUN_STATUS] = TILEXR_RUN_STARTED;
    }
    bool ok = true;
    if (guard && w.epoch >= 3 && static_cast<int>(threadIdx.x) < args->rankSize &&
        static_cast<int>(threadIdx.x) != args->rank) {
        ok = WaitPeerFinished(w, threadIdx.x, w.epoch - 2);
    }
    return BlockBroadcastOk(ok);
}

// Everything a kernel body does last.  `exitCounter` is a 32-bit word in the rank's control
// block that counts finished blocks; the last block publishes the done epoch and the status.
// `scratchWords` operator scratch words of the rank's control block (work cursors and the like) are returned
// to zero by the last block, so that the next launch that uses them finds them clear.
__device__ __forceinline__ void KernelEpilogue(Waiter &w, bool ok, int scratchWords = 0)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        CommArgs *a = w.args;
        fence_acq_rel_sys();
        uint32_t *exitCounter =
            reinterpret_cast<uint32_t *>(CtrlWord(a, a->rank, TILEXR_CTRL_GRIDBAR_WORD + TILEXR_CTRL_GRIDBAR_COUNT));
        if (atom_add_acq_rel_gpu_u32(exitCounter, 1) == gridDim.x - 1) {
            for (int i = 0; i < scratchWords; ++i) *CtrlWord(a, a->rank, TILEXR_CTRL_SCRATCH_WORD + i) = 0;
            st_release_gpu_u32(exitCounter, 0);
            PublishDone(w);
            *CtrlWord(a, a->rank, TILEXR_CTRL_EPOCH_WORD) = w.epoch;
            if (a->dfx[TileXR::TILEXR_DFX_FAIL_CODE] == 0 && ok) {
                a->dfx[TileXR::TILEXR_DFX_RUN_STATUS] = TILEXR_RUN_FINISHED;
            }
            a->dfx[TileXR::TILEXR_DFX_LAUNCHES] += 1;
        }
    }
}

// Barrier among all blocks of this rank's launch, callable by whole blocks.
__device__ __forceinline__ bool GridBarrier(Waiter &w, int index)
{
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) {
        __threadfence();
        ok = GridBarrierThread0(w, index, gridDim.x);
    }
    return BlockBroadcastOk(ok);
}

#endif // __CUDACC__

// ---- SyncCollectives ------------------------------------------------------------------------
// The reference's helper class (src/include/tilexr_sync.h:28-394) keeps "inner" flags, one per
// block in the rank's own window, and "outer" flags that other ranks wait on.  The same
// surface is kept for code written against it; slots live in the operator flag region.
class SyncCollectives {
public:
    TXR_D void Init(CommArgs *args, int64_t magic, int block, int blockNum)
    {
        w_ = MakeWaiter(args, magic, block);
        block_ = block;
        blockNum_ = blockNum;
    }

    TXR_D Waiter &waiter() { return w_; }

    // eventID selects a flag slot; rank defaults to this rank's own window.
    TXR_D void SetSyncFlag(uint32_t value, int eventID, int rank)
    {
        SetFlag(FlagSlot(w_.args, rank, TILEXR_FLAG_OP_BASE + eventID), w_.epoch, value);
    }
    TXR_D bool WaitSyncFlag(uint32_t value, int eventID, int rank)
    {
        return WaitFlagGE(w_, FlagSlot(w_.args, rank, TILEXR_FLAG_OP_BASE + eventID), value, rank, eventID);
    }
    // Inner flags: slot = block index, in this rank's window.
    TXR_D void SetInnerFlag(uint32_t value) { SetSyncFlag(value, block_, w_.args->rank); }
    TXR_D void SetInnerFlag(uint32_t value, int block) { SetSyncFlag(value, block, w_.args->rank); }
    TXR_D bool WaitInnerFlag(uint32_t value, int block) { return WaitSyncFlag(value, block, w_.args->rank); }
    TXR_D bool WaitRankInnerFlag(uint32_t value, int rank, int block) { return WaitSyncFlag(value, block, rank); }
    TXR_D bool CheckRankInnerFlag(uint32_t value, int rank, int block)
    {
        return CheckFlagGE(FlagSlot(w_.args, rank, TILEXR_FLAG_OP_BASE + block), w_.epoch, value);
    }
    TXR_D uint64_t GetInnerFlag(int rank, int block)
    {
        return ld_acquire_sys_u64(FlagSlot(w_.args, rank, TILEXR_FLAG_OP_BASE + block));
    }
    // Outer flags: one per (block, source rank) in the destination's window, after the inner flags.
    TXR_D int OuterSlot(int block, int srcRank) const { return blockNum_ + block * TILEXR_MAX_RANK_SIZE + srcRank; }
    TXR_D void SetOuterFlag(uint32_t value, int dstRank)
    {
        SetSyncFlag(value, OuterSlot(block_, w_.args->rank), dstRank);
    }
    TXR_D bool WaitOneRankOuterFlag(uint32_t value, int srcRank)
    {
        return WaitSyncFlag(value, OuterSlot(block_, srcRank), w_.args->rank);
    }
    // Waits for every rank's outer flag, starting at rank+1 so that ranks do not all poll the
    // same producer first (reference: staggered start tilexr_sync.h:197).
    TXR_D bool WaitOuterFlag(uint32_t value)
    {
        bool ok = true;
        for (int i = 1; i <= w_.args->rankSize; ++i) {
            const int r = (w_.args->rank + i) % w_.args->rankSize;
            ok = WaitOneRankOuterFlag(value, r) && ok;
        }
        return ok;
    }
    TXR_D bool WaitAllRankPartOuterFlag(uint32_t value, int firstRank, int rankCount)
    {
        bool ok = true;
        for (int i = 0; i < rankCount; ++i) {
            ok = WaitOneRankOuterFlag(value, (firstRank + i) % w_.args->rankSize) && ok;
        }
        return ok;
    }
    TXR_D uint64_t GetOuterFlag(int srcRank)
    {
        return ld_acquire_sys_u64(FlagSlot(w_.args, w_.args->rank, TILEXR_FLAG_OP_BASE + OuterSlot(block_, srcRank)));
    }

private:
    Waiter w_;
    int block_;
    int blockNum_;
};

} // namespace tilexr

#endif // TILEXR_SYNC_CUH
