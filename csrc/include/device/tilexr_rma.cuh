// One-sided registered-memory verbs issued from inside a kernel: put, get, put-with-signal,
// signal, quiet.  This is the B200 counterpart of the reference's UDMA device API
// (src/include/tilexr_udma.h:636-1046).  There is no NIC queue between two GPUs behind an
// NVSwitch: a registered region of a peer is simply mapped into this GPU's address space, so
//
//   put     = vector stores (or a TMA bulk store from shared memory) to the peer mapping
//   get     = vector loads (or a non-multicast TMA bulk load) from the peer mapping
//   signal  = a release store / release add on a 64-bit word of the peer's signal plane
//   quiet   = a system-scope fence (plus bulk-group wait when TMA stores were used)
//   "QP"    = an ordering lane: operations issued by one thread are ordered by its fences;
//             independent lanes are simply different warps or blocks.
//
// What is kept from the reference is the registry: every access names a registered region
// handle and an offset, is range-checked on the device before the first byte moves, and a
// bad range yields a status instead of a fault (tilexr_udma.h:166-181, 692-709).
#ifndef TILEXR_RMA_CUH
#define TILEXR_RMA_CUH

#include "tilexr_sync.cuh"

namespace tilexr {

using TileXR::TileXRRegistry;

enum RmaStatus : int {
    RMA_OK = 0,
    RMA_BAD_REGISTRY = 1,
    RMA_BAD_HANDLE = 2,
    RMA_BAD_PEER = 3,
    RMA_OUT_OF_RANGE = 4,
    RMA_MISALIGNED = 5,
    RMA_TIMEOUT = 6,
};

// Validates [offset, offset+bytes) against region `handle` and returns the address of that
// range in rank `peer`'s copy of the region as mapped here; null with `*status` set on error.
// Usable on the host for tests.
TXR_D uint8_t *RmaTranslate(const TileXRRegistry *reg, uint32_t handle, int peer, uint64_t offset, uint64_t bytes,
                            int *status)
{
    if (reg == nullptr || reg->magic != TILEXR_REGISTRY_MAGIC) {
        *status = RMA_BAD_REGISTRY;
        return nullptr;
    }
    if (handle >= reg->regionCount || reg->regions[handle].bytes == 0) {
        *status = RMA_BAD_HANDLE;
        return nullptr;
    }
    if (peer < 0 || static_cast<uint32_t>(peer) >= reg->rankSize) {
        *status = RMA_BAD_PEER;
        return nullptr;
    }
    const uint64_t regionBytes = reg->regions[handle].bytes;
    if (offset > regionBytes || bytes > regionBytes - offset) {
        *status = RMA_OUT_OF_RANGE;
        return nullptr;
    }
    *status = RMA_OK;
    return reg->regions[handle].peerBase[peer] + offset;
}

// ---- cooperative copies: `lane` of `lanes` threads, 16-byte aligned fast path ----------------

TXR_D void CopyLanes(void *dst, const void *src, uint64_t bytes, int lane, int lanes)
{
    uint8_t *d = reinterpret_cast<uint8_t *>(dst);
    const uint8_t *s = reinterpret_cast<const uint8_t *>(src);
    if (((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(s)) & 15u) == 0) {
        const uint64_t vecs = bytes / 16;
        uint64_t i = lane;
        // four independent 16-byte transfers in flight per thread
        for (; i + 3ull * lanes < vecs; i += 4ull * lanes) {
            const Vec16 a = ld_vec16_stream(s + i * 16);
            const Vec16 b = ld_vec16_stream(s + (i + lanes) * 16);
            const Vec16 c = ld_vec16_stream(s + (i + 2ull * lanes) * 16);
            const Vec16 e = ld_vec16_stream(s + (i + 3ull * lanes) * 16);
            st_vec16(d + i * 16, a);
            st_vec16(d + (i + lanes) * 16, b);
            st_vec16(d + (i + 2ull * lanes) * 16, c);
            st_vec16(d + (i + 3ull * lanes) * 16, e);
        }
        for (; i < vecs; i += lanes) st_vec16(d + i * 16, ld_vec16_stream(s + i * 16));
        for (uint64_t b = vecs * 16 + lane; b < bytes; b += lanes) d[b] = s[b];
    } else {
        for (uint64_t b = lane; b < bytes; b += lanes) d[b] = s[b];
    }
}

// The same copy with eight 16-byte transfers in flight per thread, for stores that cross NVLink while many other
// ranks do the same (an all-to-all): an acknowledgement then takes several microseconds, and a warp has to cover that
// time with bytes on the way.  What is left after the full rounds (fewer than eight vectors per thread) goes in rounds
// of four with the missing ones switched off: one vector at a time, the second half of a 7 KB row on one warp would
// cost six round trips.  Both addresses 16-byte aligned, `bytes` a multiple of 16.
TXR_D void CopyLanesDeep(void *dst, const void *src, uint64_t bytes, int lane, int lanes)
{
    uint8_t *d = reinterpret_cast<uint8_t *>(dst);
    const uint8_t *s = reinterpret_cast<const uint8_t *>(src);
    const uint64_t vecs = bytes / 16;
    uint64_t i = lane;
    for (; i + 7ull * lanes < vecs; i += 8ull * lanes) {
        Vec16 q[8];
#if TXR_ON_DEVICE
#pragma unroll
#endif
        for (int u = 0; u < 8; ++u) q[u] = ld_vec16_stream(s + (i + static_cast<uint64_t>(u) * lanes) * 16);
#if TXR_ON_DEVICE
#pragma unroll
#endif
        for (int u = 0; u < 8; ++u) st_vec16(d + (i + static_cast<uint64_t>(u) * lanes) * 16, q[u]);
    }
    for (; i < vecs; i += 4ull * lanes) {
        Vec16 q[4];
#if TXR_ON_DEVICE
#pragma unroll
#endif
        for (int u = 0; u < 4; ++u) {
            const uint64_t k = i + static_cast<uint64_t>(u) * lanes;
            if (k < vecs) q[u] = ld_vec16_stream(s + k * 16);
        }
#if TXR_ON_DEVICE
#pragma unroll
#endif
        for (int u = 0; u < 4; ++u) {
            const uint64_t k = i + static_cast<uint64_t>(u) * lanes;
            if (k < vecs) st_vec16(d + k * 16, q[u]);
        }
    }
}

// put: local -> peer region.  Non-blocking: returns when the stores are issued.
TXR_D int PutNbi(const TileXRRegistry *reg, uint32_t handle, int peer, uint64_t dstOffset, const void *localSrc,
                 uint64_t bytes, int lane, int lanes)
{
    int st;
    uint8_t *dst = RmaTranslate(reg, handle, peer, dstOffset, bytes, &st);
    if (st != RMA_OK) return st;
    CopyLanes(dst, localSrc, bytes, lane, lanes);
    return RMA_OK;
}

// get: peer region -> local.
TXR_D int GetNbi(const TileXRRegistry *reg, uint32_t handle, int peer, uint64_t srcOffset, void *localDst,
                 uint64_t bytes, int lane, int lanes)
{
    int st;
    const uint8_t *src = RmaTranslate(reg, handle, peer, srcOffset, bytes, &st);
    if (st != RMA_OK) return st;
    CopyLanes(localDst, src, bytes, lane, lanes);
    return RMA_OK;
}

// Signal word `index` of rank `peer`'s signal plane.
TXR_D uint64_t *SignalWord(const CommArgs *args, int peer, uint32_t index)
{
    return reinterpret_cast<uint64_t *>(args->signalMems[peer] + static_cast<uint64_t>(index) * TILEXR_SIGNAL_STRIDE);
}
TXR_HD uint32_t SignalWordCount() { return static_cast<uint32_t>(TILEXR_CTRL_SIGNAL_BYTES / TILEXR_SIGNAL_STRIDE); }

// All earlier stores of the calling thread (and of threads it synchronised with) become
// visible before the signal.
TXR_D void SignalSet(const CommArgs *args, int peer, uint32_t index, uint64_t value)
{
    st_release_sys_u64(SignalWord(args, peer, index), value);
}
TXR_D void SignalAdd(const CommArgs *args, int peer, uint32_t index, uint64_t value)
{
    red_release_sys_add_u64(SignalWord(args, peer, index), value);
}

// put followed by a signal on the same peer.  `syncLanes` joins the cooperating threads so
// that one of them can publish the signal after everybody's stores.
template <typename SyncFn>
TXR_D int PutSignalNbi(const CommArgs *args, const TileXRRegistry *reg, uint32_t handle, int peer, uint64_t dstOffset,
                       const void *localSrc, uint64_t bytes, uint32_t signalIndex, uint64_t signalValue, int lane,
                       int lanes, SyncFn syncLanes)
{
    if (signalIndex >= SignalWordCount()) return RMA_OUT_OF_RANGE;
    const int st = PutNbi(reg, handle, peer, dstOffset, localSrc, bytes, lane, lanes);
    fence_acq_rel_sys();
    syncLanes();
    if (st == RMA_OK && lane == 0) SignalSet(args, peer, signalIndex, signalValue);
    return st;
}

// Completes every put/get the calling thread issued so far.
TXR_D int Quiet()
{
    fence_acq_rel_sys();
    return RMA_OK;
}

// Bounded wait for a signal word of this rank to reach `value` (monotone signals).
TXR_D int WaitSignalGE(Waiter &w, uint32_t index, uint64_t value)
{
    const uint64_t *p = SignalWord(w.args, w.args->rank, index);
    uint32_t polls = 0;
    for (;;) {
        const uint64_t seen = ld_acquire_sys_u64(p);
        if (seen >= value) return RMA_OK;
        if (!w.ok()) return RMA_TIMEOUT;
        if ((++polls & 63u) == 0) {
            const uint64_t t = now_ns();
            if (w.deadline == 0) {
                w.deadline = t + w.args->waitTimeoutNs;
            } else if (t > w.deadline || AbortRaised(w)) {
                RaiseFailure(w, TileXR::TILEXR_DEV_WAIT_TIMEOUT, w.args->rank, index, value, seen);
                return RMA_TIMEOUT;
            }
        }
        spin_pause();
    }
}

#if defined(__CUDACC__)

// ---- TMA (bulk async copy) forms, one issuing thread ----------------------------------------
// Untiled cp.async.bulk: both addresses 16-byte aligned, size a multiple of 16.  The load form
// is the plain one: no cluster multicast, so it may read a peer's memory.

__device__ __forceinline__ uint32_t SmemAddr(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void MbarInit(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarInitFence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done) : "r"(SmemAddr(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded: gives up after `budgetNs`.  Returns false on timeout.
__device__ __forceinline__ bool MbarWait(uint64_t *bar, uint32_t parity, uint64_t budgetNs)
{
    if (MbarTryWait(bar, parity)) return true;
    uint64_t deadline = 0;
    uint32_t polls = 0;
    for (;;) {
        if (MbarTryWait(bar, parity)) return true;
        if ((++polls & 255u) == 0) {
            const uint64_t t = now_ns();
            if (deadline == 0) deadline = t + budgetNs;
            else if (t > deadline) return false;
        }
    }
}

__device__ __forceinline__ void BulkLoadToSmem(void *smemDst, const void *gmemSrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(SmemAddr(smemDst)), "l"(gmemSrc), "r"(bytes), "r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ void BulkStoreFromSmem(void *gmemDst, const void *smemSrc, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gmemDst), "r"(SmemAddr(smemSrc)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void BulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void BulkWaitRead()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void BulkWait()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

#endif // __CUDACC__

} // namespace tilexr

#endif // TILEXR_RMA_CUH
