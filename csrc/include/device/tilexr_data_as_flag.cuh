// In-band readiness: the payload itself tells the reader that it has arrived, so a row needs
// one transfer instead of "data, fence, flag".
//
// Two layouts are provided.
//
//  * LL16: every 16-byte unit carries 12 payload bytes and a 4-byte epoch.  A 16-byte aligned
//    vector store is a single transaction on NVLink, so an observed epoch proves the other
//    twelve bytes.  Because the epoch changes with every launch, consumed units are never
//    cleared.  Use for latency-bound rows (decode all-reduce, small EP batches).
//
//  * Block512: the reference's layout (src/include/tilexr_data_as_flag.h:22-53): 480 payload
//    bytes followed by a 32-byte flag unit, 512 bytes per block.  The reference marks a block
//    ready with the float 1.0 and clears it after use; here the first flag word holds the
//    launch epoch (never zero) and the seven others hold 1.0f, so both "sum of flags" checks
//    and epoch checks work and clearing is optional.  The payload and the flag unit are two
//    ordered stores (payload, system fence, flag), which is correct on any interconnect.
//
// Size helpers are usable from host code.
#ifndef TILEXR_DATA_AS_FLAG_CUH
#define TILEXR_DATA_AS_FLAG_CUH

#include "tilexr_sync.cuh"

namespace tilexr {

constexpr uint32_t DATA_AS_FLAG_BLOCK_BYTES = 512;
constexpr uint32_t DATA_AS_FLAG_PAYLOAD_BYTES = 480;
constexpr uint32_t DATA_AS_FLAG_FLAG_BYTES = 32;
constexpr uint32_t DATA_AS_FLAG_FLAG_OFFSET = 480;
constexpr uint32_t DATA_AS_FLAG_FLAG_FLOATS = 8;
constexpr float DATA_AS_FLAG_READY = 1.0f;

static_assert(DATA_AS_FLAG_PAYLOAD_BYTES + DATA_AS_FLAG_FLAG_BYTES == DATA_AS_FLAG_BLOCK_BYTES, "block layout");

TXR_HD uint64_t DataAsFlagBlockCount(uint64_t payloadBytes)
{
    return (payloadBytes + DATA_AS_FLAG_PAYLOAD_BYTES - 1) / DATA_AS_FLAG_PAYLOAD_BYTES;
}
TXR_HD uint64_t DataAsFlagPackedBytes(uint64_t payloadBytes)
{
    return DataAsFlagBlockCount(payloadBytes) * DATA_AS_FLAG_BLOCK_BYTES;
}

constexpr uint32_t LL16_UNIT_BYTES = 16;
constexpr uint32_t LL16_PAYLOAD_BYTES = 12;

TXR_HD uint64_t Ll16UnitCount(uint64_t payloadBytes) { return (payloadBytes + LL16_PAYLOAD_BYTES - 1) / LL16_PAYLOAD_BYTES; }
TXR_HD uint64_t Ll16PackedBytes(uint64_t payloadBytes) { return Ll16UnitCount(payloadBytes) * LL16_UNIT_BYTES; }

// ---- LL16 -----------------------------------------------------------------------------------
// `lane`/`lanes` describe the cooperating threads (a warp: lane id / 32, a block: tid / size).
// The payload length must be a multiple of 4 bytes; a trailing partial unit is zero padded.

TXR_D void Ll16Send(void *dst, const void *src, uint64_t payloadBytes, uint32_t epoch, int lane, int lanes)
{
    const uint64_t units = Ll16UnitCount(payloadBytes);
    const uint32_t *s = reinterpret_cast<const uint32_t *>(src);
    const uint64_t words = payloadBytes / 4;
    for (uint64_t u = lane; u < units; u += lanes) {
        Vec16 v;
        const uint64_t w0 = u * 3;
        v.x = w0 < words ? s[w0] : 0u;
        v.y = w0 + 1 < words ? s[w0 + 1] : 0u;
        v.z = w0 + 2 < words ? s[w0 + 2] : 0u;
        v.w = epoch;
        st_vec16_flagged(reinterpret_cast<uint8_t *>(dst) + u * LL16_UNIT_BYTES, v);
    }
}

// One unit, stored with a single 16-byte transaction.
TXR_D void Ll16SendUnit(void *dst, uint32_t a, uint32_t b, uint32_t c, uint32_t epoch)
{
    st_vec16_flagged(dst, Vec16{a, b, c, epoch});
}

// Polls one unit until it carries the waiter's epoch.  Returns false if the budget ran out or another rank
// raised the abort word; `index` only labels the failure record.
TXR_D bool Ll16WaitUnit(Waiter &w, const void *unit, int peer, int64_t index, Vec16 *out)
{
    Vec16 v = ld_vec16_volatile(unit);
    uint32_t polls = 0;
    while (v.w != w.epoch) {
        if (!w.ok()) return false;
        if ((++polls & 63u) == 0) {
            if (AbortRaised(w)) {
                RaiseFailure(w, TileXR::TILEXR_DEV_ABORTED, peer, index, w.epoch, v.w);
                return false;
            }
            const uint64_t t = now_ns();
            if (w.deadline == 0) {
                w.deadline = t + w.args->waitTimeoutNs;
            } else if (t > w.deadline) {
                RaiseFailure(w, TileXR::TILEXR_DEV_WAIT_TIMEOUT, peer, index, w.epoch, v.w);
                return false;
            }
        }
        spin_pause();
        v = ld_vec16_volatile(unit);
    }
    *out = v;
    return true;
}

// Polls each unit until it carries `epoch`, then stores its payload words to `dst`.
// Returns false if the waiter's budget ran out.
TXR_D bool Ll16Recv(Waiter &w, void *dst, const void *src, uint64_t payloadBytes, int peer, int lane, int lanes)
{
    const uint64_t units = Ll16UnitCount(payloadBytes);
    uint32_t *d = reinterpret_cast<uint32_t *>(dst);
    const uint64_t words = payloadBytes / 4;
    for (uint64_t u = lane; u < units; u += lanes) {
        const uint8_t *p = reinterpret_cast<const uint8_t *>(src) + u * LL16_UNIT_BYTES;
        Vec16 v;
        if (!Ll16WaitUnit(w, p, peer, static_cast<int64_t>(u), &v)) return false;
        const uint64_t w0 = u * 3;
        if (w0 < words) d[w0] = v.x;
        if (w0 + 1 < words) d[w0 + 1] = v.y;
        if (w0 + 2 < words) d[w0 + 2] = v.z;
    }
    return w.ok();
}

// ---- Block512 -------------------------------------------------------------------------------

// Writes `payloadBytes` (multiple of 16) as 512-byte blocks at `dst`.  Call with all `lanes`
// cooperating threads; `syncLanes` must synchronise them (__syncwarp / __syncthreads).
template <typename SyncFn>
TXR_D void DataAsFlagSend(void *dst, const void *src, uint64_t payloadBytes, uint32_t epoch, int lane, int lanes,
                          SyncFn syncLanes)
{
    const uint64_t blocks = DataAsFlagBlockCount(payloadBytes);
    const uint64_t vecs = payloadBytes / 16;
    constexpr uint64_t VECS_PER_BLOCK = DATA_AS_FLAG_PAYLOAD_BYTES / 16;   // 30
    for (uint64_t i = lane; i < vecs; i += lanes) {
        const uint64_t blk = i / VECS_PER_BLOCK;
        const uint64_t off = i % VECS_PER_BLOCK;
        st_vec16(reinterpret_cast<uint8_t *>(dst) + blk * DATA_AS_FLAG_BLOCK_BYTES + off * 16,
                 ld_vec16(reinterpret_cast<const uint8_t *>(src) + i * 16));
    }
    fence_acq_rel_sys();
    syncLanes();
    const float ready = DATA_AS_FLAG_READY;
    uint32_t readyBits;
    memcpy(&readyBits, &ready, 4);
    for (uint64_t b = lane; b < blocks; b += lanes) {
        uint8_t *f = reinterpret_cast<uint8_t *>(dst) + b * DATA_AS_FLAG_BLOCK_BYTES + DATA_AS_FLAG_FLAG_OFFSET;
        Vec16 hi{readyBits, readyBits, readyBits, readyBits};
        Vec16 lo{epoch, readyBits, readyBits, readyBits};
        st_vec16(f + 16, hi);
        st_vec16_flagged(f, lo);
    }
}

// True when the first `blocks` blocks at `src` all carry `epoch`.
TXR_D bool DataAsFlagCheck(const void *src, uint64_t blocks, uint32_t epoch)
{
    for (uint64_t b = 0; b < blocks; ++b) {
        const uint8_t *f = reinterpret_cast<const uint8_t *>(src) + b * DATA_AS_FLAG_BLOCK_BYTES + DATA_AS_FLAG_FLAG_OFFSET;
        if (ld_vec16_volatile(f).x != epoch) return false;
    }
    return true;
}

// Waits (bounded) for every block, then copies the compacted payload to `dst`.
template <typename SyncFn>
TXR_D bool DataAsFlagCheckAndRecv(Waiter &w, void *dst, const void *src, uint64_t payloadBytes, int peer, int lane,
                                  int lanes, SyncFn syncLanes)
{
    const uint64_t blocks = DataAsFlagBlockCount(payloadBytes);
    for (uint64_t b = lane; b < blocks; b += lanes) {
        const uint64_t *f = reinterpret_cast<const uint64_t *>(reinterpret_cast<const uint8_t *>(src) +
                                                               b * DATA_AS_FLAG_BLOCK_BYTES + DATA_AS_FLAG_FLAG_OFFSET);
        uint32_t polls = 0;
        while (static_cast<uint32_t>(ld_acquire_sys_u64(f)) != w.epoch) {
            if (!w.ok()) break;
            if ((++polls & 63u) == 0) {
                const uint64_t t = now_ns();
                if (w.deadline == 0) {
                    w.deadline = t + w.args->waitTimeoutNs;
                } else if (t > w.deadline || AbortRaised(w)) {
                    RaiseFailure(w, TileXR::TILEXR_DEV_WAIT_TIMEOUT, peer, static_cast<int64_t>(b), w.epoch, 0);
                    break;
                }
            }
            spin_pause();
        }
    }
    syncLanes();
    if (!w.ok()) return false;
    const uint64_t vecs = payloadBytes / 16;
    constexpr uint64_t VECS_PER_BLOCK = DATA_AS_FLAG_PAYLOAD_BYTES / 16;
    for (uint64_t i = lane; i < vecs; i += lanes) {
        const uint64_t blk = i / VECS_PER_BLOCK;
        const uint64_t off = i % VECS_PER_BLOCK;
        st_vec16(reinterpret_cast<uint8_t *>(dst) + i * 16,
                 ld_vec16_stream(reinterpret_cast<const uint8_t *>(src) + blk * DATA_AS_FLAG_BLOCK_BYTES + off * 16));
    }
    return true;
}

// Clears the flag units of `blocks` blocks (only needed by code that reuses a slot within
// one epoch) and reports whether they read back as zero.
TXR_D void DataAsFlagClear(void *dst, uint64_t blocks, int lane, int lanes)
{
    for (uint64_t b = lane; b < blocks; b += lanes) {
        uint8_t *f = reinterpret_cast<uint8_t *>(dst) + b * DATA_AS_FLAG_BLOCK_BYTES + DATA_AS_FLAG_FLAG_OFFSET;
        Vec16 z{0, 0, 0, 0};
        st_vec16(f, z);
        st_vec16(f + 16, z);
    }
}
TXR_D bool CheckBatchCleared(const void *src, uint64_t blocks)
{
    for (uint64_t b = 0; b < blocks; ++b) {
        const uint8_t *f = reinterpret_cast<const uint8_t *>(src) + b * DATA_AS_FLAG_BLOCK_BYTES + DATA_AS_FLAG_FLAG_OFFSET;
        const Vec16 v = ld_vec16_volatile(f);
        if ((v.x | v.y | v.z | v.w) != 0) return false;
    }
    return true;
}

} // namespace tilexr

#endif // TILEXR_DATA_AS_FLAG_CUH
