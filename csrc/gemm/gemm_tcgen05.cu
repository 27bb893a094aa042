// bf16/fp16 GEMM on Blackwell's fifth-generation tensor cores, alone or fused with a collective.
//
//   C[M,N] = A[M,K] x B[N,K]^T      (both operands K-major, fp32 accumulation, 16-bit output)
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//               of a 128x64 A tile and a 256x64 B tile per stage into a 4-stage ring;
//   warp 1      one lane issues tcgen05.mma (M128 N256 K16, cta_group::1); the fp32 accumulator
//               lives in tensor memory, 2 x 256 columns so that the next tile's main loop
//               overlaps this tile's epilogue;
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp owns 32 TMEM lanes = 32 rows),
//               convert, store.
// Every mbarrier wait is bounded: if one gives up, the CTA raises a shared abort flag, every
// role leaves its loop, tensor memory is released and `status` tells the host.
//
// All-gather -> GEMM: the leading `commBlocks` CTAs do no math; they push this rank's A shard
// into every peer's staging buffer in (128 rows x K/4) pieces and raise one flag per piece.
// The GEMM CTAs start on the local shard and then walk the other shards in ring order; the
// TMA lane acquires the piece's flag before it loads from the staging buffer.  Remote data is
// therefore read by TMA from LOCAL memory only.
//
// GEMM -> reduce-scatter: tiles are produced owner by owner starting with rank+1; the epilogue
// stores each partial tile straight into the owner's staging slot for this source and raises a
// flag; when a CTA has no GEMM tile left its epilogue warps reduce the tiles this rank owns in
// rank order (bit-identical to a staged reduce-scatter of the same 16-bit partials).
//
// The reference names these operators (ALL_GATHER_MATMUL, MATMUL_REDUCE_SCATTER) but ships no
// kernel for them (src/include/tilexr_types.h:108-125).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "gemm_kernels.cuh"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr int FLAG_PLANE_A = TILEXR_FLAG_DATA_BASE;
constexpr int FLAG_PLANE_B = TILEXR_FLAG_ACK_BASE;
constexpr uint32_t TMEM_COLS = 512;

struct SharedState {
    uint64_t full[GEMM_STAGES];
    uint64_t empty[GEMM_STAGES];
    uint64_t tmemFull[2];
    uint64_t tmemEmpty[2];
    uint32_t tmemBase;
    volatile int abortFlag;
};

// ---- PTX wrappers --------------------------------------------------------------------------------

__device__ __forceinline__ void TmaLoad2D(void *smemDst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(SmemAddr(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(SmemAddr(bar))
        : "memory");
}

__device__ __forceinline__ void TmaPrefetchDescriptor(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile written by TMA with 128-byte swizzle: rows of 128 bytes, 8-row groups
// 1024 bytes apart.  Bits: [0,14) address>>4, [16,30) leading offset>>4 (unused here),
// [32,46) stride offset>>4, [46,48) version = 1, [61,64) layout = 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t MakeSmemDesc(uint32_t smemAddr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smemAddr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// kind::f16 instruction descriptor: D fp32 (bits 4-5 = 1), A/B format at bits 7-9 / 10-12
// (0 = fp16, 1 = bf16), both K-major, N>>3 at bits 17-22, M>>4 at bits 24-28.
__device__ __forceinline__ uint32_t MakeInstrDesc(bool bf16)
{
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(GEMM_BN >> 3) << 17) |
           (static_cast<uint32_t>(GEMM_BM >> 4) << 24);
}

__device__ __forceinline__ void UmmaF16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void UmmaCommit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

__device__ __forceinline__ void TmemLoad32(uint32_t taddr, uint32_t *r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void TmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded mbarrier wait that also gives up when another role raised the abort flag.
__device__ __forceinline__ bool WaitBar(uint64_t *bar, uint32_t parity, SharedState *st, uint64_t budgetNs)
{
    if (MbarTryWait(bar, parity)) return true;
    uint64_t deadline = 0;
    uint32_t polls = 0;
    for (;;) {
        if (MbarTryWait(bar, parity)) return true;
        if ((++polls & 127u) == 0) {
            if (st->abortFlag != 0) return false;
            const uint64_t t = now_ns();
            if (deadline == 0) {
                deadline = t + budgetNs;
            } else if (t > deadline) {
                st->abortFlag = 1;
                return false;
            }
        }
    }
}

struct TileCoord {
    int mBlock;     // row block of the whole product
    int nBlock;
    int shard;      // owner / source rank of the row block (fused modes)
    int mLocal;     // row block inside the shard
};

// Order in which a rank walks its tiles.  Row blocks advance fastest inside a group, so CTAs
// that run side by side share a B tile and the group's A rows stay in L2.
__device__ __forceinline__ TileCoord TileAt(const GemmArgs &a, int t, int rank, int ranks)
{
    TileCoord c;
    if (a.mode == GEMM_PLAIN) {
        constexpr int GROUP = 8;
        const int perGroup = GROUP * a.nBlocks;
        const int group = t / perGroup;
        const int first = group * GROUP;
        const int size = min(GROUP, a.mBlocks - first);
        const int u = t - group * perGroup;
        c.mBlock = first + u % size;
        c.nBlock = u / size;
        c.shard = 0;
        c.mLocal = c.mBlock;
    } else {
        const int perShard = a.blocksPerShard * a.nBlocks;
        const int i = t / perShard;
        const int u = t - i * perShard;
        c.shard = a.mode == GEMM_ALL_GATHER ? (rank + i) % ranks : (rank + 1 + i) % ranks;
        c.mLocal = u % a.blocksPerShard;
        c.nBlock = u / a.blocksPerShard;
        c.mBlock = c.shard * a.blocksPerShard + c.mLocal;
    }
    return c;
}

__device__ __forceinline__ uint32_t PackPair(float lo, float hi, bool bf16)
{
    if (bf16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&v);
    }
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

__device__ void GemmBody(const GemmArgs &a)
{
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t *stageBase = smem;
    SharedState *st = reinterpret_cast<SharedState *>(smem + GEMM_STAGES * GEMM_STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const bool fused = a.mode != GEMM_PLAIN;
    Waiter w;
    bool ok = true;
    int rank = 0, ranks = 1;
    if (fused) {
        // The staging buffers are not double buffered: nobody may write into a peer's staging
        // buffer before that peer finished the previous launch on this communicator.
        w = MakeWaiter(a.comm, a.magic, blockIdx.x);
        rank = a.comm->rank;
        ranks = a.comm->rankSize;
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            a.comm->dfx[TILEXR_DFX_MAGIC] = w.epoch;
            a.comm->dfx[TILEXR_DFX_OP] = a.mode == GEMM_ALL_GATHER ? TILEXR_OP_ALL_GATHER_MATMUL : TILEXR_OP_MATMUL_REDUCE_SCATTER;
            a.comm->dfx[TILEXR_DFX_RUN_STATUS] = TILEXR_RUN_STARTED;
        }
        bool g = true;
        if (w.epoch >= 2 && static_cast<int>(threadIdx.x) < ranks && static_cast<int>(threadIdx.x) != rank) {
            g = WaitPeerFinished(w, threadIdx.x, w.epoch - 1);
        }
        ok = BlockBroadcastOk(g);
    }
    const uint64_t budgetNs = fused ? a.comm->waitTimeoutNs : 4000000000ull;
    const uint32_t epoch = fused ? w.epoch : 0;

    // ---- all-gather: CTAs that only move data ----------------------------------------------------------
    if (fused && a.mode == GEMM_ALL_GATHER && blockIdx.x < a.commBlocks) {
        if (ok) {
            const TileXRRegistry *reg = a.comm->registryPtr;
            const int pieces = a.blocksPerShard * a.kChunks;
            const int64_t items = static_cast<int64_t>(ranks - 1) * pieces;
            const uint64_t rowBytes = static_cast<uint64_t>(a.K) * 2;
            const uint64_t chunkBytes = static_cast<uint64_t>(a.kBlocksPerChunk) * GEMM_BK * 2;
            for (int64_t it = blockIdx.x; it < items; it += a.commBlocks) {
                // peer rank-1 needs this shard first, then rank-2, ...
                const int peer = (rank - 1 - static_cast<int>(it / pieces) + 2 * ranks) % ranks;
                const int piece = static_cast<int>(it % pieces);
                const int mLocal = piece / a.kChunks;
                const int kc = piece % a.kChunks;
                const uint64_t colOff = kc * chunkBytes;
                const uint64_t n = min(chunkBytes, rowBytes > colOff ? rowBytes - colOff : 0);
                uint8_t *dstBase = reg->regions[a.stageHandle].peerBase[peer] + a.stageOffset +
                                   (static_cast<uint64_t>(rank) * a.shardRows + static_cast<uint64_t>(mLocal) * GEMM_BM) * rowBytes + colOff;
                const uint8_t *srcBase = a.aLocal + static_cast<uint64_t>(mLocal) * GEMM_BM * rowBytes + colOff;
                const int rows = min(GEMM_BM, a.shardRows - mLocal * GEMM_BM);
                for (int r = warp; r < rows; r += GEMM_THREADS / 32) {
                    CopyLanes(dstBase + r * rowBytes, srcBase + r * rowBytes, n, lane, 32);
                }
                __syncthreads();
                if (threadIdx.x == 0) {
                    SetFlag(FlagSlot(a.comm, peer, FLAG_PLANE_A + static_cast<int64_t>(rank) * a.flagStride + piece), epoch, 1);
                }
            }
        }
        KernelEpilogue(w, ok);
        return;
    }

    // ---- set-up -------------------------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; ++s) {
            MbarInit(&st->full[s], 1);
            MbarInit(&st->empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            MbarInit(&st->tmemFull[i], 1);
            MbarInit(&st->tmemEmpty[i], 4);
        }
        st->abortFlag = ok ? 0 : 1;
        MbarInitFence();
        TmaPrefetchDescriptor(&a.tmapA);
        TmaPrefetchDescriptor(&a.tmapB);
        if (a.mode == GEMM_ALL_GATHER) TmaPrefetchDescriptor(&a.tmapALocal);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&st->tmemBase)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmemBase = st->tmemBase;

    const int firstCta = (fused && a.mode == GEMM_ALL_GATHER) ? static_cast<int>(a.commBlocks) : 0;
    const int cta = static_cast<int>(blockIdx.x) - firstCta;
    const int nCta = static_cast<int>(gridDim.x) - firstCta;
    const int totalTiles = a.mBlocks * a.nBlocks;
    const bool bf16 = a.isBf16 != 0;

    if (warp == 0) {
        // ---- TMA producer -----------------------------------------------------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (int t = cta; t < totalTiles && st->abortFlag == 0; t += nCta) {
                const TileCoord tc = TileAt(a, t, rank, ranks);
                const bool remoteA = a.mode == GEMM_ALL_GATHER && tc.shard != rank;
                const CUtensorMap *mapA = (a.mode == GEMM_ALL_GATHER && !remoteA) ? &a.tmapALocal : &a.tmapA;
                const int rowA = (a.mode == GEMM_ALL_GATHER && !remoteA) ? tc.mLocal * GEMM_BM : tc.mBlock * GEMM_BM;
                for (int kb = 0; kb < a.kBlocks; ++kb) {
                    if (!WaitBar(&st->empty[stage], phase ^ 1u, st, budgetNs)) break;
                    if (remoteA && kb % a.kBlocksPerChunk == 0) {
                        const int piece = tc.mLocal * a.kChunks + kb / a.kBlocksPerChunk;
                        const int64_t slot = FLAG_PLANE_A + static_cast<int64_t>(tc.shard) * a.flagStride + piece;
                        if (!WaitFlagGE(w, FlagSlot(a.comm, rank, slot), 1, tc.shard, slot)) {
                            st->abortFlag = 1;
                            break;
                        }
                        fence_proxy_async();   // the rows were written by a peer's stores, TMA reads them next
                    }
                    uint8_t *sa = stageBase + stage * GEMM_STAGE_BYTES;
                    uint8_t *sb = sa + GEMM_STAGE_A_BYTES;
                    MbarExpectTx(&st->full[stage], GEMM_STAGE_BYTES);
                    TmaLoad2D(sa, mapA, kb * GEMM_BK, rowA, &st->full[stage]);
                    TmaLoad2D(sb, &a.tmapB, kb * GEMM_BK, tc.nBlock * GEMM_BN, &st->full[stage]);
                    if (++stage == GEMM_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = MakeInstrDesc(bf16);
            uint32_t stage = 0, phase = 0;
            int iter = 0;
            for (int t = cta; t < totalTiles && st->abortFlag == 0; t += nCta, ++iter) {
                const int acc = iter & 1;
                const uint32_t accPhase = (iter >> 1) & 1;
                if (!WaitBar(&st->tmemEmpty[acc], accPhase ^ 1u, st, budgetNs)) break;
                TcFenceAfter();
                const uint32_t tmemD = tmemBase + static_cast<uint32_t>(acc) * GEMM_BN;
                bool broke = false;
                for (int kb = 0; kb < a.kBlocks; ++kb) {
                    if (!WaitBar(&st->full[stage], phase, st, budgetNs)) {
                        broke = true;
                        break;
                    }
                    TcFenceAfter();
                    const uint32_t sa = SmemAddr(stageBase + stage * GEMM_STAGE_BYTES);
                    const uint64_t descA = MakeSmemDesc(sa);
                    const uint64_t descB = MakeSmemDesc(sa + GEMM_STAGE_A_BYTES);
#pragma unroll
                    for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
                        // 16 elements = 32 bytes further along K inside the swizzled row
                        UmmaF16(tmemD, descA + static_cast<uint64_t>(k * 2), descB + static_cast<uint64_t>(k * 2), idesc,
                                (kb | k) != 0 ? 1u : 0u);
                    }
                    UmmaCommit(&st->empty[stage]);   // the stage may be refilled once these MMAs have read it
                    if (++stage == GEMM_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (broke) break;
                UmmaCommit(&st->tmemFull[acc]);
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31 -----------------------------------------------
        const int quad = warp & 3;
        const int rowInTile = quad * 32 + lane;
        const TileXRRegistry *reg = fused ? a.comm->registryPtr : nullptr;
        int iter = 0;
        for (int t = cta; t < totalTiles; t += nCta, ++iter) {
            const TileCoord tc = TileAt(a, t, rank, ranks);
            const int acc = iter & 1;
            const uint32_t accPhase = (iter >> 1) & 1;
            bool got = true;
            if (lane == 0) got = WaitBar(&st->tmemFull[acc], accPhase, st, budgetNs);
            got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
            if (!got) break;
            TcFenceAfter();
            // where this thread's row goes
            const int64_t row = static_cast<int64_t>(tc.mBlock) * GEMM_BM + rowInTile;
            uint8_t *dstRow;
            bool rowValid;
            if (a.mode == GEMM_REDUCE_SCATTER) {
                const int64_t localRow = static_cast<int64_t>(tc.mLocal) * GEMM_BM + rowInTile;
                rowValid = localRow < a.shardRows;
                dstRow = reg->regions[a.stageHandle].peerBase[tc.shard] + a.stageOffset +
                         (static_cast<uint64_t>(rank) * a.shardRows + static_cast<uint64_t>(localRow)) * a.N * 2;
            } else {
                rowValid = row < a.M;
                dstRow = a.c + static_cast<uint64_t>(row) * a.N * 2;
            }
            const int col0 = tc.nBlock * GEMM_BN;
#pragma unroll 1
            for (int c = 0; c < GEMM_BN / 32; ++c) {
                uint32_t r[32];
                const uint32_t taddr = tmemBase + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * GEMM_BN + c * 32);
                TmemLoad32(taddr, r);
                TmemLoadWait();
                const int col = col0 + c * 32;
                if (rowValid && col < a.N) {
                    uint32_t packed[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) packed[j] = PackPair(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), bf16);
                    uint8_t *p = dstRow + static_cast<uint64_t>(col) * 2;
                    if (col + 32 <= a.N) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) st_vec16(p + v * 16, Vec16{packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]});
                    } else {
                        for (int j = 0; j < 32 && col + j < a.N; ++j) {
                            reinterpret_cast<uint16_t *>(p)[j] = static_cast<uint16_t>(j & 1 ? packed[j >> 1] >> 16 : packed[j >> 1] & 0xffffu);
                        }
                    }
                }
            }
            // the accumulator buffer may be overwritten by the tile after next
            TcFenceBefore();
            __syncwarp();
            if (lane == 0) MbarArrive(&st->tmemEmpty[acc]);
            if (a.mode == GEMM_REDUCE_SCATTER) {
                // all four epilogue warps have stored their rows of the tile: announce it to the owner
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int tileLocal = tc.mLocal * a.nBlocks + tc.nBlock;
                    SetFlag(FlagSlot(a.comm, tc.shard, FLAG_PLANE_B + static_cast<int64_t>(rank) * a.flagStride + tileLocal), epoch, 1);
                }
            }
        }
        // ---- reduce-scatter: sum the tiles this rank owns ---------------------------------------------------------
        if (a.mode == GEMM_REDUCE_SCATTER && st->abortFlag == 0) {
            const int et = static_cast<int>(threadIdx.x) - 64;     // 0..127 among the epilogue threads
            const int owned = a.blocksPerShard * a.nBlocks;
            const uint8_t *stage = reg->regions[a.stageHandle].peerBase[rank] + a.stageOffset;
            const uint64_t rowBytes = static_cast<uint64_t>(a.N) * 2;
            for (int tl = cta; tl < owned; tl += nCta) {
                bool got = true;
                if (et < ranks) {
                    const int64_t slot = FLAG_PLANE_B + static_cast<int64_t>(et) * a.flagStride + tl;
                    got = WaitFlagGE(w, FlagSlot(a.comm, rank, slot), 1, et, slot);
                }
                // join the 128 epilogue threads and share the verdict
                __shared__ int sGot;
                if (et == 0) sGot = 1;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!got) sGot = 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (sGot == 0) {
                    st->abortFlag = 1;
                    break;
                }
                const int mLocal = tl / a.nBlocks;
                const int nBlock = tl % a.nBlocks;
                const int rows = min(GEMM_BM, a.shardRows - mLocal * GEMM_BM);
                const int cols = min(GEMM_BN, a.N - nBlock * GEMM_BN);
                const int vecsPerRow = cols / 8;
                // four 16-byte columns per thread and step, all ranks' copies of them fetched before they are summed
                // in rank order: enough loads in flight to run the tail of the kernel at memory speed
                const int total = rows * vecsPerRow;
                for (int i0 = et; i0 < total; i0 += 128 * 4) {
                    float accv[4][8];
                    uint64_t off[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int i = min(i0 + q * 128, total - 1);
                        const int r = i / vecsPerRow;
                        const int v = i % vecsPerRow;
                        off[q] = (static_cast<uint64_t>(mLocal) * GEMM_BM + r) * rowBytes + (static_cast<uint64_t>(nBlock) * GEMM_BN + v * 8) * 2;
                    }
                    for (int s = 0; s < ranks; ++s) {
                        Vec16 x[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) x[q] = ld_vec16_stream(stage + static_cast<uint64_t>(s) * a.shardRows * rowBytes + off[q]);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint32_t wds[4] = {x[q].x, x[q].y, x[q].z, x[q].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float lo, hi;
                                if (bf16) {
                                    lo = __uint_as_float(wds[j] << 16);
                                    hi = __uint_as_float(wds[j] & 0xffff0000u);
                                } else {
                                    const float2 f2 = __half22float2(*reinterpret_cast<const __half2 *>(&wds[j]));
                                    lo = f2.x;
                                    hi = f2.y;
                                }
                                accv[q][2 * j] = s == 0 ? lo : accv[q][2 * j] + lo;
                                accv[q][2 * j + 1] = s == 0 ? hi : accv[q][2 * j + 1] + hi;
                            }
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (i0 + q * 128 < total) {
                            st_vec16(a.c + off[q], Vec16{PackPair(accv[q][0], accv[q][1], bf16), PackPair(accv[q][2], accv[q][3], bf16),
                                                         PackPair(accv[q][4], accv[q][5], bf16), PackPair(accv[q][6], accv[q][7], bf16)});
                        }
                    }
                }
            }
        }
    }

    // ---- tear-down ---------------------------------------------------------------------------------------------
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(TMEM_COLS) : "memory");
    }
    const bool failed = st->abortFlag != 0;
    if (failed && threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, TILEXR_DEV_MBARRIER_TIMEOUT);
    if (fused) {
        if (failed && threadIdx.x == 0 && w.ok()) RaiseFailure(w, TILEXR_DEV_MBARRIER_TIMEOUT, rank, blockIdx.x, 0, 0);
        KernelEpilogue(w, !failed);
    }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1) TileXRGemmTcgen05_single(const __grid_constant__ GemmArgs a) { GemmBody(a); }
// Emulated worlds: one argument block per rank in global memory, rank = blockIdx.y.
__global__ void __launch_bounds__(GEMM_THREADS, 1) TileXRGemmTcgen05_emulated(const GemmArgs *perRank) { GemmBody(perRank[blockIdx.y]); }

} // namespace

const void *GemmKernelSingle() { return reinterpret_cast<const void *>(&TileXRGemmTcgen05_single); }
const void *GemmKernelEmulated() { return reinterpret_cast<const void *>(&TileXRGemmTcgen05_emulated); }

} // namespace TileXR
