// bf16/fp16 GEMM on CTA pairs: tcgen05.mma with cta_group::2.
//
//   C[M,N] = A[M,K] x B[N,K]^T      (both operands K-major, fp32 accumulation, 16-bit output)
//
// Two CTAs of a cluster (one per SM of a pair) work on one 256x256 tile of C.  Each CTA stages its own
// 128 rows of A and HALF of the B tile (128 of its 256 rows) per 64-wide K step, so a K step costs each SM
// 32 KB of shared-memory fill instead of the 48 KB of the one-CTA kernel: the operand stream from L2, which
// bounds that kernel, shrinks by a third, and the ring holds six stages instead of four.  The leader CTA
// (cluster rank 0) issues every tcgen05.mma for the pair; the accumulator of each CTA's 128 rows lives in that
// CTA's own tensor memory, 2 x 256 columns, so epilogue and main loop overlap.
//
// Roles per CTA (256 threads; warps 6-7 only work in the all-gather mode, see below): warp 0 lane 0 issues TMA loads (cp.async.bulk.tensor with cta_group::2 and no
// multicast: both CTAs signal the LEADER's "full" barrier); warp 1 owns tensor memory and, in the leader, issues
// the MMAs and commits them to both CTAs' barriers; warps 2-5 read the accumulator with tcgen05.ld and store C.
// Every mbarrier wait is bounded and checks the pair's abort flags; on a give-up all roles fall through to the
// tear-down, both CTAs meet at the cluster barrier, tensor memory is released and `status` tells the host.
//
// Fused modes: all-gather -> GEMM: warps 6-7 of EVERY CTA write this rank's A shard into the peers' staging buffers
// piece by piece (128 rows x a chunk of K) and raise each piece's flag -- through the NVLink multicast alias of the
// staging buffer where the runtime has one (multimem.st: one store, the switch replicates it), else one store per
// peer -- so no SM is taken from the GEMM (with commBlocks > 0 leading CTA pairs push instead and compute afterwards,
// the earlier scheme); each TMA lane acquires the flag of a remote 128-row piece before loading it from LOCAL staging
// memory; GEMM -> reduce-scatter: every CTA's epilogue stores its 128x256 partial tile into
// the row owner's staging slot and raises the tile's flag, then the epilogue warps sum the tiles this rank owns
// in rank order).  They need shards of a multiple of 256 rows, so that a pair's tile lies within one shard.
//
// The reference has no GEMM of its own (operators ALL_GATHER_MATMUL / MATMUL_REDUCE_SCATTER are named in
// src/include/tilexr_types.h:108-125 without a kernel).
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
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;   // clears the CTA-rank bit of a shared::cluster address: the leader's copy

struct PairState {
    uint64_t full[GEMM_PAIR_STAGES];       // used in the leader: both CTAs' loads of a stage have landed
    uint64_t empty[GEMM_PAIR_STAGES];      // in each CTA: the MMAs that read this stage have finished
    uint64_t tmemFull[2];                  // in each CTA: accumulator buffer complete
    uint64_t tmemEmpty[2];                 // used in the leader: all eight epilogue warps of the pair drained it
    uint32_t tmemBase;
    volatile int abortFlag;
};

__device__ __forceinline__ uint32_t ClusterCtaRank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void ClusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory object in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t MapToCta(uint32_t smemAddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
    return r;
}

__device__ __forceinline__ int LoadRemoteInt(uint32_t clusterAddr)
{
    int v;
    asm volatile("ld.volatile.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(clusterAddr) : "memory");
    return v;
}

__device__ __forceinline__ void ArriveCluster(uint32_t clusterBarAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterBarAddr) : "memory");
}

// TMA load whose completion bytes are counted on the LEADER's barrier (no multicast: each CTA fetches its own box).
__device__ __forceinline__ void TmaLoadPair2D(void *smemDst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(SmemAddr(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(SmemAddr(bar) & PEER_BIT_MASK)
        : "memory");
}

__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major tile written by TMA with 128-byte swizzle (see the one-CTA kernel for the field layout).
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

// kind::f16, D fp32, A/B K-major; M = 256 rows over the pair, N = 256.
__device__ __forceinline__ uint32_t MakeInstrDesc(bool bf16)
{
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(GEMM_BN >> 3) << 17) |
           (static_cast<uint32_t>((2 * GEMM_BM) >> 4) << 24);
}

__device__ __forceinline__ void UmmaPairF16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    const uint32_t zero = 0;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        "}\n"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}

// 8-bit floating point operands: kind::f8f6f4, D fp32, format codes 0 = e4m3, 1 = e5m2, K = 32 per instruction.
__device__ __forceinline__ uint32_t MakeInstrDescFp8(int fp8Format)
{
    const uint32_t fmt = fp8Format == 2 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(GEMM_BN >> 3) << 17) |
           (static_cast<uint32_t>((2 * GEMM_BM) >> 4) << 24);
}

__device__ __forceinline__ void UmmaPairF8(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    const uint32_t zero = 0;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        "}\n"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}

// Arrives on `bar` in BOTH CTAs of the pair once every MMA issued so far has finished.
__device__ __forceinline__ void UmmaCommitPair(uint64_t *bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(SmemAddr(bar)), "h"(mask) : "memory");
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

// Bounded mbarrier wait; gives up when the budget runs out or either CTA of the pair raised its abort flag.
__device__ __forceinline__ bool WaitBar(uint64_t *bar, uint32_t parity, PairState *st, uint32_t peerAbortAddr, uint64_t budgetNs)
{
    if (MbarTryWait(bar, parity)) return true;
    uint64_t deadline = 0;
    uint32_t polls = 0;
    for (;;) {
        if (MbarTryWait(bar, parity)) return true;
        if ((++polls & 127u) == 0) {
            if (st->abortFlag != 0 || LoadRemoteInt(peerAbortAddr) != 0) {
                st->abortFlag = 1;
                return false;
            }
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

__device__ __forceinline__ uint32_t PackPair(float lo, float hi, bool bf16)
{
    if (bf16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&v);
    }
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// Tile t of the pair's walk: 256-row blocks advance fastest inside a group (eight by default), so pairs that run side by
// side share a B tile and the group's A rows stay in L2.
__device__ __forceinline__ void PairTileAt(int t, int mTiles, int nBlocks, int GROUP, int *mTile, int *nBlock)
{
    const int perGroup = GROUP * nBlocks;
    const int group = t / perGroup;
    const int first = group * GROUP;
    const int size = min(GROUP, mTiles - first);
    const int u = t - group * perGroup;
    *mTile = first + u % size;
    *nBlock = u / size;
}

struct PairTile {
    int mTile;      // 256-row block of the whole product
    int nBlock;
    int shard;      // owner / source rank of the rows (fused modes)
    int mLocalPair; // 256-row block inside the shard
    int row0;       // grouped mode: first row of the pair's 256-row block in A and C
    int rowEnd;     // grouped mode: end of the group's rows
    int rowB0;      // grouped mode: first row of the group's weight in B
};

// Grouped mode: where the rows and the 256-row blocks of each group of this launch start (shared memory, behind the barriers).
struct GroupTable {
    int rowStart[GEMM_MAX_GROUPS + 1];
    int blockStart[GEMM_MAX_GROUPS + 1];
};

__device__ __forceinline__ PairTile TileOf(const GemmArgs &a, int t, int mTiles, int rank, int ranks, const GroupTable *gt)
{
    PairTile c;
    if (a.mode == GEMM_GROUPED) {
        PairTileAt(t, mTiles, a.nBlocks, a.rasterGroup, &c.mTile, &c.nBlock);
        int lo = 0, hi = a.groups - 1;           // last group whose first block is at or before mTile (empty groups share a start)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (gt->blockStart[mid] <= c.mTile) lo = mid;
            else hi = mid - 1;
        }
        c.shard = lo;
        c.mLocalPair = c.mTile - gt->blockStart[lo];
        c.row0 = gt->rowStart[lo] + c.mLocalPair * 2 * GEMM_BM;
        c.rowEnd = gt->rowStart[lo + 1];
        c.rowB0 = (a.groupBase + lo) * a.N;
        return c;
    }
    c.row0 = c.rowEnd = c.rowB0 = 0;
    if (a.mode == GEMM_PLAIN) {
        PairTileAt(t, mTiles, a.nBlocks, a.rasterGroup, &c.mTile, &c.nBlock);
        c.shard = 0;
        c.mLocalPair = c.mTile;
    } else {
        const int pairsPerShard = a.blocksPerShard / 2;
        const int perShard = pairsPerShard * a.nBlocks;
        const int i = t / perShard;
        const int u = t - i * perShard;
        c.shard = a.mode == GEMM_ALL_GATHER ? (rank + i) % ranks : (rank + 1 + i) % ranks;
        // inside a shard the same grouped walk as the plain mode: with many row blocks per shard (few ranks) a wave
        // of pairs would otherwise span all of the shard's A rows and little of B, and A would stream from DRAM
        PairTileAt(u, pairsPerShard, a.nBlocks, max(1, a.rasterGroup), &c.mLocalPair, &c.nBlock);
        c.mTile = c.shard * pairsPerShard + c.mLocalPair;
    }
    return c;
}

__device__ void PairBody(const GemmArgs &a)
{
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t *stageBase = smem;
    PairState *st = reinterpret_cast<PairState *>(smem + GEMM_PAIR_STAGES * GEMM_PAIR_STAGE_BYTES);
    GroupTable *gt = reinterpret_cast<GroupTable *>(smem + GEMM_PAIR_STAGES * GEMM_PAIR_STAGE_BYTES + 256);
    static_assert(sizeof(PairState) <= 256 && 256 + sizeof(GroupTable) <= 1024, "barriers and group table share one KB");
    uint8_t *stageC = smem + GEMM_PAIR_STAGES * GEMM_PAIR_STAGE_BYTES + 1024;      // 128 rows x 256 bytes for the epilogue

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ctaRank = ClusterCtaRank();
    const bool leader = ctaRank == 0;
    const bool fused = a.mode == GEMM_ALL_GATHER || a.mode == GEMM_REDUCE_SCATTER;     // the modes with a communicator
    Waiter w;
    bool ok = true;
    int rank = 0, ranks = 1;
    if (fused) {
        // The staging buffers are not double buffered: nobody may write into a peer's staging buffer before that
        // peer finished the previous launch on this communicator.
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

    // ---- all-gather: leading CTAs (whole pairs) first push this rank's shard, then compute the last tiles --------
    const bool commCta = fused && a.mode == GEMM_ALL_GATHER && blockIdx.x < a.commBlocks;
    if (commCta) {
        if (ok) {
            const TileXRRegistry *reg = a.comm->registryPtr;
            const int pieces = a.blocksPerShard * a.kChunks;
            const int64_t items = static_cast<int64_t>(ranks - 1) * pieces;
            const uint64_t rowBytes = static_cast<uint64_t>(a.K) * 2;
            const uint64_t chunkBytes = static_cast<uint64_t>(a.kBlocksPerChunk) * GEMM_BK * 2;
            for (int64_t it = blockIdx.x; it < items; it += a.commBlocks) {
                const int peer = (rank - 1 - static_cast<int>(it / pieces) + 2 * ranks) % ranks;   // rank-1 needs it first
                const int piece = static_cast<int>(it % pieces);
                const int mLocal = piece / a.kChunks;
                const int kc = piece % a.kChunks;
                const uint64_t colOff = kc * chunkBytes;
                const uint64_t n = min(chunkBytes, rowBytes > colOff ? rowBytes - colOff : 0);
                uint8_t *dstBase = reg->regions[a.stageHandle].peerBase[peer] + a.stageOffset +
                                   (static_cast<uint64_t>(rank) * a.shardRows + static_cast<uint64_t>(mLocal) * GEMM_BM) * rowBytes + colOff;
                const uint8_t *srcBase = a.aLocal + static_cast<uint64_t>(mLocal) * GEMM_BM * rowBytes + colOff;
                const int rows = min(GEMM_BM, a.shardRows - mLocal * GEMM_BM);
                // 128 rows x n bytes: every thread keeps eight 16-byte loads in flight before it stores them, so a
                // pushing CTA has 24 KB on the way instead of the few KB of a row-by-row copy
                const int vecsPerRow = static_cast<int>(n / 16);
                const int total = rows * vecsPerRow;
                for (int i0 = static_cast<int>(threadIdx.x); i0 < total; i0 += static_cast<int>(GEMM_PAIR_THREADS) * 8) {
                    Vec16 v[8];
                    uint64_t off[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const int i = min(i0 + q * static_cast<int>(GEMM_PAIR_THREADS), total - 1);
                        off[q] = static_cast<uint64_t>(i / vecsPerRow) * rowBytes + static_cast<uint64_t>(i % vecsPerRow) * 16;
                        v[q] = ld_vec16_stream(srcBase + off[q]);
                    }
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (i0 + q * static_cast<int>(GEMM_PAIR_THREADS) < total) st_vec16(dstBase + off[q], v[q]);
                    }
                }
                __syncthreads();
                if (threadIdx.x == 0) {
                    SetFlag(FlagSlot(a.comm, peer, FLAG_PLANE_A + static_cast<int64_t>(rank) * a.flagStride + piece), epoch, 1);
                }
            }
        }
        __syncthreads();
    }

    const uint32_t peerAbortAddr = MapToCta(SmemAddr(const_cast<int *>(&st->abortFlag)), ctaRank ^ 1u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_PAIR_STAGES; ++s) {
            MbarInit(&st->full[s], 1);        // the leader's TMA lane arms it with the bytes of both CTAs
            MbarInit(&st->empty[s], 1);       // one commit from the leader's MMA lane
        }
        for (int i = 0; i < 2; ++i) {
            MbarInit(&st->tmemFull[i], 1);    // one commit
            MbarInit(&st->tmemEmpty[i], 8);   // four epilogue warps in each of the two CTAs
        }
        st->abortFlag = ok ? 0 : 1;
        MbarInitFence();
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&a.tmapA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&a.tmapB)) : "memory");
        if (a.mode == GEMM_ALL_GATHER) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&a.tmapALocal)) : "memory");
    }
    if (a.mode == GEMM_GROUPED && warp == 2) {
        // rows before this launch's first group, then the running row and block offsets of its groups
        long long before = 0;
        for (int g = lane; g < a.groupBase; g += 32) before += max(0ll, static_cast<long long>(a.groupRows[g]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
        if (lane == 0) {
            int row = static_cast<int>(min(before, static_cast<long long>(a.M)));
            int block = 0;
            for (int g = 0; g < a.groups; ++g) {
                gt->rowStart[g] = row;
                gt->blockStart[g] = block;
                const long long want = max(0ll, static_cast<long long>(a.groupRows[a.groupBase + g]));
                const int rows = static_cast<int>(min(want, static_cast<long long>(a.M - row)));      // never past the buffers
                row += rows;
                block += (rows + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
            }
            gt->rowStart[a.groups] = row;
            gt->blockStart[a.groups] = block;
        }
    }
    __syncthreads();
    if (warp == 1) {
        // the same warp of both CTAs allocates for the pair; the address is the same in both
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&st->tmemBase)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    TcFenceBefore();
    __syncthreads();
    ClusterSync();          // both CTAs' barriers exist before anything arrives on them from the other CTA
    TcFenceAfter();
    const uint32_t tmemBase = st->tmemBase;

    // Tile walk: computing pairs stride over the front of the walk; the pairs that pushed take
    // `commTilesPerPair` tiles each from its end (the shards that arrive last), so their SMs are not lost.
    const int firstCta = (fused && a.mode == GEMM_ALL_GATHER) ? static_cast<int>(a.commBlocks) : 0;
    const int commPairs = firstCta >> 1;
    const int mTiles = a.mode == GEMM_GROUPED ? gt->blockStart[a.groups] : (a.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
    const int allTiles = mTiles * a.nBlocks;
    const int commTiles = min(allTiles, commPairs * static_cast<int>(a.commTilesPerPair));
    int pair, nPairs, totalTiles, tileBase, tileSign;
    if (commCta) {
        pair = static_cast<int>(blockIdx.x) >> 1;
        nPairs = commPairs;
        totalTiles = commTiles;             // walk index u -> tile allTiles - 1 - u
        tileBase = allTiles - 1;
        tileSign = -1;
    } else {
        pair = (static_cast<int>(blockIdx.x) - firstCta) >> 1;
        nPairs = (static_cast<int>(gridDim.x) - firstCta) >> 1;
        totalTiles = allTiles - commTiles;
        tileBase = 0;
        tileSign = 1;
    }
    const bool bf16 = a.isBf16 != 0;
    const bool fp8 = a.fp8Format != 0;
    const int kPerStage = fp8 ? 2 * GEMM_BK : GEMM_BK;      // elements of K in one 128-byte swizzle row

    if (warp == 0) {
        // ---- TMA producer: this CTA's 128 rows of A and its half of the B tile ---------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (int t = pair; t < totalTiles && st->abortFlag == 0; t += nPairs) {
                const PairTile tc = TileOf(a, tileBase + tileSign * t, mTiles, rank, ranks, gt);
                const int mLocal = tc.mLocalPair * 2 + static_cast<int>(ctaRank);        // this CTA's 128-row block in the shard
                const bool remoteA = a.mode == GEMM_ALL_GATHER && tc.shard != rank;
                const CUtensorMap *mapA = (a.mode == GEMM_ALL_GATHER && !remoteA) ? &a.tmapALocal : &a.tmapA;
                // grouped: a block starts wherever its group's rows start; rows past the group's end belong to the
                // next group (or are filled with zeros past the end of A) and are computed but never stored
                const int rowA = a.mode == GEMM_GROUPED ? tc.row0 + static_cast<int>(ctaRank) * GEMM_BM
                                 : (a.mode == GEMM_ALL_GATHER && !remoteA) ? mLocal * GEMM_BM
                                                                           : tc.mTile * 2 * GEMM_BM + static_cast<int>(ctaRank) * GEMM_BM;
                const int rowB = tc.rowB0 + tc.nBlock * GEMM_BN + static_cast<int>(ctaRank) * (GEMM_BN / 2);
                bool broke = false;
                for (int kb = 0; kb < a.kBlocks; ++kb) {
                    if (!WaitBar(&st->empty[stage], phase ^ 1u, st, peerAbortAddr, budgetNs)) {
                        broke = true;
                        break;
                    }
                    if (remoteA && kb % a.kBlocksPerChunk == 0) {
                        const int piece = mLocal * a.kChunks + kb / a.kBlocksPerChunk;
                        const int64_t slot = FLAG_PLANE_A + static_cast<int64_t>(tc.shard) * a.flagStride + piece;
                        if (!WaitFlagGE(w, FlagSlot(a.comm, rank, slot), 1, tc.shard, slot)) {
                            st->abortFlag = 1;
                            broke = true;
                            break;
                        }
                        fence_proxy_async();   // the rows were written by a peer's stores, TMA reads them next
                    }
                    uint8_t *sa = stageBase + stage * GEMM_PAIR_STAGE_BYTES;
                    uint8_t *sb = sa + GEMM_STAGE_A_BYTES;
                    if (leader) MbarExpectTx(&st->full[stage], 2 * GEMM_PAIR_STAGE_BYTES);
                    TmaLoadPair2D(sa, mapA, kb * kPerStage, rowA, &st->full[stage]);
                    TmaLoadPair2D(sb, &a.tmapB, kb * kPerStage, rowB, &st->full[stage]);
                    if (++stage == GEMM_PAIR_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (broke) break;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the leader's lane 0 drives the tensor cores of both SMs ---------------------------------
        if (leader && lane == 0) {
            const uint32_t idesc = fp8 ? MakeInstrDescFp8(a.fp8Format) : MakeInstrDesc(bf16);
            uint32_t stage = 0, phase = 0;
            int iter = 0;
            for (int t = pair; t < totalTiles && st->abortFlag == 0; t += nPairs, ++iter) {
                const int acc = iter & 1;
                const uint32_t accPhase = (iter >> 1) & 1;
                if (!WaitBar(&st->tmemEmpty[acc], accPhase ^ 1u, st, peerAbortAddr, budgetNs)) break;
                TcFenceAfter();
                const uint32_t tmemD = tmemBase + static_cast<uint32_t>(acc) * GEMM_BN;
                bool broke = false;
                for (int kb = 0; kb < a.kBlocks; ++kb) {
                    if (!WaitBar(&st->full[stage], phase, st, peerAbortAddr, budgetNs)) {
                        broke = true;
                        break;
                    }
                    TcFenceAfter();
                    const uint32_t sa = SmemAddr(stageBase + stage * GEMM_PAIR_STAGE_BYTES);
                    const uint64_t descA = MakeSmemDesc(sa);
                    const uint64_t descB = MakeSmemDesc(sa + GEMM_STAGE_A_BYTES);
#pragma unroll
                    for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
                        // each instruction consumes 32 bytes of K (16 16-bit or 32 8-bit elements): +2 in descriptor units
                        if (fp8) {
                            UmmaPairF8(tmemD, descA + static_cast<uint64_t>(k * 2), descB + static_cast<uint64_t>(k * 2), idesc,
                                       (kb | k) != 0 ? 1u : 0u);
                        } else {
                            UmmaPairF16(tmemD, descA + static_cast<uint64_t>(k * 2), descB + static_cast<uint64_t>(k * 2), idesc,
                                        (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    UmmaCommitPair(&st->empty[stage]);    // both CTAs may refill the stage once these MMAs have read it
                    if (++stage == GEMM_PAIR_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (broke) break;
                UmmaCommitPair(&st->tmemFull[acc]);
            }
        }
    } else if (warp >= 6) {
        // ---- warps 6-7: in the all-gather mode (without pushing CTAs) write this rank's shard into every peer's staging buffer ----
        if (fused && a.mode == GEMM_ALL_GATHER && a.commBlocks == 0 && ok && ranks > 1) {
            const int pt = static_cast<int>(threadIdx.x) - 192;          // 0..63
            const TileXRRegistry *reg = a.comm->registryPtr;
            uint8_t *mc = reg->regions[a.stageHandle].mcBase;
            const bool multicast = mc != nullptr;
            const int pieces = a.blocksPerShard * a.kChunks;
            const int items = multicast ? pieces : (ranks - 1) * pieces;
            const uint64_t rowBytes = static_cast<uint64_t>(a.K) * 2;
            const uint64_t chunkBytes = static_cast<uint64_t>(a.kBlocksPerChunk) * GEMM_BK * 2;
            for (int it = blockIdx.x; it < items; it += gridDim.x) {
                const int peer = (rank - 1 - it / pieces + 2 * ranks) % ranks;      // rank-1 needs it first
                const int piece = it % pieces;
                const int mLocal = piece / a.kChunks;
                const int kc = piece % a.kChunks;
                const uint64_t colOff = kc * chunkBytes;
                const uint64_t n = min(chunkBytes, rowBytes > colOff ? rowBytes - colOff : 0);
                uint8_t *dstBase = (multicast ? mc : reg->regions[a.stageHandle].peerBase[peer]) + a.stageOffset +
                                   (static_cast<uint64_t>(rank) * a.shardRows + static_cast<uint64_t>(mLocal) * GEMM_BM) * rowBytes + colOff;
                const uint8_t *srcBase = a.aLocal + static_cast<uint64_t>(mLocal) * GEMM_BM * rowBytes + colOff;
                const int rows = min(GEMM_BM, a.shardRows - mLocal * GEMM_BM);
                const int vecsPerRow = static_cast<int>(n / 16);
                const int total = rows * vecsPerRow;
                for (int i0 = pt; i0 < total; i0 += 64 * 8) {
                    Vec16 v[8];
                    uint64_t off[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const int i = min(i0 + q * 64, total - 1);
                        off[q] = static_cast<uint64_t>(i / vecsPerRow) * rowBytes + static_cast<uint64_t>(i % vecsPerRow) * 16;
                        v[q] = ld_vec16_stream(srcBase + off[q]);
                    }
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (i0 + q * 64 < total) {
                            if (multicast) {
                                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dstBase + off[q]), "r"(v[q].x),
                                             "r"(v[q].y), "r"(v[q].z), "r"(v[q].w) : "memory");
                            } else {
                                st_vec16(dstBase + off[q], v[q]);
                            }
                        }
                    }
                }
                asm volatile("bar.sync 2, 64;" ::: "memory");
                if (pt == 0) {
                    fence_acq_rel_sys();
                    const uint64_t up = MakeFlag(epoch, 1);
                    const int64_t slot = FLAG_PLANE_A + static_cast<int64_t>(rank) * a.flagStride + piece;
                    if (multicast) {
                        for (int r = 0; r < ranks; ++r) {
                            if (r != rank) st_relaxed_sys_u64(FlagSlot(a.comm, r, slot), up);
                        }
                    } else {
                        st_relaxed_sys_u64(FlagSlot(a.comm, peer, slot), up);
                    }
                }
                asm volatile("bar.sync 2, 64;" ::: "memory");
            }
        }
    } else {
        // ---- epilogue: warps 2..5 of each CTA own TMEM lanes 32*(warp%4) .. +31 = 32 of the CTA's 128 rows --------
        // Per tile: TMEM -> registers -> a swizzled 128x128 staging tile in shared memory -> global memory with every
        // warp store covering two whole 256-byte row pieces.  (Storing straight from the TMEM layout, one thread per
        // row, sends 16-byte pieces to 32 different rows per instruction: fine for local memory behind L2, slow
        // when the destination is a peer's staging buffer behind NVLink.)
        const int quad = warp & 3;
        const int et = static_cast<int>(threadIdx.x) - 64;          // 0..127 among the epilogue threads
        const int myRow = quad * 32 + lane;                          // row of this CTA's 128-row sub-tile held by this thread
        const TileXRRegistry *reg = fused ? a.comm->registryPtr : nullptr;
        __shared__ int sEpiGot[4];
        const float outScale = fp8 ? a.alpha : 1.0f;
        int iter = 0;
        for (int t = pair; t < totalTiles; t += nPairs, ++iter) {
            const PairTile tc = TileOf(a, tileBase + tileSign * t, mTiles, rank, ranks, gt);
            const int nBlock = tc.nBlock;
            const int acc = iter & 1;
            const uint32_t accPhase = (iter >> 1) & 1;
            bool got = true;
            if (lane == 0) {
                got = WaitBar(&st->tmemFull[acc], accPhase, st, peerAbortAddr, budgetNs);
                sEpiGot[quad] = got ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");           // the four warps leave the loop together or not at all
            if ((sEpiGot[0] & sEpiGot[1] & sEpiGot[2] & sEpiGot[3]) == 0) break;
            TcFenceAfter();
            // first row of this CTA's sub-tile at its destination, and how many of its 128 rows exist
            const bool swiglu = a.epilogue == GEMM_EPI_SWIGLU && a.mode != GEMM_REDUCE_SCATTER;
            const int outN = swiglu ? a.N / 2 : a.N;                  // columns of C
            const uint64_t outRowBytes = static_cast<uint64_t>(outN) * 2;
            uint8_t *rowBase;
            int rowsValid;
            if (a.mode == GEMM_REDUCE_SCATTER) {
                const int64_t localRow0 = static_cast<int64_t>(tc.mLocalPair) * 2 * GEMM_BM + static_cast<int64_t>(ctaRank) * GEMM_BM;
                rowsValid = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(GEMM_BM), a.shardRows - localRow0)));
                rowBase = reg->regions[a.stageHandle].peerBase[tc.shard] + a.stageOffset +
                          (static_cast<uint64_t>(rank) * a.shardRows + static_cast<uint64_t>(localRow0)) * a.N * 2;
            } else if (a.mode == GEMM_GROUPED) {
                const int row0 = tc.row0 + static_cast<int>(ctaRank) * GEMM_BM;
                rowsValid = max(0, min(GEMM_BM, tc.rowEnd - row0));
                rowBase = a.c + static_cast<uint64_t>(row0) * outRowBytes;
            } else {
                const int64_t row0 = static_cast<int64_t>(tc.mTile) * 2 * GEMM_BM + static_cast<int64_t>(ctaRank) * GEMM_BM;
                rowsValid = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(GEMM_BM), a.M - row0)));
                rowBase = a.c + static_cast<uint64_t>(row0) * outRowBytes;
            }
            const int col0 = nBlock * GEMM_BN;
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {                   // 128 columns of the product at a time
#pragma unroll 1
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t r[32];
                    const uint32_t taddr = tmemBase + (static_cast<uint32_t>(quad * 32) << 16) +
                                           static_cast<uint32_t>(acc * GEMM_BN + pass * 128 + cc * 32);
                    TmemLoad32(taddr, r);
                    TmemLoadWait();
                    if (swiglu) {
                        // 32 columns = 16 (gate, up) pairs -> 16 outputs = two 16-byte chunks of a 128-byte row piece
                        uint32_t packed[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float o[2];
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                const float gate = __uint_as_float(r[4 * j + 2 * q]) * outScale;
                                const float up = __uint_as_float(r[4 * j + 2 * q + 1]) * outScale;
                                o[q] = gate / (1.0f + __expf(-gate)) * up;
                            }
                            packed[j] = PackPair(o[0], o[1], bf16);
                        }
#pragma unroll
                        for (int v = 0; v < 2; ++v) {
                            const int chunk = (cc * 2 + v) ^ (myRow & 7);
                            *reinterpret_cast<uint4 *>(stageC + myRow * 256 + chunk * 16) =
                                make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                        }
                    } else {
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            packed[j] = PackPair(__uint_as_float(r[2 * j]) * outScale, __uint_as_float(r[2 * j + 1]) * outScale, bf16);
                        }
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const int chunk = (cc * 4 + v) ^ (myRow & 15);    // 16-byte chunks of a 256-byte row, XOR-swizzled
                            *reinterpret_cast<uint4 *>(stageC + myRow * 256 + chunk * 16) =
                                make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                        }
                    }
                }
                if (pass == 1) {
                    // the accumulator buffer is read out: the MMA lane may overwrite it with the tile after next
                    TcFenceBefore();
                    __syncwarp();
                    if (lane == 0) ArriveCluster(SmemAddr(&st->tmemEmpty[acc]) & PEER_BIT_MASK);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (swiglu) {
#pragma unroll 4
                    for (int k = 0; k < 8; ++k) {
                        const int idx = et + k * 128;
                        const int rr = idx >> 3;
                        const int ch = idx & 7;
                        const int col = (col0 + pass * 128) / 2 + ch * 8;
                        if (rr < rowsValid && col < outN) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(stageC + rr * 256 + ((ch ^ (rr & 7)) * 16));
                            st_vec16(rowBase + static_cast<uint64_t>(rr) * outRowBytes + static_cast<uint64_t>(col) * 2, Vec16{v.x, v.y, v.z, v.w});
                        }
                    }
                } else {
#pragma unroll 4
                    for (int k = 0; k < 16; ++k) {
                        const int idx = et + k * 128;
                        const int rr = idx >> 4;
                        const int ch = idx & 15;
                        const int col = col0 + pass * 128 + ch * 8;
                        if (rr < rowsValid && col < a.N) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(stageC + rr * 256 + ((ch ^ (rr & 15)) * 16));
                            st_vec16(rowBase + static_cast<uint64_t>(rr) * a.N * 2 + static_cast<uint64_t>(col) * 2, Vec16{v.x, v.y, v.z, v.w});
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");       // the staging tile may be rewritten
            }
            if (a.mode == GEMM_REDUCE_SCATTER) {
                // this CTA's four epilogue warps have stored their rows of its 128x256 tile: announce it to the owner
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int tileLocal = (tc.mLocalPair * 2 + static_cast<int>(ctaRank)) * a.nBlocks + tc.nBlock;
                    SetFlag(FlagSlot(a.comm, tc.shard, FLAG_PLANE_B + static_cast<int64_t>(rank) * a.flagStride + tileLocal), epoch, 1);
                }
            }
        }
        // ---- reduce-scatter: sum the 128x256 tiles this rank owns, in rank order -----------------------------------
        if (a.mode == GEMM_REDUCE_SCATTER && st->abortFlag == 0) {
            const int et = static_cast<int>(threadIdx.x) - 64;     // 0..127 among the epilogue threads
            const int owned = a.blocksPerShard * a.nBlocks;
            const uint8_t *stage = reg->regions[a.stageHandle].peerBase[rank] + a.stageOffset;
            const uint64_t rowBytes = static_cast<uint64_t>(a.N) * 2;
            __shared__ int sGot;
            for (int tl = static_cast<int>(blockIdx.x); tl < owned; tl += static_cast<int>(gridDim.x)) {
                bool got = true;
                if (et < ranks) {
                    const int64_t slot = FLAG_PLANE_B + static_cast<int64_t>(et) * a.flagStride + tl;
                    got = WaitFlagGE(w, FlagSlot(a.comm, rank, slot), 1, et, slot);
                }
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
                asm volatile("bar.sync 1, 128;" ::: "memory");     // sGot is rewritten in the next round
            }
        }
    }

    // ---- tear-down: nobody frees tensor memory while the other CTA's MMAs or loads may still target it -------------
    TcFenceBefore();
    __syncthreads();
    ClusterSync();
    TcFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(TMEM_COLS) : "memory");
    }
    const bool failed = st->abortFlag != 0;
    if (failed && threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, TILEXR_DEV_MBARRIER_TIMEOUT);
    if (fused) {
        if (failed && threadIdx.x == 0 && w.ok()) RaiseFailure(w, TILEXR_DEV_MBARRIER_TIMEOUT, rank, blockIdx.x, 0, 0);
        KernelEpilogue(w, !failed);
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_PAIR_THREADS, 1)
TileXRGemmTcgen05Pair_single(const __grid_constant__ GemmArgs a) { PairBody(a); }
// Emulated worlds: one argument block per rank in global memory, rank = blockIdx.y.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_PAIR_THREADS, 1)
TileXRGemmTcgen05Pair_emulated(const GemmArgs *perRank) { PairBody(perRank[blockIdx.y]); }

} // namespace

const void *GemmPairKernel() { return reinterpret_cast<const void *>(&TileXRGemmTcgen05Pair_single); }
const void *GemmPairKernelEmulated() { return reinterpret_cast<const void *>(&TileXRGemmTcgen05Pair_emulated); }

} // namespace TileXR
