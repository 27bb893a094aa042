// Block-scaled fp8 GEMM on CTA pairs (tcgen05.mma cta_group::2, kind::f8f6f4) with fp32 scales:
//
//   C[m, n] = sum over 128-wide blocks kb of  sA[m, kb] * sB[n / 128, kb] * sum_{k in kb} A[m, k] * B[n, k]
//
// A is [M, K] e4m3 with one fp32 scale per row and 128 elements of K (what the expert-parallel dispatch delivers:
// csrc/ep/ep_kernels.cu, quantisation 1 x 128), B is [N, K] e4m3 with one fp32 scale per 128 x 128 block (the usual
// weight layout beside it), C is bf16 or fp16.  fp32 scales cannot ride inside the tensor-core instruction (its
// block-scaled kinds take power-of-two E8M0 factors per 32 elements), so the sum over K is formed in two levels:
// the tensor cores produce the exact fp32 partial product of ONE 128-wide block of K into a scratch accumulator in
// tensor memory, and CUDA cores fold it into register accumulators with the block's two scales, while the tensor
// cores already work on the next block.  A stage of the TMA ring is exactly one block of K (128 bytes per row),
// so the main loop alternates two scratch accumulators:
//
//   tensor memory   4 x 128 columns: scratch (p, h) receives, for blocks of K of parity p, the 128 columns
//                   {h*64..h*64+63} u {128+h*64..128+h*64+63} of the pair's 256 x 256 tile (with cta_group::2 each
//                   CTA supplies half of B's rows); two blocks of K are in flight for each half;
//   warp 0          TMA producer (this CTA's 128 rows of A and 128 rows of B per block of K, no multicast);
//   warp 1          tensor-memory owner; in the leader CTA it issues two N = 128 instructions groups per block of K;
//   warps 2-3       idle: they complete the first warpgroup, which hands most of its registers to the others
//                   (setmaxnreg), because the promoters keep a quarter of the tile each in registers;
//   warps 4-7, 8-11 promoters of the two column halves: tcgen05.ld, scale, fused multiply-add into 128 fp32
//                   registers per thread (one row of the CTA's 128, 128 columns), release the scratch buffer;
//                   at the end of a tile they round to the output type and store through a swizzled staging tile.
//
// Fused with the collectives of a tensor-parallel layer (mode of GemmBlockArgs):
//
//   all-gather -> GEMM    warps 2-3 of EVERY CTA, idle otherwise, write this rank's shard of A (fp8 rows and their
//                   scales) into all ranks' staging buffers, 128 rows at a time, and raise the piece's flag: through
//                   the NVLink multicast alias of the staging buffer where the runtime has one (multimem.st: one
//                   store, the switch replicates it), else with one store per peer.  No SM is set aside for
//                   communication.  The TMA lane of a CTA acquires the flag of its 128 rows before the first load of a
//                   tile (TMA then reads LOCAL memory, without multicast); each promoter warp acquires it before it
//                   reads the rows' scales.  Every rank walks the shards starting with its own.
//   GEMM -> reduce-scatter    the promoters store their 128 x 256 partial tile into the row owner's staging slot and
//                   raise the tile's flag; when a CTA has run out of tiles its promoters add, in rank order, the
//                   R partial tiles of the output tiles it owns.  Every rank starts with the rows of the next rank
//                   and ends with its own.
//
// Every mbarrier wait is bounded; on a give-up all roles fall through to the tear-down, tensor memory is released
// and `status` tells the host.  The numerics reference is the fp32 product of the dequantised operands
// (reference numerics of the block scales: src/ep/kernels/tilexr_ep_mxfp8_quant.h:36-168 for the exponent form,
// tests/ep/demo for the 1 x 128 form).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "gemm_kernels.cuh"
#include "tilexr_types.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr uint32_t FB_TMEM_COLS = 512;
constexpr int FB_SCRATCH = 4;               // scratch accumulators: two blocks of K in flight for each half of the tile
constexpr uint32_t FB_PEER_BIT_MASK = 0xFEFFFFFFu;
constexpr int FB_HALF_N = GEMM_BN / 2;       // columns of one scratch accumulator
constexpr int FB_MAX_KB = 256;               // blocks of K whose weight scales fit the shared-memory copy (K up to 32768)
constexpr int FB_FLAG_PLANE_A = TILEXR_FLAG_DATA_BASE;    // all-gather: piece (source rank, 128-row block) has landed
constexpr int FB_FLAG_PLANE_B = TILEXR_FLAG_ACK_BASE;     // reduce-scatter: partial tile (source rank, tile) has landed

__device__ __forceinline__ void FbMultimemSt(uint8_t *p, const Vec16 &v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// `bytes` (a multiple of 16) from local memory to `dst`, four vectors per thread in flight (the pushing warps live on the 88 registers of the first warpgroup); `multicast` stores through
// an NVLink multicast address (every rank's copy at once).
__device__ __forceinline__ void FbPush(uint8_t *dst, const uint8_t *src, uint64_t bytes, int lane, int lanes, bool multicast)
{
    const uint64_t vecs = bytes / 16;
    for (uint64_t i = lane; i < vecs; i += 4ull * lanes) {
        Vec16 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint64_t k = i + static_cast<uint64_t>(u) * lanes;
            if (k < vecs) q[u] = ld_vec16_stream(src + k * 16);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint64_t k = i + static_cast<uint64_t>(u) * lanes;
            if (k < vecs) {
                if (multicast) FbMultimemSt(dst + k * 16, q[u]);
                else st_vec16(dst + k * 16, q[u]);
            }
        }
    }
}


struct BlockState {
    uint64_t full[GEMM_FP8_BLOCK_STAGES];       // leader: both CTAs' loads of a stage have landed
    uint64_t empty[GEMM_FP8_BLOCK_STAGES];      // each CTA: the MMAs that read this stage have finished
    uint64_t scratchFull[FB_SCRATCH];      // each CTA: scratch s holds the product of one block of K
    uint64_t scratchEmpty[FB_SCRATCH];     // leader: the eight promoter warps of scratch s (four per CTA) have read it
    uint32_t tmemBase;
    volatile int abortFlag;
    uint32_t epoch;                        // fused modes: the epoch of this launch (kept here, not in every thread's registers)
};

__device__ __forceinline__ uint32_t FbCtaRank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void FbClusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t FbMapToCta(uint32_t smemAddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
    return r;
}
__device__ __forceinline__ int FbLoadRemoteInt(uint32_t clusterAddr)
{
    int v;
    asm volatile("ld.volatile.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(clusterAddr) : "memory");
    return v;
}
__device__ __forceinline__ void FbArriveCluster(uint32_t clusterBarAddr)
{
    // Default semantics (release at CTA scope): what the arrive has to order are this warp's tensor-memory reads, which
    // tcgen05.wait::ld and tcgen05.fence::before_thread_sync have completed; a cluster-scope release would add a
    // memory barrier to every block of K.
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(clusterBarAddr) : "memory");
}
__device__ __forceinline__ void FbTmaLoad(void *smemDst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(SmemAddr(smemDst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(SmemAddr(bar) & FB_PEER_BIT_MASK)
        : "memory");
}
__device__ __forceinline__ void FbFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void FbFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile written by TMA with 128-byte swizzle: rows 128 bytes apart, groups of eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t FbSmemDesc(uint32_t smemAddr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smemAddr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// kind::f8f6f4, D fp32, A and B K-major, M = 256 rows over the pair, N = 128.
__device__ __forceinline__ uint32_t FbInstrDesc(int fp8Format)
{
    const uint32_t fmt = fp8Format == 2 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(FB_HALF_N >> 3) << 17) |
           (static_cast<uint32_t>((2 * GEMM_BM) >> 4) << 24);
}

__device__ __forceinline__ void FbUmma(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
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

// Arrives on `bar` in BOTH CTAs of the pair once every MMA issued so far has finished (an mbarrier arrive, not a load).
__device__ __forceinline__ void FbCommitPair(uint64_t *bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(SmemAddr(bar)), "h"(mask) : "memory");
}

__device__ __forceinline__ void FbTmemLoad32(uint32_t taddr, uint32_t *r)
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
__device__ __forceinline__ void FbTmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ bool FbWaitBar(uint64_t *bar, uint32_t parity, BlockState *st, uint32_t peerAbortAddr, uint64_t budgetNs)
{
    if (MbarTryWait(bar, parity)) return true;
    uint64_t deadline = 0;
    uint32_t polls = 0;
    for (;;) {
        if (MbarTryWait(bar, parity)) return true;
        if ((++polls & 127u) == 0) {
            if (st->abortFlag != 0 || FbLoadRemoteInt(peerAbortAddr) != 0) {
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

// Bounded acquire of a flag by one thread that has no Waiter of its own (the promoters are short of registers).
__device__ __forceinline__ bool FbAcquireFlag(const uint64_t *flag, uint64_t want, BlockState *st, uint64_t budgetNs)
{
    uint64_t deadline = 0;
    uint32_t polls = 0;
    while (ld_acquire_sys_u64(flag) < want) {
        if ((++polls & 63u) == 0) {
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
    return true;
}

__device__ __forceinline__ uint32_t FbPackPair(float lo, float hi, bool bf16)
{
    if (bf16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&v);
    }
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// The grouped tile walk of the bf16 CTA-pair kernel: 256-row blocks advance fastest inside a group.
__device__ __forceinline__ void FbTileAt(int t, int mTiles, int nBlocks, int GROUP, int *mTile, int *nBlock)
{
    const int perGroup = GROUP * nBlocks;
    const int group = t / perGroup;
    const int first = group * GROUP;
    const int size = min(GROUP, mTiles - first);
    const int u = t - group * perGroup;
    *mTile = first + u % size;
    *nBlock = u / size;
}

// Tile t of this pair's walk.  In the fused modes the 256-row blocks are rotated so that every rank starts with its own
// shard (all-gather: its rows are there first) or with the next rank's (reduce-scatter: its own rows come last, when the
// peers' partial tiles have had time to arrive).
__device__ __forceinline__ void FbTileOf(const GemmBlockArgs &a, int t, int mTiles, int rank, int *mTile, int *nBlock)
{
    FbTileAt(t, mTiles, a.nBlocks, a.rasterGroup, mTile, nBlock);
    if (a.mode != GEMM_PLAIN) {
        const int pairsPerShard = a.blocksPerShard / 2;
        const int first = (a.mode == GEMM_ALL_GATHER ? rank : rank + 1) * pairsPerShard;
        *mTile = (*mTile + first) % mTiles;
    }
}

// Twelve warps start with 168 registers each (the most a block of this size can have); the first warpgroup then
// shrinks to 88 and the two promoter warpgroups grow to 200, so that 128 accumulators and two 32-register
// tensor-memory reads fit without spilling.
__device__ __forceinline__ void FbBody(const GemmBlockArgs &a)
{
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t *stageBase = smem;
    BlockState *st = reinterpret_cast<BlockState *>(smem + GEMM_FP8_BLOCK_STAGES * GEMM_PAIR_STAGE_BYTES);
    uint8_t *stageC = smem + GEMM_FP8_BLOCK_STAGES * GEMM_PAIR_STAGE_BYTES + 1024;      // 128 rows x 256 bytes

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ctaRank = FbCtaRank();
    const bool leader = ctaRank == 0;
    const bool fused = a.mode != GEMM_PLAIN;
    const uint32_t peerAbortAddr = FbMapToCta(SmemAddr(const_cast<int *>(&st->abortFlag)), ctaRank ^ 1u);

    // The promoters have no register to spare for values that only the prologue, the TMA lane and the epilogue need: the
    // launch's epoch lives in shared memory, and rank, rank count and the wait budget are read where they are used.
    bool ok = true;
    if (fused) {
        // The staging buffers are not double buffered: nobody writes into a peer's before that peer has finished the
        // previous launch on this communicator.
        Waiter w = MakeWaiter(a.comm, a.magic, blockIdx.x);
        const int rank = a.comm->rank;
        const int ranks = a.comm->rankSize;
        if (threadIdx.x == 0) st->epoch = w.epoch;
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

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_FP8_BLOCK_STAGES; ++s) {
            MbarInit(&st->full[s], 1);
            MbarInit(&st->empty[s], 1);
        }
        for (int h = 0; h < FB_SCRATCH; ++h) {
            MbarInit(&st->scratchFull[h], 1);     // one commit
            MbarInit(&st->scratchEmpty[h], 8);    // four promoter warps in each of the two CTAs
        }
        st->abortFlag = ok ? 0 : 1;
        MbarInitFence();
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&a.tmapA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&a.tmapB)) : "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&st->tmemBase)), "r"(FB_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    FbFenceBefore();
    __syncthreads();
    FbClusterSync();
    FbFenceAfter();
    const uint32_t tmemBase = st->tmemBase;

    const int mTiles = (a.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
    const int totalTiles = mTiles * a.nBlocks;
    const int pair = static_cast<int>(blockIdx.x) >> 1;
    const int nPairs = static_cast<int>(gridDim.x) >> 1;
    const bool bf16 = a.isBf16 != 0;

    if (warp < 4) {
    // the first warpgroup gives registers away (all four warps execute this together) and then splits into its roles
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;" ::: "memory");
    if (warp == 0) {
        // ---- TMA producer -----------------------------------------------------------------------------------------
        if (lane == 0) {
            const uint64_t budgetNs = fused ? a.comm->waitTimeoutNs : 4000000000ull;
            const int rank = fused ? a.comm->rank : 0;
            Waiter w{fused ? a.comm : nullptr, st->epoch, static_cast<int32_t>(blockIdx.x), TILEXR_DEV_OK, 0};
            uint32_t stage = 0, phase = 0;
            for (int t = pair; t < totalTiles && st->abortFlag == 0; t += nPairs) {
                int mTile, nBlock;
                FbTileOf(a, t, mTiles, rank, &mTile, &nBlock);
                const int rowA = mTile * 2 * GEMM_BM + static_cast<int>(ctaRank) * GEMM_BM;
                const int rowB = nBlock * GEMM_BN + static_cast<int>(ctaRank) * (GEMM_BN / 2);
                if (a.mode == GEMM_ALL_GATHER) {
                    // this CTA's 128 rows of the gathered A: wait until their owner has written them here
                    const int block = rowA / GEMM_BM;
                    const int shard = block / a.blocksPerShard;
                    const int64_t slot = FB_FLAG_PLANE_A + static_cast<int64_t>(shard) * a.flagStride + (block - shard * a.blocksPerShard);
                    if (!WaitFlagGE(w, FlagSlot(a.comm, rank, slot), 1, shard, slot)) {
                        st->abortFlag = 1;
                        break;
                    }
                    fence_proxy_async();       // the rows were written by generic-proxy stores, TMA reads them next
                }
                bool broke = false;
                for (int kb = 0; kb < a.kBlocks; ++kb) {
                    if (!FbWaitBar(&st->empty[stage], phase ^ 1u, st, peerAbortAddr, budgetNs)) {
                        broke = true;
                        break;
                    }
                    uint8_t *sa = stageBase + stage * GEMM_PAIR_STAGE_BYTES;
                    uint8_t *sb = sa + GEMM_STAGE_A_BYTES;
                    if (leader) MbarExpectTx(&st->full[stage], 2 * GEMM_PAIR_STAGE_BYTES);
                    FbTmaLoad(sa, &a.tmapA, kb * 128, rowA, &st->full[stage]);       // x in bytes = elements: a multiple of 128
                    FbTmaLoad(sb, &a.tmapB, kb * 128, rowB, &st->full[stage]);
                    if (++stage == GEMM_FP8_BLOCK_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (broke) break;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: per block of K, one N = 128 group into each scratch accumulator ----------------------------
        if (leader && lane == 0) {
            const uint64_t budgetNs = fused ? a.comm->waitTimeoutNs : 4000000000ull;
            const uint32_t idesc = FbInstrDesc(a.fp8Format);
            uint32_t stage = 0, phase = 0;
            uint32_t sPhase = 0;                   // bit s: parity of the next wait on scratchEmpty[s]
            int kbAll = 0;                         // blocks of K issued so far, over all tiles: scratch buffers alternate with it
            for (int t = pair; t < totalTiles && st->abortFlag == 0; t += nPairs) {
                bool broke = false;
                for (int kb = 0; kb < a.kBlocks && !broke; ++kb, ++kbAll) {
                    if (!FbWaitBar(&st->full[stage], phase, st, peerAbortAddr, budgetNs)) {
                        broke = true;
                        break;
                    }
                    const uint32_t sa = SmemAddr(stageBase + stage * GEMM_PAIR_STAGE_BYTES);
                    const uint64_t descA = FbSmemDesc(sa);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int sIdx = (kbAll & 1) * 2 + h;
                        if (!FbWaitBar(&st->scratchEmpty[sIdx], ((sPhase >> sIdx) & 1u) ^ 1u, st, peerAbortAddr, budgetNs)) {
                            broke = true;
                            break;
                        }
                        sPhase ^= 1u << sIdx;
                        FbFenceAfter();
                        // rows h*64 .. h*64+63 of this CTA's 128 rows of B (and the same rows of the other CTA's half)
                        const uint64_t descB = FbSmemDesc(sa + GEMM_STAGE_A_BYTES + static_cast<uint32_t>(h) * 64u * 128u);
                        const uint32_t tmemD = tmemBase + static_cast<uint32_t>(sIdx) * FB_HALF_N;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {       // 32 elements of K (32 bytes) per instruction: +2 descriptor units
                            FbUmma(tmemD, descA + static_cast<uint64_t>(k * 2), descB + static_cast<uint64_t>(k * 2), idesc, k != 0 ? 1u : 0u);
                        }
                        FbCommitPair(&st->scratchFull[sIdx]);
                    }
                    if (broke) break;
                    FbCommitPair(&st->empty[stage]);
                    if (++stage == GEMM_FP8_BLOCK_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (broke) break;
            }
        }
    } else if (a.mode == GEMM_ALL_GATHER && ok) {
        // ---- warps 2-3: write this rank's shard, rows and scales, into every rank's staging buffers -------------------
        const int pt2 = static_cast<int>(threadIdx.x) - 64;           // 0..63
        const int rank = a.comm->rank, ranks = a.comm->rankSize;
        const uint32_t epoch = st->epoch;
        const TileXRRegistry *reg = a.comm->registryPtr;
        uint8_t *mcRows = reg->regions[a.aHandle].mcBase;
        uint8_t *mcScales = reg->regions[a.sHandle].mcBase;
        const bool multicast = ranks > 1 && mcRows != nullptr && mcScales != nullptr;
        const int pieces = a.blocksPerShard;
        const int items = multicast ? pieces : ranks * pieces;
        const uint64_t rowBytes = static_cast<uint64_t>(a.K);
        const uint64_t scaleRowBytes = static_cast<uint64_t>(a.kBlocks) * 4;
        for (int it = blockIdx.x; it < items; it += gridDim.x) {
            const int piece = it % pieces;
            const int peer = (rank - it / pieces + ranks) % ranks;          // itself first, then rank-1 (which needs it next), ...
            const uint64_t srcRow = static_cast<uint64_t>(piece) * GEMM_BM;
            const uint64_t dstRow = static_cast<uint64_t>(rank) * a.shardRows + srcRow;
            uint8_t *rowsTo = (multicast ? mcRows : reg->regions[a.aHandle].peerBase[peer]) + a.aOffset + dstRow * rowBytes;
            uint8_t *scalesTo = (multicast ? mcScales : reg->regions[a.sHandle].peerBase[peer]) + a.sOffset + dstRow * scaleRowBytes;
            FbPush(rowsTo, a.aLocal + srcRow * rowBytes, GEMM_BM * rowBytes, pt2, 64, multicast);
            FbPush(scalesTo, reinterpret_cast<const uint8_t *>(a.scaleALocal) + srcRow * scaleRowBytes, GEMM_BM * scaleRowBytes, pt2, 64, multicast);
            asm volatile("bar.sync 2, 64;" ::: "memory");
            if (pt2 == 0) {
                fence_acq_rel_sys();
                const uint64_t up = MakeFlag(epoch, 1);
                const int64_t slot = FB_FLAG_PLANE_A + static_cast<int64_t>(rank) * a.flagStride + piece;
                if (multicast) {
                    for (int r = 0; r < ranks; ++r) st_relaxed_sys_u64(FlagSlot(a.comm, r, slot), up);
                } else {
                    st_relaxed_sys_u64(FlagSlot(a.comm, peer, slot), up);
                }
            }
            asm volatile("bar.sync 2, 64;" ::: "memory");
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;" ::: "memory");
        // ---- promoters: warps 4-7 own column half 0, warps 8-11 half 1; TMEM lanes 32 * (warp % 4) .. + 31 --------------
        const int quad = warp & 3;
        const int h = (warp - 4) >> 2;
        const int myRow = quad * 32 + lane;                       // row of this CTA's 128-row sub-tile
        const int pt = static_cast<int>(threadIdx.x) - 128;       // 0..255 among the promoter threads
        __shared__ int sGot[8];
        __shared__ int sExit;
        __shared__ float sScaleB[2 * FB_MAX_KB];
        uint32_t fPhase = 0;                       // bit p: parity of the next wait on this half's scratch buffer p
        int kbAll = 0;
        const int KB = a.kBlocks;
        const bool vec4 = (KB & 3) == 0;           // rows of the scale tables are 16-byte aligned: four blocks per load
        const bool gathered = a.mode == GEMM_ALL_GATHER;
        const uint64_t budgetNs = fused ? a.comm->waitTimeoutNs : 4000000000ull;
        for (int t = pair; t < totalTiles; t += nPairs) {
            int mTile, nBlock;
            FbTileOf(a, t, mTiles, fused ? a.comm->rank : 0, &mTile, &nBlock);
            const int64_t row0 = static_cast<int64_t>(mTile) * 2 * GEMM_BM + static_cast<int64_t>(ctaRank) * GEMM_BM;
            const int64_t gRow = row0 + myRow;
            const bool rowValid = gRow < a.M;
            const float *saRow = a.scaleA + (rowValid ? gRow : 0) * KB;
            // scale blocks of B for the two 64-column groups of this scratch accumulator
            const int nb0 = min(nBlock * 2, a.scaleBRows - 1);
            const int nb1 = min(nBlock * 2 + 1, a.scaleBRows - 1);
            const float *sb0 = a.scaleB + static_cast<int64_t>(nb0) * KB;
            const float *sb1 = a.scaleB + static_cast<int64_t>(nb1) * KB;
            float acc[FB_HALF_N];
#pragma unroll
            for (int j = 0; j < FB_HALF_N; ++j) acc[j] = 0.f;
            // The weight's scales of this tile (two rows of the table) go to shared memory once per tile; the activation
            // scales of the thread's row travel four blocks of K at a time and one group ahead of their use, so that
            // their latency (an L2 round trip, longer than one block's work) never shows.
            asm volatile("bar.sync 1, 256;" ::: "memory");          // the previous tile's readers are done with sScaleB
            for (int i = pt; i < 2 * KB && i < 2 * FB_MAX_KB; i += 256) {
                sScaleB[i] = __ldg((i < KB ? sb0 + i : sb1 + (i - KB)));
            }
            if (gathered) {
                // the scales of these 128 rows were written by their owner during this launch: acquire the rows' flag first
                if (lane == 0) {
                    const int block = static_cast<int>(row0 / GEMM_BM);
                    const int shard = block / a.blocksPerShard;
                    const int64_t slot = FB_FLAG_PLANE_A + static_cast<int64_t>(shard) * a.flagStride + (block - shard * a.blocksPerShard);
                    FbAcquireFlag(FlagSlot(a.comm, a.comm->rank, slot), MakeFlag(st->epoch, 1), st, budgetNs);
                }
                __syncwarp();
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const bool bInSmem = KB <= FB_MAX_KB;
            float4 curA = make_float4(0.f, 0.f, 0.f, 0.f), nxtA = curA;
            auto loadGroup = [&](int kb0, float4 &ga) {
                if (!rowValid) {
                    ga = make_float4(0.f, 0.f, 0.f, 0.f);
                } else if (gathered) {
                    // written during this launch: through L2, never through the read-only path
                    if (vec4) {
                        ga = __ldcg(reinterpret_cast<const float4 *>(saRow + kb0));
                    } else {
                        ga = make_float4(__ldcg(saRow + min(kb0, KB - 1)), __ldcg(saRow + min(kb0 + 1, KB - 1)), __ldcg(saRow + min(kb0 + 2, KB - 1)),
                                         __ldcg(saRow + min(kb0 + 3, KB - 1)));
                    }
                } else if (vec4) {
                    ga = __ldg(reinterpret_cast<const float4 *>(saRow + kb0));
                } else {
                    ga = make_float4(__ldg(saRow + min(kb0, KB - 1)), __ldg(saRow + min(kb0 + 1, KB - 1)), __ldg(saRow + min(kb0 + 2, KB - 1)),
                                     __ldg(saRow + min(kb0 + 3, KB - 1)));
                }
            };
            loadGroup(0, curA);
            bool alive = true;
            for (int kb = 0; kb < KB; ++kb) {
                const int q = kb & 3;
                if (q == 0 && kb + 4 < KB) loadGroup(kb + 4, nxtA);
                const float saq = q == 0 ? curA.x : q == 1 ? curA.y : q == 2 ? curA.z : curA.w;
                const int p = kbAll & 1;
                const int sIdx = p * 2 + h;
                ++kbAll;
                bool got = true;
                if (lane == 0) {
                    got = FbWaitBar(&st->scratchFull[sIdx], (fPhase >> p) & 1u, st, peerAbortAddr, budgetNs);
                    sGot[warp - 4] = got ? 1 : 0;
                }
                __syncwarp();
                if (sGot[warp - 4] == 0) {
                    alive = false;
                    break;
                }
                __syncwarp();
                fPhase ^= 1u << p;
                FbFenceAfter();
                const float f0 = saq * (bInSmem ? sScaleB[kb] : __ldg(sb0 + kb));
                const float f1 = saq * (bInSmem ? sScaleB[KB + kb] : __ldg(sb1 + kb));
#pragma unroll
                for (int cc = 0; cc < 4; cc += 2) {
                    uint32_t r0[32], r1[32];
                    const uint32_t taddr = tmemBase + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(sIdx * FB_HALF_N + cc * 32);
                    FbTmemLoad32(taddr, r0);
                    FbTmemLoad32(taddr + 32, r1);
                    FbTmemLoadWait();
                    const float f = cc < 2 ? f0 : f1;
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[cc * 32 + j] = fmaf(__uint_as_float(r0[j]), f, acc[cc * 32 + j]);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[(cc + 1) * 32 + j] = fmaf(__uint_as_float(r1[j]), f, acc[(cc + 1) * 32 + j]);
                }
                // the scratch accumulator is read out: the MMA lane may overwrite it two blocks of K from now
                FbFenceBefore();
                __syncwarp();
                if (lane == 0) FbArriveCluster(SmemAddr(&st->scratchEmpty[sIdx]) & FB_PEER_BIT_MASK);
                if (q == 3) curA = nxtA;
            }
            // All eight promoter warps of the CTA arrive here whether or not their waits succeeded, and leave the tile
            // loop together: the store below uses block-wide barriers, which a lone warp must never reach.
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (pt == 0) sExit = (st->abortFlag != 0) ? 1 : 0;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (sExit != 0) break;
            (void)alive;
            // ---- store the tile: the two groups take turns with the staging tile, everybody stores ---------------------
            int rowsValid = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(GEMM_BM), a.M - row0)));
            uint8_t *rowBase = a.c + static_cast<uint64_t>(row0) * a.N * 2;
            int owner = 0, tileLocal = 0;
            if (a.mode == GEMM_REDUCE_SCATTER) {
                // the partial tile goes into the row owner's staging slot for this rank
                const int block = static_cast<int>(row0 / GEMM_BM);
                owner = block / a.blocksPerShard;
                const int localBlock = block - owner * a.blocksPerShard;
                tileLocal = localBlock * a.nBlocks + nBlock;
                rowBase = a.comm->registryPtr->regions[a.outHandle].peerBase[owner] + a.outOffset +
                          (static_cast<uint64_t>(a.comm->rank) * a.shardRows + static_cast<uint64_t>(localBlock) * GEMM_BM) * a.N * 2;
                rowsValid = GEMM_BM;
            }
            const int col0 = nBlock * GEMM_BN;
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {
                if (h == pass) {
#pragma unroll
                    for (int v = 0; v < 16; ++v) {
                        const int chunk = v ^ (myRow & 15);           // 16-byte chunks of a 256-byte row, XOR-swizzled
                        *reinterpret_cast<uint4 *>(stageC + myRow * 256 + chunk * 16) =
                            make_uint4(FbPackPair(acc[8 * v], acc[8 * v + 1], bf16), FbPackPair(acc[8 * v + 2], acc[8 * v + 3], bf16),
                                       FbPackPair(acc[8 * v + 4], acc[8 * v + 5], bf16), FbPackPair(acc[8 * v + 6], acc[8 * v + 7], bf16));
                    }
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
#pragma unroll 2
                for (int k = 0; k < 8; ++k) {
                    const int idx = pt + k * 256;
                    const int rr = idx >> 4;
                    const int ch = idx & 15;
                    // chunk ch of scratch `pass`: columns pass*64 + ch*8 (first group) or 128 + pass*64 + (ch-8)*8
                    const int col = col0 + (ch < 8 ? pass * 64 + ch * 8 : 128 + pass * 64 + (ch - 8) * 8);
                    if (rr < rowsValid && col < a.N) {
                        const uint4 v = *reinterpret_cast<const uint4 *>(stageC + rr * 256 + ((ch ^ (rr & 15)) * 16));
                        st_vec16(rowBase + static_cast<uint64_t>(rr) * a.N * 2 + static_cast<uint64_t>(col) * 2, Vec16{v.x, v.y, v.z, v.w});
                    }
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
            }
            if (a.mode == GEMM_REDUCE_SCATTER && pt == 0) {
                // all 256 promoter threads have stored (the barrier above): order their stores, then tell the owner
                fence_acq_rel_sys();
                st_relaxed_sys_u64(FlagSlot(a.comm, owner, FB_FLAG_PLANE_B + static_cast<int64_t>(a.comm->rank) * a.flagStride + tileLocal),
                                   MakeFlag(st->epoch, 1));
            }
        }
        // ---- reduce-scatter: add the partial tiles of the output tiles this CTA owns, in rank order ---------------------
        if (a.mode == GEMM_REDUCE_SCATTER) {
            const int owned = a.blocksPerShard * a.nBlocks;
            const int rank = a.comm->rank, ranks = a.comm->rankSize;
            const uint32_t epoch = st->epoch;
            const uint8_t *stage = a.comm->registryPtr->regions[a.outHandle].peerBase[rank] + a.outOffset;
            const uint64_t rowBytes = static_cast<uint64_t>(a.N) * 2;
            for (int tl = static_cast<int>(blockIdx.x); tl < owned; tl += static_cast<int>(gridDim.x)) {
                asm volatile("bar.sync 1, 256;" ::: "memory");          // sExit of the previous round has been read
                if (pt == 0) sExit = (st->abortFlag != 0) ? 1 : 0;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (sExit != 0) break;
                if (pt < ranks) {
                    const int64_t slot = FB_FLAG_PLANE_B + static_cast<int64_t>(pt) * a.flagStride + tl;
                    FbAcquireFlag(FlagSlot(a.comm, rank, slot), MakeFlag(epoch, 1), st, budgetNs);
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (st->abortFlag != 0) continue;                       // uniform after the barrier: the next round leaves
                const int mLocal = tl / a.nBlocks;
                const int nBlock = tl % a.nBlocks;
                const int cols = min(GEMM_BN, a.N - nBlock * GEMM_BN);
                const int vecsPerRow = cols / 8;
                const int total = GEMM_BM * vecsPerRow;
                for (int i0 = pt; i0 < total; i0 += 256 * 2) {
                    float accv[2][8];
                    uint64_t off[2];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const int i = min(i0 + q * 256, total - 1);
                        off[q] = (static_cast<uint64_t>(mLocal) * GEMM_BM + i / vecsPerRow) * rowBytes +
                                 (static_cast<uint64_t>(nBlock) * GEMM_BN + (i % vecsPerRow) * 8) * 2;
                    }
                    for (int s = 0; s < ranks; ++s) {
                        Vec16 x[2];
#pragma unroll
                        for (int q = 0; q < 2; ++q) x[q] = ld_vec16_stream(stage + static_cast<uint64_t>(s) * a.shardRows * rowBytes + off[q]);
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
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
                    for (int q = 0; q < 2; ++q) {
                        if (i0 + q * 256 < total) {
                            st_vec16(a.c + off[q], Vec16{FbPackPair(accv[q][0], accv[q][1], bf16), FbPackPair(accv[q][2], accv[q][3], bf16),
                                                         FbPackPair(accv[q][4], accv[q][5], bf16), FbPackPair(accv[q][6], accv[q][7], bf16)});
                        }
                    }
                }
            }
        }
    }

    // ---- tear-down -------------------------------------------------------------------------------------------------------
    FbFenceBefore();
    __syncthreads();
    FbClusterSync();
    FbFenceAfter();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(FB_TMEM_COLS) : "memory");
    }
    const bool failed = st->abortFlag != 0;
    if (failed && threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, TILEXR_DEV_MBARRIER_TIMEOUT);
    if (fused) {
        Waiter w{a.comm, st->epoch, static_cast<int32_t>(blockIdx.x), TILEXR_DEV_OK, 0};
        if (failed && threadIdx.x == 0) RaiseFailure(w, TILEXR_DEV_MBARRIER_TIMEOUT, a.comm->rank, blockIdx.x, 0, 0);
        KernelEpilogue(w, !failed);
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_FP8_BLOCK_THREADS, 1)
TileXRGemmFp8BlockScaled(const __grid_constant__ GemmBlockArgs a) { FbBody(a); }
// Emulated worlds: one argument block per rank in global memory, rank = blockIdx.y.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_FP8_BLOCK_THREADS, 1)
TileXRGemmFp8BlockScaled_emulated(const GemmBlockArgs *perRank) { FbBody(perRank[blockIdx.y]); }

} // namespace

const void *GemmFp8BlockKernel() { return reinterpret_cast<const void *>(&TileXRGemmFp8BlockScaled); }
const void *GemmFp8BlockKernelEmulated() { return reinterpret_cast<const void *>(&TileXRGemmFp8BlockScaled_emulated); }

} // namespace TileXR
