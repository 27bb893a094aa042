// Argument block of the tcgen05 GEMM family (plain, all-gather -> GEMM, GEMM -> reduce-scatter).
#ifndef TILEXR_GEMM_KERNELS_CUH
#define TILEXR_GEMM_KERNELS_CUH

#include <cuda.h>
#include <stdint.h>

#include "tilexr_comm_args.h"
#include "tilexr_launch.h"

namespace TileXR {

constexpr int GEMM_BM = 128;        // rows of C per tile  = UMMA M
constexpr int GEMM_BN = 256;        // columns of C per tile = UMMA N
constexpr int GEMM_BK = 64;         // K per pipeline stage = one 128-byte swizzle row of bf16
constexpr int GEMM_UMMA_K = 16;     // K of one tcgen05.mma for 16-bit inputs
constexpr int GEMM_STAGES = 4;
constexpr unsigned GEMM_THREADS = 192;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr unsigned GEMM_PAIR_THREADS = 256;   // CTA-pair kernel: two more warps that push this rank's shard in the all-gather mode
constexpr uint32_t GEMM_STAGE_A_BYTES = GEMM_BM * GEMM_BK * 2;
constexpr uint32_t GEMM_STAGE_B_BYTES = GEMM_BN * GEMM_BK * 2;
constexpr uint32_t GEMM_STAGE_BYTES = GEMM_STAGE_A_BYTES + GEMM_STAGE_B_BYTES;
constexpr size_t GEMM_SMEM_BYTES = 1024 /* alignment slack */ + GEMM_STAGES * GEMM_STAGE_BYTES + 256 /* barriers */;
constexpr int GEMM_MAX_K_CHUNKS = 4;     // all-gather flags per 128-row block
// CTA-pair kernel (cta_group::2): per CTA and stage 128 rows of A and half of the 256-row B tile.
constexpr uint32_t GEMM_PAIR_STAGE_BYTES = GEMM_STAGE_A_BYTES + GEMM_STAGE_B_BYTES / 2;
constexpr int GEMM_PAIR_STAGES = 6;
constexpr size_t GEMM_PAIR_SMEM_BYTES = 1024 /* alignment slack */ + GEMM_PAIR_STAGES * GEMM_PAIR_STAGE_BYTES + 1024 /* barriers */ +
                                        GEMM_BM * 256 /* epilogue staging tile */;

enum GemmMode : int32_t {
    GEMM_PLAIN = 0,
    GEMM_ALL_GATHER = 1,      // A is gathered: local shard + staging filled by peers
    GEMM_REDUCE_SCATTER = 2,  // C is reduce-scattered: partial tiles pushed to the row owner
    GEMM_GROUPED = 3,         // rows of A grouped by expert, one weight per group, row counts read on the device
};
constexpr int GEMM_MAX_GROUPS = 64;      // groups of one launch (their row and tile offsets live in shared memory)

struct GemmArgs {
    CUtensorMap tmapA;        // A [M, K] row-major (all-gather: the staging buffer [R * shardRows, K])
    CUtensorMap tmapALocal;   // all-gather: this rank's shard [shardRows, K]
    CUtensorMap tmapB;        // B [N, K] row-major (the weight; C = A x B^T)
    uint8_t *c;               // plain / all-gather: C [M, N]; reduce-scatter: out [shardRows, N]
    const uint8_t *aLocal;    // all-gather: shard to push to the peers
    CommArgs *comm;
    int32_t *status;          // device int, set non-zero when a pipeline wait gave up
    int64_t magic;
    int32_t mode;
    int32_t M, N, K;          // M = rows of the whole product (R * shardRows in the fused modes)
    int32_t mBlocks, nBlocks, kBlocks;
    int32_t shardRows;        // rows per rank in the fused modes
    int32_t blocksPerShard;   // shardRows / GEMM_BM
    int32_t kChunks;          // all-gather: flags per row block
    int32_t flagStride;       // flags of one (source, destination) pair: the flag plane divided by the rank count
    int32_t kBlocksPerChunk;
    uint32_t commBlocks;      // all-gather: leading CTAs that push the local shard to the peers first
    uint32_t commTilesPerPair; // CTA-pair kernel: tiles (taken from the END of the walk) that each pushing pair computes afterwards
    uint32_t stageHandle;     // registry handle of the staging buffer (A staging or partial-C staging)
    uint64_t stageOffset;
    uint32_t isBf16;
    int32_t rasterGroup;      // CTA-pair kernel, plain mode: 256-row blocks per group of the tile walk
    // 8-bit operands (CTA-pair kernel, plain mode): 0 = 16-bit operands per isBf16, 1 = fp8 e4m3, 2 = fp8 e5m2.
    // A stage still holds one 128-byte swizzle row per operand row, i.e. 128 elements of K, and one tcgen05.mma
    // (kind::f8f6f4) covers 32 of them; C = alpha * A x B^T is written in the 16-bit type named by isBf16.
    int32_t fp8Format;
    float alpha;
    // Grouped mode (CTA-pair kernel): A [M, K] holds the rows of group 0, then group 1, ...; groupRows[g] of them (a
    // device array, so that no host round trip separates the kernel that counted the rows from this one).  B is
    // [groupsTotal * N, K], the weight of group g in rows [g * N, (g + 1) * N); C [M, N].  One launch covers groups
    // [groupBase, groupBase + groups).
    const int64_t *groupRows;
    int32_t groups, groupBase, groupsTotal;
    // Epilogue of the CTA-pair kernel (plain and grouped modes): 0 stores the product; 1 treats the columns as
    // (gate, up) pairs -- weight row 2i the gate row i, row 2i+1 the up row i -- and stores silu(gate) * up, so C is
    // [M, N / 2] and the [M, N] intermediate of a SwiGLU feed-forward never reaches memory.
    int32_t epilogue;
};
enum GemmEpilogue : int32_t { GEMM_EPI_STORE = 0, GEMM_EPI_SWIGLU = 1 };

// Block-scaled fp8 GEMM (gemm_tcgen05_fp8_block.cu): warp 0 TMA, warp 1 MMA, warps 4-11 fold the scratch accumulators.
constexpr unsigned GEMM_FP8_BLOCK_THREADS = 384;
constexpr int GEMM_FP8_BLOCK_STAGES = 5;     // one stage less than the bf16 kernel: the weight scales of a tile live in shared memory too
constexpr size_t GEMM_FP8_BLOCK_SMEM_BYTES = 1024 /* alignment slack */ + GEMM_FP8_BLOCK_STAGES * GEMM_PAIR_STAGE_BYTES + 1024 /* barriers */ +
                                             GEMM_BM * 256 /* epilogue staging tile */;

struct GemmBlockArgs {
    CUtensorMap tmapA;        // A [M, K] 8-bit, box 128 rows x 128 bytes
    CUtensorMap tmapB;        // B [N, K] 8-bit, box 128 rows x 128 bytes
    const float *scaleA;      // [M, K / 128]
    const float *scaleB;      // [scaleBRows, K / 128], one row per 128 rows of B
    uint8_t *c;               // [M, N] bf16 or fp16
    int32_t *status;
    int32_t M, N, K;
    int32_t nBlocks;          // 256-column tiles
    int32_t kBlocks;          // K / 128
    int32_t scaleBRows;       // ceil(N / 128)
    int32_t rasterGroup;
    uint32_t isBf16;
    int32_t fp8Format;        // 1 = e4m3, 2 = e5m2
    // Fused modes (GemmMode).  ALL_GATHER: tmapA and scaleA describe THIS rank's staging buffers ([R * shardRows, K] rows,
    // [R * shardRows, K / 128] scales, both registered on every rank); every rank writes its shard and the shard's
    // scales into all of them while the tiles are computed, and a tile starts when the flag of its 128 rows is up.
    // REDUCE_SCATTER: every 128 x 256 partial tile is stored into the row owner's partial staging buffer
    // ([R, shardRows, N] 16-bit, registered) and the owner adds the R partials in rank order into c [shardRows, N].
    int32_t mode;
    CommArgs *comm;
    int64_t magic;
    const uint8_t *aLocal;    // all-gather: [shardRows, K]
    const float *scaleALocal; // all-gather: [shardRows, K / 128]
    uint32_t aHandle, sHandle, outHandle;
    uint64_t aOffset, sOffset, outOffset;
    int32_t shardRows, blocksPerShard, flagStride;
};

const void *GemmFp8BlockKernel();
const void *GemmFp8BlockKernelEmulated();
const void *GemmKernelSingle();
const void *GemmKernelEmulated();
const void *GemmPairKernel();
const void *GemmPairKernelEmulated();

} // namespace TileXR

#endif
