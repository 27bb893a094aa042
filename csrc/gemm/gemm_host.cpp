// Host side of the tcgen05 GEMM family: tensor-map construction, tiling, launch.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime_api.h>

#include "gemm_kernels.cuh"
#include "tilexr_fused.h"
#include "tilexr_log.h"

using namespace TileXR;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn EncodeTiled()
{
    static EncodeTiledFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

long EnvLong(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

// Row-major [rows, cols] 8-bit matrix, box = boxRows x 128 columns (one 128-byte swizzle row).
int MakeMap8(CUtensorMap *map, const void *base, int64_t rows, int64_t cols, int boxRows)
{
    EncodeTiledFn fn = EncodeTiled();
    if (fn == nullptr) {
        TILEXR_LOG(ERROR) << "cuTensorMapEncodeTiled is not available from this driver";
        return TILEXR_ERROR_RUNTIME;
    }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols)};
    const cuuint32_t box[2] = {2 * GEMM_BK, static_cast<cuuint32_t>(boxRows)};
    const cuuint32_t elemStrides[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elemStrides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        TILEXR_LOG(ERROR) << "cuTensorMapEncodeTiled failed with " << static_cast<int>(r) << " for an 8-bit " << rows << "x" << cols
                          << " matrix at " << base;
        return TILEXR_ERROR_RUNTIME;
    }
    return TILEXR_SUCCESS;
}

// Row-major [rows, cols] 16-bit matrix, box = boxRows x 64 columns, 128-byte swizzle.
int MakeMap(CUtensorMap *map, const void *base, int64_t rows, int64_t cols, int boxRows, bool bf16)
{
    EncodeTiledFn fn = EncodeTiled();
    if (fn == nullptr) {
        TILEXR_LOG(ERROR) << "cuTensorMapEncodeTiled is not available from this driver";
        return TILEXR_ERROR_RUNTIME;
    }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {GEMM_BK, static_cast<cuuint32_t>(boxRows)};
    const cuuint32_t elemStrides[2] = {1, 1};
    const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                          const_cast<void *>(base), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        TILEXR_LOG(ERROR) << "cuTensorMapEncodeTiled failed with " << static_cast<int>(r) << " for a " << rows << "x" << cols
                          << " matrix at " << base;
        return TILEXR_ERROR_RUNTIME;
    }
    return TILEXR_SUCCESS;
}

int CheckShape(const void *a, const void *b, const void *c, int64_t m, int64_t n, int64_t k, int dtype)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (dtype != TILEXR_DATA_TYPE_FP16 && dtype != TILEXR_DATA_TYPE_BFP16) {
        TILEXR_LOG(ERROR) << "matmul: fp16 or bf16 only";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (k % 8 != 0 || n % 8 != 0) {
        TILEXR_LOG(ERROR) << "matmul: K and N must be multiples of 8 (16-byte rows for TMA and vector stores)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) {
        TILEXR_LOG(ERROR) << "matmul: operands must be 16-byte aligned";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    return TILEXR_SUCCESS;
}

int SmCount(int *sms)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    if (cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    return TILEXR_SUCCESS;
}

const KernelEntry &GemmEntry()
{
    static const KernelEntry e = {GemmKernelSingle(), GemmKernelEmulated(), sizeof(GemmArgs), "TileXRGemmTcgen05"};
    return e;
}

void FillTiling(GemmArgs *g, int64_t m, int64_t n, int64_t k)
{
    g->M = static_cast<int32_t>(m);
    g->N = static_cast<int32_t>(n);
    g->K = static_cast<int32_t>(k);
    g->mBlocks = static_cast<int32_t>((m + GEMM_BM - 1) / GEMM_BM);
    g->nBlocks = static_cast<int32_t>((n + GEMM_BN - 1) / GEMM_BN);
    g->kBlocks = static_cast<int32_t>((k + GEMM_BK - 1) / GEMM_BK);
}

} // namespace

extern "C" {

int TileXRMatmul(const void *a, const void *b, void *c, int64_t m, int64_t n, int64_t k, TileXRDataType dtype,
                 int32_t *status, TileXRStream stream)
{
    int ret = CheckShape(a, b, c, m, n, k, dtype);
    if (ret != TILEXR_SUCCESS) return ret;
    const bool bf16 = dtype == TILEXR_DATA_TYPE_BFP16;
    GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    ret = MakeMap(&g.tmapA, a, m, k, GEMM_BM, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = MakeMap(&g.tmapB, b, n, k, GEMM_BN, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    g.tmapALocal = g.tmapA;
    g.c = static_cast<uint8_t *>(c);
    g.status = status;
    g.mode = GEMM_PLAIN;
    g.isBf16 = bf16 ? 1u : 0u;
    FillTiling(&g, m, n, k);
    int sms = 0;
    ret = SmCount(&sms);
    if (ret != TILEXR_SUCCESS) return ret;
    if (m > GEMM_BM && EnvLong("TILEXR_GEMM_PAIR", 1) != 0) {
        // CTA pairs on 256x256 tiles: each CTA loads half of the B tile (its own tensor map box of 128 rows)
        ret = MakeMap(&g.tmapB, b, n, k, GEMM_BN / 2, bf16);
        if (ret != TILEXR_SUCCESS) return ret;
        g.rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
        const int pairTiles = static_cast<int>((m + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) * g.nBlocks;
        const int pairs = std::max(1, std::min<int>(pairTiles, static_cast<int>(EnvLong("TILEXR_GEMM_CTAS", sms)) / 2));
        static std::once_flag pairOnce;
        std::call_once(pairOnce, [] {
            cudaFuncSetAttribute(GemmPairKernel(), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(GEMM_PAIR_SMEM_BYTES));
        });
        void *pairParams[] = {&g};
        const cudaError_t pe = cudaLaunchKernel(GemmPairKernel(), dim3(2 * pairs), dim3(GEMM_PAIR_THREADS), pairParams,
                                                GEMM_PAIR_SMEM_BYTES, static_cast<cudaStream_t>(stream));
        if (pe != cudaSuccess) {
            TILEXR_LOG(ERROR) << "matmul (CTA pairs) launch failed: " << cudaGetErrorString(pe);
            cudaGetLastError();
            return TILEXR_ERROR_RUNTIME;
        }
        NoteLaunch();
        return TILEXR_SUCCESS;
    }
    const int tiles = g.mBlocks * g.nBlocks;
    const unsigned grid = static_cast<unsigned>(std::max(1, std::min<int>(tiles, static_cast<int>(EnvLong("TILEXR_GEMM_CTAS", sms)))));
    static std::once_flag once;
    std::call_once(once, [] {
        cudaFuncSetAttribute(GemmKernelSingle(), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(GEMM_SMEM_BYTES));
        cudaFuncSetAttribute(GemmKernelEmulated(), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(GEMM_SMEM_BYTES));
    });
    void *params[] = {&g};
    const cudaError_t e = cudaLaunchKernel(GemmKernelSingle(), dim3(grid), dim3(GEMM_THREADS), params, GEMM_SMEM_BYTES,
                                           static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        TILEXR_LOG(ERROR) << "matmul launch failed: " << cudaGetErrorString(e);
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    NoteLaunch();
    return TILEXR_SUCCESS;
}

int TileXRGroupedMatmul(const void *a, const void *b, const int64_t *groupRows, void *c, int64_t maxRows, int64_t n, int64_t k,
                        int64_t groups, TileXRDataType dtype, int epilogue, int32_t *status, TileXRStream stream)
{
    int ret = CheckShape(a, b, c, maxRows, n, k, dtype);
    if (ret != TILEXR_SUCCESS) return ret;
    if ((epilogue != GEMM_EPI_STORE && epilogue != GEMM_EPI_SWIGLU) || (epilogue == GEMM_EPI_SWIGLU && n % 16 != 0)) {
        TILEXR_LOG(ERROR) << "grouped matmul: epilogue 0 (store) or 1 (SwiGLU over interleaved gate / up rows, N a multiple of 16)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (groupRows == nullptr || groups <= 0 || groups * n > INT32_MAX || maxRows > INT32_MAX - 512) {
        TILEXR_LOG(ERROR) << "grouped matmul: a device array of row counts, at least one group, groups * N and rows within int32";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const bool bf16 = dtype == TILEXR_DATA_TYPE_BFP16;
    GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    ret = MakeMap(&g.tmapA, a, maxRows, k, GEMM_BM, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = MakeMap(&g.tmapB, b, groups * n, k, GEMM_BN / 2, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    g.tmapALocal = g.tmapA;
    g.c = static_cast<uint8_t *>(c);
    g.status = status;
    g.mode = GEMM_GROUPED;
    g.isBf16 = bf16 ? 1u : 0u;
    g.groupRows = groupRows;
    g.groupsTotal = static_cast<int32_t>(groups);
    g.epilogue = epilogue;
    FillTiling(&g, maxRows, n, k);
    g.rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
    int sms = 0;
    ret = SmCount(&sms);
    if (ret != TILEXR_SUCCESS) return ret;
    static std::once_flag pairOnce;
    std::call_once(pairOnce, [] {
        cudaFuncSetAttribute(GemmPairKernel(), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(GEMM_PAIR_SMEM_BYTES));
    });
    // The row counts stay on the device, so the number of tiles is not known here: every launch gets as many CTA pairs
    // as could be busy if all rows fell into its groups, and pairs without a tile leave at once.
    for (int64_t base = 0; base < groups; base += GEMM_MAX_GROUPS) {
        g.groupBase = static_cast<int32_t>(base);
        g.groups = static_cast<int32_t>(std::min<int64_t>(GEMM_MAX_GROUPS, groups - base));
        const int64_t tilesAtMost = ((maxRows + 2 * GEMM_BM - 1) / (2 * GEMM_BM) + g.groups) * g.nBlocks;
        const int pairs = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(tilesAtMost, EnvLong("TILEXR_GEMM_CTAS", sms) / 2)));
        void *params[] = {&g};
        const cudaError_t e = cudaLaunchKernel(GemmPairKernel(), dim3(2 * pairs), dim3(GEMM_PAIR_THREADS), params, GEMM_PAIR_SMEM_BYTES,
                                               static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) {
            TILEXR_LOG(ERROR) << "grouped matmul launch failed: " << cudaGetErrorString(e);
            cudaGetLastError();
            return TILEXR_ERROR_RUNTIME;
        }
        NoteLaunch();
    }
    return TILEXR_SUCCESS;
}

int TileXRMatmulFp8(const void *a, const void *b, void *c, int64_t m, int64_t n, int64_t k, TileXRDataType inDtype,
                    TileXRDataType outDtype, float alpha, int32_t *status, TileXRStream stream)
{
    if (a == nullptr || b == nullptr || c == nullptr || m <= 0 || n <= 0 || k <= 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if ((inDtype != TILEXR_DATA_TYPE_FP8E4M3 && inDtype != TILEXR_DATA_TYPE_FP8E5M2) ||
        (outDtype != TILEXR_DATA_TYPE_FP16 && outDtype != TILEXR_DATA_TYPE_BFP16)) {
        TILEXR_LOG(ERROR) << "fp8 matmul: operands e4m3 or e5m2, output fp16 or bf16";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (k % 16 != 0 || n % 8 != 0 ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) != 0) {
        TILEXR_LOG(ERROR) << "fp8 matmul: K a multiple of 16, N a multiple of 8, operands 16-byte aligned";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    int ret = MakeMap8(&g.tmapA, a, m, k, GEMM_BM);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = MakeMap8(&g.tmapB, b, n, k, GEMM_BN / 2);
    if (ret != TILEXR_SUCCESS) return ret;
    g.tmapALocal = g.tmapA;
    g.c = static_cast<uint8_t *>(c);
    g.status = status;
    g.mode = GEMM_PLAIN;
    g.isBf16 = outDtype == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
    g.fp8Format = inDtype == TILEXR_DATA_TYPE_FP8E5M2 ? 2 : 1;
    g.alpha = alpha;
    FillTiling(&g, m, n, k);
    g.kBlocks = static_cast<int32_t>((k + 2 * GEMM_BK - 1) / (2 * GEMM_BK));
    g.rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
    int sms = 0;
    ret = SmCount(&sms);
    if (ret != TILEXR_SUCCESS) return ret;
    const int pairTiles = static_cast<int>((m + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) * g.nBlocks;
    const int pairs = std::max(1, std::min<int>(pairTiles, static_cast<int>(EnvLong("TILEXR_GEMM_CTAS", sms)) / 2));
    static std::once_flag once;
    std::call_once(once, [] {
        cudaFuncSetAttribute(GemmPairKernel(), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(GEMM_PAIR_SMEM_BYTES));
    });
    void *params[] = {&g};
    const cudaError_t e = cudaLaunchKernel(GemmPairKernel(), dim3(2 * pairs), dim3(GEMM_PAIR_THREADS), params, GEMM_PAIR_SMEM_BYTES,
                                           static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        TILEXR_LOG(ERROR) << "fp8 matmul launch failed: " << cudaGetErrorString(e);
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    NoteLaunch();
    return TILEXR_SUCCESS;
}

int TileXRMatmulFp8BlockScaled(const void *a, const float *scaleA, const void *b, const float *scaleB, void *c, int64_t m, int64_t n,
                               int64_t k, TileXRDataType inDtype, TileXRDataType outDtype, int32_t *status, TileXRStream stream)
{
    if (a == nullptr || b == nullptr || c == nullptr || scaleA == nullptr || scaleB == nullptr || m <= 0 || n <= 0 || k <= 0) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if ((inDtype != TILEXR_DATA_TYPE_FP8E4M3 && inDtype != TILEXR_DATA_TYPE_FP8E5M2) ||
        (outDtype != TILEXR_DATA_TYPE_FP16 && outDtype != TILEXR_DATA_TYPE_BFP16)) {
        TILEXR_LOG(ERROR) << "block-scaled fp8 matmul: operands e4m3 or e5m2, output fp16 or bf16";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (k % 128 != 0 || n % 8 != 0 ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) != 0) {
        TILEXR_LOG(ERROR) << "block-scaled fp8 matmul: K a multiple of 128 (the scale block), N a multiple of 8, operands 16-byte aligned";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    GemmBlockArgs g;
    std::memset(&g, 0, sizeof(g));
    int ret = MakeMap8(&g.tmapA, a, m, k, GEMM_BM);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = MakeMap8(&g.tmapB, b, n, k, GEMM_BN / 2);
    if (ret != TILEXR_SUCCESS) return ret;
    g.scaleA = scaleA;
    g.scaleB = scaleB;
    g.c = static_cast<uint8_t *>(c);
    g.status = status;
    g.M = static_cast<int32_t>(m);
    g.N = static_cast<int32_t>(n);
    g.K = static_cast<int32_t>(k);
    g.nBlocks = static_cast<int32_t>((n + GEMM_BN - 1) / GEMM_BN);
    g.kBlocks = static_cast<int32_t>(k / 128);
    g.scaleBRows = static_cast<int32_t>((n + 127) / 128);
    g.rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
    g.isBf16 = outDtype == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
    g.fp8Format = inDtype == TILEXR_DATA_TYPE_FP8E5M2 ? 2 : 1;
    int sms = 0;
    ret = SmCount(&sms);
    if (ret != TILEXR_SUCCESS) return ret;
    const int pairTiles = static_cast<int>((m + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) * g.nBlocks;
    const int pairs = std::max(1, std::min<int>(pairTiles, static_cast<int>(EnvLong("TILEXR_GEMM_CTAS", sms)) / 2));
    static std::once_flag once;
    std::call_once(once, [] {
        cudaFuncSetAttribute(GemmFp8BlockKernel(), cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(GEMM_FP8_BLOCK_SMEM_BYTES));
    });
    void *params[] = {&g};
    const cudaError_t e = cudaLaunchKernel(GemmFp8BlockKernel(), dim3(2 * pairs), dim3(GEMM_FP8_BLOCK_THREADS), params, GEMM_FP8_BLOCK_SMEM_BYTES,
                                           static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        TILEXR_LOG(ERROR) << "block-scaled fp8 matmul launch failed: " << cudaGetErrorString(e);
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    NoteLaunch();
    return TILEXR_SUCCESS;
}

static int FusedCommon(TileXRCommPtr comm, TileXRCommArgs **hostArgs, GM_ADDR *devArgs)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    int ret = TileXRGetCommArgsHost(comm, hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if ((*hostArgs)->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_ERROR_NOT_SUPPORT;
    return TILEXR_SUCCESS;
}

static const KernelEntry &GemmPairEntry()
{
    static const KernelEntry e = {GemmPairKernel(), GemmPairKernelEmulated(), sizeof(GemmArgs), "TileXRGemmTcgen05Pair"};
    return e;
}

// The CTA-pair kernel serves a fused call when a pair's 256-row tile lies within one shard.
static bool UsePairs(int64_t shardRows) { return shardRows % (2 * GEMM_BM) == 0 && EnvLong("TILEXR_GEMM_PAIR", 1) != 0; }

static int FusedGrid(TileXRCommPtr comm, const TileXRCommArgs *hostArgs, unsigned *grid, bool pairs = false)
{
    const int ranksPerDevice = (hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? hostArgs->rankSize : 1;
    unsigned maxGrid = 0;
    int ret = pairs ? MaxCooperativeGrid(comm, GemmPairEntry(), GEMM_PAIR_THREADS, GEMM_PAIR_SMEM_BYTES, ranksPerDevice, &maxGrid)
                    : MaxCooperativeGrid(comm, GemmEntry(), GEMM_THREADS, GEMM_SMEM_BYTES, ranksPerDevice, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    if (pairs) maxGrid &= ~1u;
    if (maxGrid < 2) {
        TILEXR_LOG(ERROR) << "fused GEMM needs at least two co-resident CTAs per rank";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    *grid = static_cast<unsigned>(std::min<long>(maxGrid, EnvLong("TILEXR_GEMM_CTAS", maxGrid)));
    if (pairs) *grid &= ~1u;
    return TILEXR_SUCCESS;
}

int TileXRAllGatherMatmul(const void *aShard, void *aStaging, const void *b, void *c, int64_t shardRows, int64_t n, int64_t k,
                          TileXRDataType dtype, TileXRCommPtr comm, TileXRStream stream)
{
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = FusedCommon(comm, &hostArgs, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    const int R = hostArgs->rankSize;
    const int64_t m = shardRows * R;
    ret = CheckShape(aShard, b, c, m, n, k, dtype);
    if (ret != TILEXR_SUCCESS) return ret;
    if (aStaging == nullptr || shardRows % GEMM_BM != 0) {
        TILEXR_LOG(ERROR) << "all-gather matmul: shardRows must be a multiple of " << GEMM_BM << " and a staging buffer is required";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    TileXRUDMAMemHandle handle = 0;
    uint64_t offset = 0;
    if (TileXRFindRegistration(comm, aStaging, static_cast<size_t>(m) * k * 2, &handle, &offset) != TILEXR_SUCCESS) {
        TILEXR_LOG(ERROR) << "all-gather matmul: the staging buffer must be registered on every rank (TileXRSymmAlloc)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const bool bf16 = dtype == TILEXR_DATA_TYPE_BFP16;
    GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    ret = MakeMap(&g.tmapA, aStaging, m, k, GEMM_BM, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = MakeMap(&g.tmapALocal, aShard, shardRows, k, GEMM_BM, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    const bool pairs = UsePairs(shardRows);
    ret = MakeMap(&g.tmapB, b, n, k, pairs ? GEMM_BN / 2 : GEMM_BN, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    g.c = static_cast<uint8_t *>(c);
    g.aLocal = static_cast<const uint8_t *>(aShard);
    g.comm = reinterpret_cast<CommArgs *>(devArgs);
    g.mode = GEMM_ALL_GATHER;
    g.isBf16 = bf16 ? 1u : 0u;
    FillTiling(&g, m, n, k);
    g.shardRows = static_cast<int32_t>(shardRows);
    g.blocksPerShard = static_cast<int32_t>(shardRows / GEMM_BM);
    g.flagStride = TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR / R;
    g.kChunks = std::max(1, std::min<int>(GEMM_MAX_K_CHUNKS, std::min<int>(g.kBlocks, (g.flagStride - 1) / g.blocksPerShard)));
    g.kBlocksPerChunk = (g.kBlocks + g.kChunks - 1) / g.kChunks;
    g.kChunks = (g.kBlocks + g.kBlocksPerChunk - 1) / g.kBlocksPerChunk;
    if (g.blocksPerShard * g.kChunks >= g.flagStride) {
        TILEXR_LOG(ERROR) << "all-gather matmul: " << shardRows << " rows per rank exceed the per-pair flag space";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    g.stageHandle = handle;
    g.stageOffset = offset;
    unsigned grid = 0;
    ret = FusedGrid(comm, hostArgs, &grid, pairs);
    if (ret != TILEXR_SUCCESS) return ret;
    g.commBlocks = R > 1 ? static_cast<uint32_t>(std::max<long>(1, std::min<long>(grid / 2, EnvLong("TILEXR_AG_GEMM_COMM_CTAS", std::max(2u, grid / 10))))) : 0;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    g.magic = magic;
    if (pairs && EnvLong("TILEXR_AG_GEMM_COMM_CTAS", 0) <= 0) {
        // two otherwise idle warps of every CTA push the shard (through the multicast alias of the staging buffer where
        // there is one): no CTA is set aside
        g.rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
        g.commBlocks = 0;
        LaunchConfig pairCfg{grid, GEMM_PAIR_THREADS, GEMM_PAIR_SMEM_BYTES, true};
        return LaunchKernel(comm, GemmPairEntry(), &g, pairCfg, stream);
    }
    if (pairs) {
        g.rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
        g.commBlocks = (g.commBlocks + 1) & ~1u;          // whole pairs push, whole pairs compute
        if (g.commBlocks + 2 > grid) g.commBlocks = grid > 2 ? (grid - 2) & ~1u : 0;
        if (g.commBlocks > 0) {
            // The pushing pairs compute afterwards: each takes as many tiles from the end of the walk as fit
            // between the end of its push and the end of the whole product (rates are estimates; an error only
            // shifts a few tiles between the two groups).
            const double tileUs = 2.0 * 256 * 256 * static_cast<double>(k) / (static_cast<double>(EnvLong("TILEXR_GEMM_PAIR_TFLOPS", 17)) * 1e6);
            const double pushBytes = static_cast<double>(R - 1) * static_cast<double>(shardRows) * static_cast<double>(k) * 2.0;
            const double pushUs = pushBytes / (g.commBlocks * static_cast<double>(EnvLong("TILEXR_AG_PUSH_GBPS_PER_CTA", 10)) * 1e3);
            const double tiles = static_cast<double>((m + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) * g.nBlocks;
            const double totalUs = tiles * tileUs / (grid / 2);
            g.commTilesPerPair = totalUs > pushUs ? static_cast<uint32_t>((totalUs - pushUs) / tileUs) : 0u;
        }
        LaunchConfig pairCfg{grid, GEMM_PAIR_THREADS, GEMM_PAIR_SMEM_BYTES, true};
        return LaunchKernel(comm, GemmPairEntry(), &g, pairCfg, stream);
    }
    LaunchConfig cfg{grid, GEMM_THREADS, GEMM_SMEM_BYTES, true};
    return LaunchKernel(comm, GemmEntry(), &g, cfg, stream);
}

int TileXRMatmulReduceScatter(const void *a, const void *b, void *partialStaging, void *out, int64_t shardRows, int64_t n,
                              int64_t k, TileXRDataType dtype, TileXRCommPtr comm, TileXRStream stream)
{
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = FusedCommon(comm, &hostArgs, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    const int R = hostArgs->rankSize;
    const int64_t m = shardRows * R;
    ret = CheckShape(a, b, out, m, n, k, dtype);
    if (ret != TILEXR_SUCCESS) return ret;
    if (partialStaging == nullptr || shardRows % GEMM_BM != 0) {
        TILEXR_LOG(ERROR) << "matmul reduce-scatter: shardRows must be a multiple of " << GEMM_BM << " and a staging buffer is required";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    TileXRUDMAMemHandle handle = 0;
    uint64_t offset = 0;
    if (TileXRFindRegistration(comm, partialStaging, static_cast<size_t>(m) * n * 2, &handle, &offset) != TILEXR_SUCCESS) {
        TILEXR_LOG(ERROR) << "matmul reduce-scatter: the staging buffer must be registered on every rank (TileXRSymmAlloc)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const bool bf16 = dtype == TILEXR_DATA_TYPE_BFP16;
    GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    ret = MakeMap(&g.tmapA, a, m, k, GEMM_BM, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    g.tmapALocal = g.tmapA;
    const bool pairs = UsePairs(shardRows);
    ret = MakeMap(&g.tmapB, b, n, k, pairs ? GEMM_BN / 2 : GEMM_BN, bf16);
    if (ret != TILEXR_SUCCESS) return ret;
    g.c = static_cast<uint8_t *>(out);
    g.comm = reinterpret_cast<CommArgs *>(devArgs);
    g.mode = GEMM_REDUCE_SCATTER;
    g.isBf16 = bf16 ? 1u : 0u;
    FillTiling(&g, m, n, k);
    g.shardRows = static_cast<int32_t>(shardRows);
    g.blocksPerShard = static_cast<int32_t>(shardRows / GEMM_BM);
    g.flagStride = TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR / R;
    if (static_cast<int64_t>(g.blocksPerShard) * g.nBlocks >= g.flagStride) {
        TILEXR_LOG(ERROR) << "matmul reduce-scatter: " << g.blocksPerShard * g.nBlocks << " tiles per owner exceed the per-pair flag space";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    g.stageHandle = handle;
    g.stageOffset = offset;
    unsigned grid = 0;
    ret = FusedGrid(comm, hostArgs, &grid, pairs);
    if (ret != TILEXR_SUCCESS) return ret;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    g.magic = magic;
    if (pairs) {
        g.rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
        LaunchConfig pairCfg{grid, GEMM_PAIR_THREADS, GEMM_PAIR_SMEM_BYTES, true};
        return LaunchKernel(comm, GemmPairEntry(), &g, pairCfg, stream);
    }
    LaunchConfig cfg{grid, GEMM_THREADS, GEMM_SMEM_BYTES, true};
    return LaunchKernel(comm, GemmEntry(), &g, cfg, stream);
}

// ---- block-scaled fp8 with the collectives of a tensor-parallel layer ----------------------------------------------------

static const KernelEntry &GemmFp8BlockEntry()
{
    static const KernelEntry e = {GemmFp8BlockKernel(), GemmFp8BlockKernelEmulated(), sizeof(GemmBlockArgs), "TileXRGemmFp8BlockScaled"};
    return e;
}

static int Fp8BlockFusedGrid(TileXRCommPtr comm, const TileXRCommArgs *hostArgs, unsigned *grid)
{
    const int ranksPerDevice = (hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? hostArgs->rankSize : 1;
    unsigned maxGrid = 0;
    int ret = MaxCooperativeGrid(comm, GemmFp8BlockEntry(), GEMM_FP8_BLOCK_THREADS, GEMM_FP8_BLOCK_SMEM_BYTES, ranksPerDevice, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;
    maxGrid &= ~1u;
    if (maxGrid < 2) {
        TILEXR_LOG(ERROR) << "fused block-scaled GEMM needs at least one co-resident CTA pair per rank";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    *grid = static_cast<unsigned>(std::min<long>(maxGrid, EnvLong("TILEXR_GEMM_CTAS", maxGrid))) & ~1u;
    return TILEXR_SUCCESS;
}

static int Fp8BlockCommon(GemmBlockArgs *g, const void *b, const float *scaleB, int64_t m, int64_t n, int64_t k, TileXRDataType inDtype,
                          TileXRDataType outDtype, int64_t shardRows, int R, const char *what)
{
    if ((inDtype != TILEXR_DATA_TYPE_FP8E4M3 && inDtype != TILEXR_DATA_TYPE_FP8E5M2) ||
        (outDtype != TILEXR_DATA_TYPE_FP16 && outDtype != TILEXR_DATA_TYPE_BFP16)) {
        TILEXR_LOG(ERROR) << what << ": operands e4m3 or e5m2, output fp16 or bf16";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (k % 128 != 0 || n % 8 != 0 || shardRows % (2 * GEMM_BM) != 0 || (reinterpret_cast<uintptr_t>(b) & 15u) != 0 || scaleB == nullptr) {
        TILEXR_LOG(ERROR) << what << ": K a multiple of 128, N a multiple of 8, rows per rank a multiple of " << 2 * GEMM_BM;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    int ret = MakeMap8(&g->tmapB, b, n, k, GEMM_BN / 2);
    if (ret != TILEXR_SUCCESS) return ret;
    g->scaleB = scaleB;
    g->M = static_cast<int32_t>(m);
    g->N = static_cast<int32_t>(n);
    g->K = static_cast<int32_t>(k);
    g->nBlocks = static_cast<int32_t>((n + GEMM_BN - 1) / GEMM_BN);
    g->kBlocks = static_cast<int32_t>(k / 128);
    g->scaleBRows = static_cast<int32_t>((n + 127) / 128);
    g->rasterGroup = static_cast<int32_t>(std::max<long>(1, EnvLong("TILEXR_GEMM_GROUP", 8)));
    g->isBf16 = outDtype == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
    g->fp8Format = inDtype == TILEXR_DATA_TYPE_FP8E5M2 ? 2 : 1;
    g->shardRows = static_cast<int32_t>(shardRows);
    g->blocksPerShard = static_cast<int32_t>(shardRows / GEMM_BM);
    g->flagStride = TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR / R;
    return TILEXR_SUCCESS;
}

int TileXRAllGatherMatmulFp8Block(const void *aShard, const float *scaleAShard, void *aStaging, float *scaleStaging, const void *b,
                                  const float *scaleB, void *c, int64_t shardRows, int64_t n, int64_t k, TileXRDataType inDtype,
                                  TileXRDataType outDtype, TileXRCommPtr comm, TileXRStream stream)
{
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = FusedCommon(comm, &hostArgs, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    const int R = hostArgs->rankSize;
    const int64_t m = shardRows * R;
    if (aShard == nullptr || scaleAShard == nullptr || aStaging == nullptr || scaleStaging == nullptr || b == nullptr || c == nullptr ||
        shardRows <= 0 || n <= 0 || k <= 0 ||
        ((reinterpret_cast<uintptr_t>(aShard) | reinterpret_cast<uintptr_t>(scaleAShard) | reinterpret_cast<uintptr_t>(c)) & 15u) != 0) {
        TILEXR_LOG(ERROR) << "all-gather block-scaled matmul: null or misaligned tensor";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    GemmBlockArgs g;
    std::memset(&g, 0, sizeof(g));
    ret = Fp8BlockCommon(&g, b, scaleB, m, n, k, inDtype, outDtype, shardRows, R, "all-gather block-scaled matmul");
    if (ret != TILEXR_SUCCESS) return ret;
    if ((k / 128 * 4) % 16 != 0) {
        TILEXR_LOG(ERROR) << "all-gather block-scaled matmul: K must be a multiple of 512 (rows of the scale table travel in 16-byte pieces)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    if (g.blocksPerShard >= g.flagStride) {
        TILEXR_LOG(ERROR) << "all-gather block-scaled matmul: " << shardRows << " rows per rank exceed the per-pair flag space";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    TileXRUDMAMemHandle aHandle = 0, sHandle = 0;
    uint64_t aOffset = 0, sOffset = 0;
    if (TileXRFindRegistration(comm, aStaging, static_cast<size_t>(m) * k, &aHandle, &aOffset) != TILEXR_SUCCESS ||
        TileXRFindRegistration(comm, scaleStaging, static_cast<size_t>(m) * (k / 128) * 4, &sHandle, &sOffset) != TILEXR_SUCCESS) {
        TILEXR_LOG(ERROR) << "all-gather block-scaled matmul: both staging buffers must be registered on every rank (TileXRSymmAlloc)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    ret = MakeMap8(&g.tmapA, aStaging, m, k, GEMM_BM);
    if (ret != TILEXR_SUCCESS) return ret;
    g.scaleA = scaleStaging;
    g.c = static_cast<uint8_t *>(c);
    g.mode = GEMM_ALL_GATHER;
    g.comm = reinterpret_cast<CommArgs *>(devArgs);
    g.aLocal = static_cast<const uint8_t *>(aShard);
    g.scaleALocal = scaleAShard;
    g.aHandle = aHandle;
    g.aOffset = aOffset;
    g.sHandle = sHandle;
    g.sOffset = sOffset;
    unsigned grid = 0;
    ret = Fp8BlockFusedGrid(comm, hostArgs, &grid);
    if (ret != TILEXR_SUCCESS) return ret;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    g.magic = magic;
    LaunchConfig cfg{grid, GEMM_FP8_BLOCK_THREADS, GEMM_FP8_BLOCK_SMEM_BYTES, true};
    return LaunchKernel(comm, GemmFp8BlockEntry(), &g, cfg, stream);
}

int TileXRMatmulReduceScatterFp8Block(const void *a, const float *scaleA, const void *b, const float *scaleB, void *partialStaging, void *out,
                                      int64_t shardRows, int64_t n, int64_t k, TileXRDataType inDtype, TileXRDataType outDtype,
                                      TileXRCommPtr comm, TileXRStream stream)
{
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = FusedCommon(comm, &hostArgs, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    const int R = hostArgs->rankSize;
    const int64_t m = shardRows * R;
    if (a == nullptr || scaleA == nullptr || b == nullptr || partialStaging == nullptr || out == nullptr || shardRows <= 0 || n <= 0 || k <= 0 ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15u) != 0) {
        TILEXR_LOG(ERROR) << "block-scaled matmul reduce-scatter: null or misaligned tensor";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    GemmBlockArgs g;
    std::memset(&g, 0, sizeof(g));
    ret = Fp8BlockCommon(&g, b, scaleB, m, n, k, inDtype, outDtype, shardRows, R, "block-scaled matmul reduce-scatter");
    if (ret != TILEXR_SUCCESS) return ret;
    if (static_cast<int64_t>(g.blocksPerShard) * g.nBlocks >= g.flagStride) {
        TILEXR_LOG(ERROR) << "block-scaled matmul reduce-scatter: " << g.blocksPerShard * g.nBlocks << " tiles per owner exceed the per-pair flag space";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    TileXRUDMAMemHandle handle = 0;
    uint64_t offset = 0;
    if (TileXRFindRegistration(comm, partialStaging, static_cast<size_t>(m) * n * 2, &handle, &offset) != TILEXR_SUCCESS) {
        TILEXR_LOG(ERROR) << "block-scaled matmul reduce-scatter: the staging buffer must be registered on every rank (TileXRSymmAlloc)";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    ret = MakeMap8(&g.tmapA, a, m, k, GEMM_BM);
    if (ret != TILEXR_SUCCESS) return ret;
    g.scaleA = scaleA;
    g.c = static_cast<uint8_t *>(out);
    g.mode = GEMM_REDUCE_SCATTER;
    g.comm = reinterpret_cast<CommArgs *>(devArgs);
    g.outHandle = handle;
    g.outOffset = offset;
    unsigned grid = 0;
    ret = Fp8BlockFusedGrid(comm, hostArgs, &grid);
    if (ret != TILEXR_SUCCESS) return ret;
    int64_t magic = 0;
    ret = TileXRCommNextMagic(comm, &magic);
    if (ret != TILEXR_SUCCESS) return ret;
    g.magic = magic;
    LaunchConfig cfg{grid, GEMM_FP8_BLOCK_THREADS, GEMM_FP8_BLOCK_SMEM_BYTES, true};
    return LaunchKernel(comm, GemmFp8BlockEntry(), &g, cfg, stream);
}

} // extern "C"
