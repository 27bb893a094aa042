// All-reduce fused with residual add and RMSNorm (the tensor-parallel epilogue of an attention
// or MLP block): one kernel, no intermediate tensor, flag-synchronised per row.
//
// One-shot (latency, small batches): every rank pushes its rows to every peer and every rank
// reduces every row itself: one NVLink hop, (R-1) x message bytes per rank.
// Two-shot (bandwidth): row r is owned by rank r / rowsPerRank.  Ranks push each row to its
// owner; the owner reduces in rank order, adds the residual, normalises, and pushes the
// normalised row and the new residual to every peer: 3 (R-1)/R x message bytes per rank.
// Both sum in rank order 0..R-1 in fp32, so all ranks hold bit-identical results.
//
// Window use inside one data half, per (source, destination) pair region of `pairStride`:
//   plane A  [row][rowBytes]                 partial rows           flag plane A slot = row
//   plane B  [row][2][rowBytes]              {y, residual} rows     flag plane B slot = row
// with at most TILEXR_FLAGS_PER_PAIR rows per pair and launch; the host splits larger batches.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "device/tilexr_rma.cuh"
#include "device/tilexr_sync.cuh"
#include "device/tilexr_convert.cuh"
#include "tilexr_fused.h"
#include "tilexr_launch.h"
#include "tilexr_log.h"

namespace TileXR {

using namespace tilexr;

namespace {

constexpr unsigned ARN_THREADS = 512;
constexpr int ARN_MAX_VECS = 4;   // 512 threads x 4 x 8 elements = 16384 columns

struct ArNormArgs {
    const uint8_t *x;
    uint8_t *residual;
    const uint8_t *gamma;
    uint8_t *y;
    CommArgs *comm;
    int64_t magic;
    float eps;
    int32_t rows;          // rows in this launch
    int32_t h;
    int32_t rowsPerRank;   // two-shot: rows owned by each rank (last ranks may own fewer / none)
    int32_t twoShot;
    uint32_t rowBytes;
    uint32_t pairStride;
    uint32_t isBf16;
    uint32_t zeroCopy;     // two-shot: y and residual are registered, peers are written directly
    uint32_t yHandle, resHandle;
    uint64_t yOffset, resOffset;
};

__device__ __forceinline__ uint8_t *PlaneA(const ArNormArgs &a, int dst, int src, int row, uint32_t epoch)
{
    return DataHalf(a.comm, dst, epoch) + static_cast<uint64_t>(src) * a.pairStride + static_cast<uint64_t>(row) * a.rowBytes;
}
__device__ __forceinline__ uint8_t *PlaneB(const ArNormArgs &a, int dst, int src, int row, int which, uint32_t epoch, int planeARows)
{
    return DataHalf(a.comm, dst, epoch) + static_cast<uint64_t>(src) * a.pairStride +
           (static_cast<uint64_t>(planeARows) + static_cast<uint64_t>(row) * 2 + which) * a.rowBytes;
}
__device__ __forceinline__ uint64_t *FlagA(const ArNormArgs &a, int owner, int src, int row)
{
    return FlagSlot(a.comm, owner, TILEXR_FLAG_DATA_BASE + static_cast<int64_t>(src) * TILEXR_FLAGS_PER_PAIR + row);
}
__device__ __forceinline__ uint64_t *FlagB(const ArNormArgs &a, int owner, int src, int row)
{
    return FlagSlot(a.comm, owner, TILEXR_FLAG_ACK_BASE + static_cast<int64_t>(src) * TILEXR_FLAGS_PER_PAIR + row);
}

// Sums row `row` over all ranks in rank order (`srcOf(s)` gives rank s's copy), adds the
// residual, normalises.  Leaves y and the new residual in `yDst` / `resDst` (local) and,
// when `stage` is not null, also in stage[0] (y) and stage[1] (residual) for the fan-out.
template <typename SrcFn>
__device__ __forceinline__ void ReduceNormRow(const ArNormArgs &a, SrcFn srcOf, int R, const uint8_t *resSrc, uint8_t *resDst,
                                              uint8_t *yDst, float *sPartial)
{
    const bool bf16 = a.isBf16 != 0;
    const int vecs = a.rowBytes / 16;
    float vals[ARN_MAX_VECS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < ARN_MAX_VECS; ++i) {
        const int v = i * ARN_THREADS + threadIdx.x;
        if (v < vecs) {
            // Four ranks' copies of the column are fetched before the first is added (in rank order, so the sum does not
            // depend on the batching): one at a time, every rank costs the thread a memory round trip of its own.
            float acc[8];
            for (int s0 = 0; s0 < R; s0 += 4) {
                Vec16 q[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (s0 + u < R) q[u] = ld_vec16_stream(srcOf(s0 + u) + v * 16);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (s0 + u < R) {
                        float f[8];
                        Unpack8(q[u], bf16, f);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] = (s0 + u == 0) ? f[j] : acc[j] + f[j];
                    }
                }
            }
            if (resSrc != nullptr) {
                float r[8];
                Unpack8(ld_vec16(resSrc + v * 16), bf16, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += r[j];
            }
            // the sum rounded to the storage type is the new residual AND the norm input
            const Vec16 packed = Pack8(acc, bf16);
            if (resDst != nullptr) st_vec16(resDst + v * 16, packed);
            Unpack8(packed, bf16, vals[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();   // sPartial of the previous row is no longer read
    if ((threadIdx.x & 31) == 0) sPartial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < static_cast<int>(ARN_THREADS / 32); ++i) tot += sPartial[i];
    const float rstd = rsqrtf(tot / static_cast<float>(a.h) + a.eps);
#pragma unroll
    for (int i = 0; i < ARN_MAX_VECS; ++i) {
        const int v = i * ARN_THREADS + threadIdx.x;
        if (v < vecs) {
            float g[8], o[8];
            Unpack8(ld_vec16(a.gamma + v * 16), bf16, g);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * g[j];
            st_vec16(yDst + v * 16, Pack8(o, bf16));
        }
    }
}

__device__ void ArNormBody(const ArNormArgs &a)
{
    __shared__ float sPartial[ARN_THREADS / 32];
    Waiter w;
    bool ok = KernelPrologue(w, a.comm, a.magic, TILEXR_OP_ALL_REDUCE_RMSNORM, a.rows, true);
    CommArgs *comm = a.comm;
    const int rank = comm->rank;
    const int R = comm->rankSize;
    const uint32_t epoch = w.epoch;
    const int tid = threadIdx.x;
    const uint64_t rb = a.rowBytes;

    if (ok && !a.twoShot) {
        // push every row of mine to every peer, then reduce every row
        for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
            const uint8_t *src = a.x + row * rb;
            for (int i = 1; i < R; ++i) {
                const int peer = (rank + i) % R;
                CopyLanes(PlaneA(a, peer, rank, row, epoch), src, rb, tid, blockDim.x);
            }
            __syncthreads();
            if (tid < R && tid != rank) SetFlag(FlagA(a, tid, rank, row), epoch, 1);
        }
        for (int row = blockIdx.x; row < a.rows && ok; row += gridDim.x) {
            bool got = true;
            if (tid < R && tid != rank) got = WaitFlagGE(w, FlagA(a, rank, tid, row), 1, tid, row);
            ok = BlockBroadcastOk(got);
            if (!ok) break;
            auto srcOf = [&](int s) -> const uint8_t * { return s == rank ? a.x + row * rb : PlaneA(a, rank, s, row, epoch); };
            uint8_t *res = a.residual != nullptr ? a.residual + row * rb : nullptr;
            ReduceNormRow(a, srcOf, R, res, res, a.y + row * rb, sPartial);
        }
    } else if (ok) {
        const int per = a.rowsPerRank;
        const int myFirst = rank * per;
        const int myRows = max(0, min(per, a.rows - myFirst));
        // 1. rows of other owners go to their owner
        const int foreign = a.rows - myRows;
        for (int it = blockIdx.x; it < foreign; it += gridDim.x) {
            // enumerate foreign rows starting after my own range so that ranks start on different owners
            const int row = (min(myFirst, a.rows) + myRows + it) % a.rows;   // with fewer rows than ranks myFirst lies past the end
            const int owner = row / per;
            const int local = row - owner * per;
            CopyLanes(PlaneA(a, owner, rank, local, epoch), a.x + row * rb, rb, tid, blockDim.x);
            __syncthreads();
            if (tid == 0) SetFlag(FlagA(a, owner, rank, local), epoch, 1);
        }
        // 2. my rows: reduce, normalise, fan out
        for (int local = blockIdx.x; local < myRows && ok; local += gridDim.x) {
            const int row = myFirst + local;
            bool got = true;
            if (tid < R && tid != rank) got = WaitFlagGE(w, FlagA(a, rank, tid, local), 1, tid, local);
            ok = BlockBroadcastOk(got);
            if (!ok) break;
            auto srcOf = [&](int s) -> const uint8_t * { return s == rank ? a.x + row * rb : PlaneA(a, rank, s, local, epoch); };
            uint8_t *yRow = a.y + row * rb;
            uint8_t *resRow = a.residual != nullptr ? a.residual + row * rb : nullptr;
            ReduceNormRow(a, srcOf, R, resRow, resRow, yRow, sPartial);
            __syncthreads();   // the finished row is read back below by other threads
            for (int i = 1; i < R; ++i) {
                const int peer = (rank + i) % R;
                uint8_t *yDst, *rDst;
                if (a.zeroCopy) {
                    yDst = comm->registryPtr->regions[a.yHandle].peerBase[peer] + a.yOffset + row * rb;
                    rDst = resRow != nullptr ? comm->registryPtr->regions[a.resHandle].peerBase[peer] + a.resOffset + row * rb : nullptr;
                } else {
                    yDst = PlaneB(a, peer, rank, local, 0, epoch, per);
                    rDst = resRow != nullptr ? PlaneB(a, peer, rank, local, 1, epoch, per) : nullptr;
                }
                CopyLanes(yDst, yRow, rb, tid, blockDim.x);
                if (rDst != nullptr) CopyLanes(rDst, resRow, rb, tid, blockDim.x);
            }
            __syncthreads();
            if (tid < R && tid != rank) SetFlag(FlagB(a, tid, rank, local), epoch, 1);
        }
        // 3. rows of other owners come back normalised
        for (int it = blockIdx.x; it < foreign && ok; it += gridDim.x) {
            const int row = (min(myFirst, a.rows) + myRows + it) % a.rows;   // with fewer rows than ranks myFirst lies past the end
            const int owner = row / per;
            const int local = row - owner * per;
            bool got = true;
            if (tid == 0) got = WaitFlagGE(w, FlagB(a, rank, owner, local), 1, owner, local);
            ok = BlockBroadcastOk(got);
            if (ok && !a.zeroCopy) {
                CopyLanes(a.y + row * rb, PlaneB(a, rank, owner, local, 0, epoch, per), rb, tid, blockDim.x);
                if (a.residual != nullptr) {
                    CopyLanes(a.residual + row * rb, PlaneB(a, rank, owner, local, 1, epoch, per), rb, tid, blockDim.x);
                }
            }
        }
    }
    KernelEpilogue(w, ok);
}

TILEXR_DEFINE_KERNEL(TileXRAllReduceRmsNormKernel, ArNormArgs, ArNormBody, ARN_THREADS)

long EnvLong(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return *end == '\0' ? x : fallback;
}

} // namespace
} // namespace TileXR

using namespace TileXR;

extern "C" {

// One-shot moves (R-1) x bytes per rank in one hop, two-shot 3 (R-1)/R x bytes in two hops.
// Below the threshold the extra hop costs more than the extra bytes.
int TileXRAllReduceRmsNormChoose(uint64_t bytes, int rankSize)
{
    const uint64_t threshold = static_cast<uint64_t>(EnvLong("TILEXR_AR_NORM_ONESHOT_MAX_BYTES", 512 * 1024));
    if (rankSize <= 3) return TILEXR_AR_ONE_SHOT;    // two-shot moves no fewer bytes up to three ranks
    return bytes <= threshold ? TILEXR_AR_ONE_SHOT : TILEXR_AR_TWO_SHOT;
}

int TileXRAllReduceRmsNorm(const void *x, void *residualInOut, const void *gamma, float eps, int64_t rows, int64_t h,
                           TileXRDataType dtype, void *yOut, int algo, TileXRCommPtr comm, TileXRStream stream)
{
    if (comm == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    TileXRCommArgs *hostArgs = nullptr;
    GM_ADDR devArgs = nullptr;
    int ret = TileXRGetCommArgsHost(comm, &hostArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    ret = TileXRGetCommArgsDev(comm, &devArgs);
    if (ret != TILEXR_SUCCESS) return ret;
    if (hostArgs->extraFlag & TILEXR_FLAG_HOST_MEMORY) return TILEXR_ERROR_NOT_SUPPORT;
    if (x == nullptr || gamma == nullptr || yOut == nullptr || rows <= 0 || h <= 0 || h % 8 != 0 ||
        h > static_cast<int64_t>(ARN_THREADS) * ARN_MAX_VECS * 8 ||
        (dtype != TILEXR_DATA_TYPE_FP16 && dtype != TILEXR_DATA_TYPE_BFP16) || algo < TILEXR_AR_AUTO || algo > TILEXR_AR_TWO_SHOT) {
        TILEXR_LOG(ERROR) << "all-reduce+rmsnorm: bad arguments (rows " << rows << ", h " << h << ", dtype " << dtype << ")";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const int R = hostArgs->rankSize;
    const int rank = hostArgs->rank;
    const uint64_t rowBytes = static_cast<uint64_t>(h) * 2;
    const uint64_t pairStride = (hostArgs->dataHalfBytes / R) & ~static_cast<uint64_t>(255);
    if (algo == TILEXR_AR_AUTO) algo = TileXRAllReduceRmsNormChoose(static_cast<uint64_t>(rows) * rowBytes, R);
    if (R == 1) algo = TILEXR_AR_ONE_SHOT;
    const bool twoShot = algo == TILEXR_AR_TWO_SHOT;

    // rows per launch: flags and window space per pair
    int64_t maxRows;
    if (twoShot) {
        const int64_t perRank = std::min<int64_t>(TILEXR_FLAGS_PER_PAIR, static_cast<int64_t>(pairStride / (3 * rowBytes)));
        maxRows = perRank * R;
    } else {
        maxRows = std::min<int64_t>(TILEXR_FLAGS_PER_PAIR, static_cast<int64_t>(pairStride / rowBytes));
    }
    if (maxRows <= 0) {
        TILEXR_LOG(ERROR) << "all-reduce+rmsnorm: a row of " << rowBytes << " bytes does not fit the window";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    TileXRUDMAMemHandle yHandle = 0, resHandle = 0;
    uint64_t yOffset = 0, resOffset = 0;
    const uint64_t totalBytes = static_cast<uint64_t>(rows) * rowBytes;
    bool zeroCopy = twoShot && TileXRFindRegistration(comm, yOut, totalBytes, &yHandle, &yOffset) == TILEXR_SUCCESS;
    if (zeroCopy && residualInOut != nullptr) {
        zeroCopy = TileXRFindRegistration(comm, residualInOut, totalBytes, &resHandle, &resOffset) == TILEXR_SUCCESS;
    }
    const int ranksPerDevice = (hostArgs->extraFlag & TILEXR_FLAG_EMULATED) ? R : 1;
    unsigned maxGrid = 0;
    ret = MaxCooperativeGrid(comm, TileXRAllReduceRmsNormKernelEntry, ARN_THREADS, 0, ranksPerDevice, &maxGrid);
    if (ret != TILEXR_SUCCESS) return ret;

    for (int64_t done = 0; done < rows; done += maxRows) {
        const int64_t n = std::min<int64_t>(maxRows, rows - done);
        ArNormArgs a;
        std::memset(&a, 0, sizeof(a));
        a.x = static_cast<const uint8_t *>(x) + done * rowBytes;
        a.residual = residualInOut != nullptr ? static_cast<uint8_t *>(residualInOut) + done * rowBytes : nullptr;
        a.gamma = static_cast<const uint8_t *>(gamma);
        a.y = static_cast<uint8_t *>(yOut) + done * rowBytes;
        a.comm = reinterpret_cast<CommArgs *>(devArgs);
        a.eps = eps;
        a.rows = static_cast<int32_t>(n);
        a.h = static_cast<int32_t>(h);
        a.rowsPerRank = static_cast<int32_t>((n + R - 1) / R);
        a.twoShot = twoShot ? 1 : 0;
        a.rowBytes = static_cast<uint32_t>(rowBytes);
        a.pairStride = static_cast<uint32_t>(pairStride);
        a.isBf16 = dtype == TILEXR_DATA_TYPE_BFP16 ? 1u : 0u;
        a.zeroCopy = zeroCopy ? 1u : 0u;
        a.yHandle = yHandle;
        a.resHandle = resHandle;
        a.yOffset = yOffset + done * rowBytes;
        a.resOffset = resOffset + done * rowBytes;
        int64_t magic = 0;
        ret = TileXRCommNextMagic(comm, &magic);
        if (ret != TILEXR_SUCCESS) return ret;
        a.magic = magic;
        (void)rank;
        const int64_t work = twoShot ? n : n;
        const unsigned want = static_cast<unsigned>(std::min<int64_t>(work, EnvLong("TILEXR_AR_NORM_BLOCKS", 64)));
        const unsigned grid = std::max(1u, std::min(want, maxGrid));
        LaunchConfig cfg{grid, ARN_THREADS, 0, true};
        ret = LaunchKernel(comm, TileXRAllReduceRmsNormKernelEntry, &a, cfg, stream);
        if (ret != TILEXR_SUCCESS) return ret;
    }
    return TILEXR_SUCCESS;
}

} // extern "C"
