// Basic enums shared by every TileXR-B200 library: status codes, element types,
// reduction operators and operator ids.  Numeric values follow the reference ABI
// (src/include/tilexr_types.h:17-25, 60-127) so existing callers keep their constants.
#ifndef TILEXR_TYPES_H
#define TILEXR_TYPES_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
namespace TileXR {
#endif

enum TileXRStatus {
    TILEXR_SUCCESS = 0,
    TILEXR_ERROR_NOT_INITIALIZED = -1,
    TILEXR_ERROR_RUNTIME = -2,          // a CUDA runtime / driver call failed (reference: MKIRT)
    TILEXR_ERROR_PARA_CHECK_FAIL = -3,
    TILEXR_ERROR_INTERNAL = -4,
    TILEXR_ERROR_TIMEOUT = -5,
    TILEXR_ERROR_NOT_SUPPORT = -6,
    TILEXR_ERROR_NOT_FOUND = -7,
};
#define TILEXR_ERROR_MKIRT TILEXR_ERROR_RUNTIME

enum TileXRDataType {
    TILEXR_DATA_TYPE_INT8 = 0,
    TILEXR_DATA_TYPE_INT16 = 1,
    TILEXR_DATA_TYPE_INT32 = 2,
    TILEXR_DATA_TYPE_FP16 = 3,
    TILEXR_DATA_TYPE_FP32 = 4,
    TILEXR_DATA_TYPE_INT64 = 5,
    TILEXR_DATA_TYPE_UINT64 = 6,
    TILEXR_DATA_TYPE_UINT8 = 7,
    TILEXR_DATA_TYPE_UINT16 = 8,
    TILEXR_DATA_TYPE_UINT32 = 9,
    TILEXR_DATA_TYPE_FP64 = 10,
    TILEXR_DATA_TYPE_BFP16 = 11,
    TILEXR_DATA_TYPE_INT128 = 12,
    TILEXR_DATA_TYPE_HIF8 = 14,
    TILEXR_DATA_TYPE_FP8E4M3 = 15,
    TILEXR_DATA_TYPE_FP8E5M2 = 16,
    TILEXR_DATA_TYPE_FP8E8M0 = 17,
    TILEXR_DATA_TYPE_NVFP4 = 18,        // Blackwell addition, two e2m1 values per byte
    TILEXR_DATA_TYPE_RESERVED = 255
};

// What the ranks of a communicator are connected by, and what the device offers (reference: PhysicalInfo with chip
// name, physical link and core count, src/include/tilexr_types.h:90-94).
enum TileXRPhysicalLink {
    TILEXR_LINK_RESERVED = 0,
    TILEXR_LINK_NVLINK = 1,        // every peer is load / store / atomic reachable over NVLink (one NVSwitch hop on B200)
    TILEXR_LINK_PCIE = 2,          // peer access exists but without native atomics: PCIe peer-to-peer
    TILEXR_LINK_SAME_DEVICE = 3,   // all ranks share one GPU (emulated worlds) or there is one rank
    TILEXR_LINK_HOST_MEMORY = 4,   // CPU plumbing mode
};

struct TileXRPhysicalInfo {
    int32_t link;                  // TileXRPhysicalLink, the weakest over all peers
    int32_t ccMajor, ccMinor;      // compute capability (10.0 on B200)
    uint32_t smCount;              // streaming multiprocessors ("core count")
    uint32_t l2Bytes;
    uint64_t memoryBytes;
    int32_t p2pNativeAtomics;      // 1: atomics on peer memory are native on every link
    int32_t p2pPerformanceRank;    // the largest (worst) CUDA performance rank over the peers, 0 = best
    int32_t multicastSupported;    // the device can join NVLink multicast objects
    int32_t nvlsBound;             // this communicator's window is bound to one (in-switch reductions are in use)
    int32_t vmmWindow;             // the window was created with the virtual-memory API
};

enum TileXRReduceOp {
    TILEXR_REDUCE_SUM = 0,
    TILEXR_REDUCE_PROD = 1,
    TILEXR_REDUCE_MAX = 2,
    TILEXR_REDUCE_MIN = 3,
    TILEXR_REDUCE_RESERVED = 255
};

// Operator ids (values as in the reference's TileXRType, src/include/tilexr_types.h:96-126).  Ids >= 100 are the
// compute+collective fusions; the reference keeps only their names, this runtime implements PURE_MATMUL,
// ALL_GATHER_MATMUL and MATMUL_REDUCE_SCATTER (MATMUL_ALL_REDUCE is the latter followed by an all-gather:
// tilexr_b200.ops.gemm.matmul_all_reduce).  The all-to-all fusions from 105 on are identifiers only here as there.
enum TileXROpType {
    TILEXR_OP_ALL_REDUCE = 1,
    TILEXR_OP_REDUCE_SCATTER = 2,
    TILEXR_OP_ALL_GATHER = 3,
    TILEXR_OP_BROADCAST = 4,
    TILEXR_OP_ALL2ALL = 5,
    TILEXR_OP_ALL2ALL_V_C = 6,
    TILEXR_OP_GATHER = 7,
    TILEXR_OP_LOCAL_REDUCE = 8,
    TILEXR_OP_SEND = 9,
    TILEXR_OP_RECV = 10,
    TILEXR_OP_PROFILE_PROBE = 11,
    TILEXR_OP_ALL_REDUCE_RMSNORM = 12,  // all-reduce + residual add + RMSNorm
    TILEXR_OP_EP_DISPATCH = 20,
    TILEXR_OP_EP_COMBINE = 21,
    TILEXR_OP_MOONEP_PLANNING = 30,
    TILEXR_OP_MOONEP_DISPATCH = 31,
    TILEXR_OP_MOONEP_PREFETCH = 32,
    TILEXR_OP_MOONEP_COMBINE = 33,
    TILEXR_OP_MOONEP_REDUCE_GRAD = 34,
    TILEXR_OP_PURE_MATMUL = 101,
    TILEXR_OP_MATMUL_ALL_REDUCE = 102,
    TILEXR_OP_MATMUL_REDUCE_SCATTER = 103,
    TILEXR_OP_ALL_GATHER_MATMUL = 104,
    TILEXR_OP_ALL_GATHER_MATMUL_V2 = 105,
    TILEXR_OP_ALL2ALL_MATMUL = 106,
    TILEXR_OP_MATMUL_ALL2ALL = 107,
    TILEXR_OP_MTE2_TEST = 108,
    TILEXR_OP_ALL_GATHER_MATMUL_REDUCE_SCATTER = 111,
    TILEXR_OP_BANDWIDTH = 201,
    TILEXR_OP_ALLTOALLV_ALLGATHER_MATMUL = 305,
    TILEXR_OP_MATMUL_REDUCESCATTER_ALLTOALLV = 306,
    TILEXR_OP_ALLTOALLVC_ALLGATHER_MATMUL = 307,
    TILEXR_OP_MATMUL_REDUCESCATTER_ALLTOALLVC = 308,
    TILEXR_OP_ALLTOALLVC_ALLGATHER_MATMUL_HIDDEN = 309,
    TILEXR_OP_MATMUL_REDUCESCATTER_ALLTOALLVC_HIDDEN = 310,
    TILEXR_TYPE_MAX = 311,
};

static inline size_t TileXRDataTypeSize(int dtype)
{
    switch (dtype) {
        case TILEXR_DATA_TYPE_INT8: case TILEXR_DATA_TYPE_UINT8: case TILEXR_DATA_TYPE_HIF8:
        case TILEXR_DATA_TYPE_FP8E4M3: case TILEXR_DATA_TYPE_FP8E5M2: case TILEXR_DATA_TYPE_FP8E8M0:
            return 1;
        case TILEXR_DATA_TYPE_INT16: case TILEXR_DATA_TYPE_UINT16: case TILEXR_DATA_TYPE_FP16:
        case TILEXR_DATA_TYPE_BFP16:
            return 2;
        case TILEXR_DATA_TYPE_INT32: case TILEXR_DATA_TYPE_UINT32: case TILEXR_DATA_TYPE_FP32:
            return 4;
        case TILEXR_DATA_TYPE_INT64: case TILEXR_DATA_TYPE_UINT64: case TILEXR_DATA_TYPE_FP64:
            return 8;
        case TILEXR_DATA_TYPE_INT128:
            return 16;
        default:
            return 0;
    }
}

static inline const char *TileXROpName(int op)
{
    switch (op) {
        case TILEXR_OP_ALL_REDUCE: return "TileXRAllReduce";
        case TILEXR_OP_REDUCE_SCATTER: return "TileXRReduceScatter";
        case TILEXR_OP_ALL_GATHER: return "TileXRAllGather";
        case TILEXR_OP_BROADCAST: return "TileXRBroadcast";
        case TILEXR_OP_ALL2ALL: return "TileXRAll2All";
        case TILEXR_OP_ALL2ALL_V_C: return "TileXRAll2AllVC";
        case TILEXR_OP_GATHER: return "TileXRGather";
        case TILEXR_OP_LOCAL_REDUCE: return "TileXRLocalReduce";
        case TILEXR_OP_SEND: return "TileXRSend";
        case TILEXR_OP_RECV: return "TileXRRecv";
        case TILEXR_OP_PROFILE_PROBE: return "TileXRProfileProbe";
        case TILEXR_OP_ALL_REDUCE_RMSNORM: return "TileXRAllReduceRmsNorm";
        case TILEXR_OP_EP_DISPATCH: return "TileXRMoeEpDispatch";
        case TILEXR_OP_EP_COMBINE: return "TileXRMoeEpCombine";
        case TILEXR_OP_MOONEP_PLANNING: return "TileXRMoonEpPlanning";
        case TILEXR_OP_MOONEP_DISPATCH: return "TileXRMoonEpDispatch";
        case TILEXR_OP_MOONEP_PREFETCH: return "TileXRMoonEpPrefetchWeight";
        case TILEXR_OP_MOONEP_COMBINE: return "TileXRMoonEpCombine";
        case TILEXR_OP_MOONEP_REDUCE_GRAD: return "TileXRMoonEpReduceGrad";
        case TILEXR_OP_PURE_MATMUL: return "TileXRPureMatmul";
        case TILEXR_OP_MATMUL_ALL_REDUCE: return "TileXRMatmulAllReduce";
        case TILEXR_OP_MATMUL_REDUCE_SCATTER: return "TileXRMatmulReduceScatter";
        case TILEXR_OP_ALL_GATHER_MATMUL: return "TileXRAllGatherMatmul";
        case TILEXR_OP_ALL_GATHER_MATMUL_V2: return "TileXRAllGatherMatmulV2";
        case TILEXR_OP_ALL2ALL_MATMUL: return "TileXRAll2AllMatmul";
        case TILEXR_OP_MATMUL_ALL2ALL: return "TileXRMatmulAll2All";
        case TILEXR_OP_MTE2_TEST: return "TileXRMTE2Test";
        case TILEXR_OP_ALL_GATHER_MATMUL_REDUCE_SCATTER: return "TileXRAllGatherMatmulReduceScatter";
        case TILEXR_OP_ALLTOALLV_ALLGATHER_MATMUL: case TILEXR_OP_ALLTOALLVC_ALLGATHER_MATMUL:
        case TILEXR_OP_ALLTOALLVC_ALLGATHER_MATMUL_HIDDEN: return "TileXRAllToAllVAllGatherMatmul";
        case TILEXR_OP_MATMUL_REDUCESCATTER_ALLTOALLV: case TILEXR_OP_MATMUL_REDUCESCATTER_ALLTOALLVC:
        case TILEXR_OP_MATMUL_REDUCESCATTER_ALLTOALLVC_HIDDEN: return "TileXRMatmulReduceScatterAllToAllV";
        case TILEXR_OP_BANDWIDTH: return "TileXRBandwidthTest";
        default: return "TileXRUnknown";
    }
}

#ifdef __cplusplus
} // namespace TileXR
#endif

#endif // TILEXR_TYPES_H
