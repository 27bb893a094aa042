// PyTorch binding of the TileXR-B200 C API: a `Comm` class, tensor-level collectives and
// expert-parallel ops on the current CUDA stream, and `torch.ops.tilexr.*` registrations for
// the plain collectives.  The reference drives its libraries from Python through ctypes
// (integrations/moonep_torch/tilexr_moonep/abi.py, runtime.py); here the glue is compiled.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "tilexr_api.h"
#include "tilexr_collectives.h"
#include "tilexr_collectives_perf.h"
#include "tilexr_ep.h"
#include "tilexr_ep_plan.h"
#include "tilexr_launch.h"
#include "tilexr_extras.h"

namespace py = pybind11;

namespace {

void Check(int status, const char *what)
{
    if (status != TileXR::TILEXR_SUCCESS) {
        throw std::runtime_error(std::string(what) + " failed: " + TileXRGetErrorString(status) + " (" +
                                 std::to_string(status) + ")");
    }
}

TileXR::TileXRDataType ToDtype(at::ScalarType t)
{
    switch (t) {
        case at::kChar: return TileXR::TILEXR_DATA_TYPE_INT8;
        case at::kByte: return TileXR::TILEXR_DATA_TYPE_UINT8;
        case at::kBool: return TileXR::TILEXR_DATA_TYPE_UINT8;
        case at::kShort: return TileXR::TILEXR_DATA_TYPE_INT16;
        case at::kInt: return TileXR::TILEXR_DATA_TYPE_INT32;
        case at::kLong: return TileXR::TILEXR_DATA_TYPE_INT64;
        case at::kHalf: return TileXR::TILEXR_DATA_TYPE_FP16;
        case at::kBFloat16: return TileXR::TILEXR_DATA_TYPE_BFP16;
        case at::kFloat: return TileXR::TILEXR_DATA_TYPE_FP32;
        case at::kDouble: return TileXR::TILEXR_DATA_TYPE_FP64;
        case at::kFloat8_e4m3fn: return TileXR::TILEXR_DATA_TYPE_FP8E4M3;
        case at::kFloat8_e5m2: return TileXR::TILEXR_DATA_TYPE_FP8E5M2;
        default: throw std::runtime_error("unsupported tensor dtype for TileXR");
    }
}

void *StreamOf(const at::Tensor &t)
{
    if (!t.is_cuda()) return nullptr;
    return at::cuda::getCurrentCUDAStream(t.get_device()).stream();
}

void RequireContiguous(const at::Tensor &t, const char *name)
{
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// Launches on an emulated world are deferred until the group ends, so tensors handed to an op
// inside a group must outlive the call: they are parked here until group_end.
thread_local int g_groupDepth = 0;
thread_local std::vector<at::Tensor> g_groupKeep;

void Keep(const at::Tensor &t)
{
    if (g_groupDepth > 0 && t.defined()) g_groupKeep.push_back(t);
}
void Keep(const c10::optional<at::Tensor> &t)
{
    if (t.has_value()) Keep(*t);
}

// Exchange over a torch Store: every rank publishes its bytes under a per-call key.
struct StoreExchangeCtx {
    c10::intrusive_ptr<c10d::Store> store;
    std::string prefix;
    int rank;
    int rankSize;
    uint64_t call = 0;
};

int StoreAllGather(void *ctxPtr, const void *send, void *recv, size_t bytes)
{
    auto *ctx = static_cast<StoreExchangeCtx *>(ctxPtr);
    try {
        const std::string base = ctx->prefix + "/" + std::to_string(ctx->call++) + "/";
        const uint8_t *s = static_cast<const uint8_t *>(send);
        ctx->store->set(base + std::to_string(ctx->rank), std::vector<uint8_t>(s, s + bytes));
        for (int r = 0; r < ctx->rankSize; ++r) {
            const std::vector<uint8_t> v = ctx->store->get(base + std::to_string(r));
            if (v.size() != bytes) return TileXR::TILEXR_ERROR_INTERNAL;
            std::memcpy(static_cast<uint8_t *>(recv) + r * bytes, v.data(), bytes);
        }
    } catch (const std::exception &e) {
        fprintf(stderr, "[TileXR] store exchange failed: %s\n", e.what());
        return TileXR::TILEXR_ERROR_TIMEOUT;
    }
    return TileXR::TILEXR_SUCCESS;
}

class Comm {
public:
    Comm(TileXRCommPtr ptr, std::shared_ptr<StoreExchangeCtx> ctx) : ptr_(ptr), storeCtx_(std::move(ctx))
    {
        Check(TileXRCommGetInfo(ptr_, &rank_, &rankSize_, &device_, &dataHalfBytes_), "TileXRCommGetInfo");
    }
    ~Comm() { Destroy(); }
    void Destroy()
    {
        if (ptr_ != nullptr) {
            TileXRCommDestroy(ptr_);
            ptr_ = nullptr;
        }
    }
    TileXRCommPtr ptr() const
    {
        TORCH_CHECK(ptr_ != nullptr, "communicator was destroyed");
        return ptr_;
    }
    int rank() const { return rank_; }
    int rankSize() const { return rankSize_; }
    int device() const { return device_; }
    uint64_t dataHalfBytes() const { return dataHalfBytes_; }
    int64_t NextMagic()
    {
        int64_t m = 0;
        Check(TileXRCommNextMagic(ptr(), &m), "TileXRCommNextMagic");
        return m;
    }
    int DeviceStatus()
    {
        int s = 0;
        Check(TileXRCommGetDeviceStatus(ptr(), &s), "TileXRCommGetDeviceStatus");
        return s;
    }
    std::vector<int64_t> Dfx()
    {
        DeviceStatus();
        TileXRCommArgs *args = nullptr;
        Check(TileXRGetCommArgsHost(ptr(), &args), "TileXRGetCommArgsHost");
        return std::vector<int64_t>(args->dfx, args->dfx + TILEXR_DFX_COUNT);
    }
    uint32_t ExtraFlag()
    {
        TileXRCommArgs *args = nullptr;
        Check(TileXRGetCommArgsHost(ptr(), &args), "TileXRGetCommArgsHost");
        return args->extraFlag;
    }
    void ResetStatus() { Check(TileXRCommResetStatus(ptr()), "TileXRCommResetStatus"); }
    void SetWaitTimeoutMs(uint64_t ms) { Check(TileXRCommSetWaitTimeoutMs(ptr(), ms), "TileXRCommSetWaitTimeoutMs"); }
    void PrintDfx() { TileXRPrintDFX2Log(ptr()); }
    void Barrier() { Check(TileXRCommHostBarrier(ptr()), "TileXRCommHostBarrier"); }

    // A tensor in peer-visible memory: every rank calls this with the same shape.
    at::Tensor SymmEmpty(std::vector<int64_t> shape, at::ScalarType dtype)
    {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        const size_t bytes = static_cast<size_t>(std::max<int64_t>(n, 1)) * c10::elementSize(dtype);
        void *p = nullptr;
        TileXRUDMAMemHandle handle = 0;
        Check(TileXRSymmAlloc(ptr(), bytes, &p, &handle), "TileXRSymmAlloc");
        // The allocation belongs to the communicator (freed by symm_free or at destroy).
        auto options = at::TensorOptions().dtype(dtype).device(at::kCUDA, device_);
        at::Tensor t = at::from_blob(p, shape, [](void *) {}, options);
        symmHandles_.emplace_back(p, handle);
        return t;
    }
    void SymmFree(const at::Tensor &t)
    {
        for (auto it = symmHandles_.begin(); it != symmHandles_.end(); ++it) {
            if (it->first == t.data_ptr()) {
                Check(TileXRSymmFree(ptr(), it->second), "TileXRSymmFree");
                symmHandles_.erase(it);
                return;
            }
        }
        throw std::runtime_error("tensor was not allocated by symm_empty on this communicator");
    }
    uint32_t Register(const at::Tensor &t)
    {
        TileXRUDMAMemHandle h = 0;
        Check(TileXRUDMARegister(ptr(), static_cast<GM_ADDR>(t.data_ptr()), t.nbytes(), &h), "TileXRUDMARegister");
        return h;
    }
    void Unregister(uint32_t h) { Check(TileXRUDMAUnregister(ptr(), h), "TileXRUDMAUnregister"); }
    std::vector<uint64_t> PeerPointers(uint32_t h)
    {
        std::vector<void *> p(rankSize_);
        Check(TileXRGetPeerPointers(ptr(), h, p.data()), "TileXRGetPeerPointers");
        std::vector<uint64_t> out;
        for (void *q : p) out.push_back(reinterpret_cast<uint64_t>(q));
        return out;
    }
    uint64_t MulticastPtr(const at::Tensor &t)
    {
        void *mc = nullptr;
        const int ret = TileXRGetMulticastPointer(ptr(), t.data_ptr(), t.nbytes(), &mc);
        if (ret == TileXR::TILEXR_ERROR_NOT_FOUND) return 0;
        Check(ret, "TileXRGetMulticastPointer");
        return reinterpret_cast<uint64_t>(mc);
    }
    bool NvlsAvailable() { return TileXRNvlsAvailable(ptr()) != 0; }
    bool IsRegistered(const at::Tensor &t)
    {
        return TileXRFindRegistration(ptr(), t.data_ptr(), t.nbytes(), nullptr, nullptr) == TileXR::TILEXR_SUCCESS;
    }

private:
    TileXRCommPtr ptr_;
    std::shared_ptr<StoreExchangeCtx> storeCtx_;
    int rank_ = 0, rankSize_ = 0, device_ = -1;
    uint64_t dataHalfBytes_ = 0;
    std::vector<std::pair<void *, TileXRUDMAMemHandle>> symmHandles_;
};

using CommPtr = std::shared_ptr<Comm>;

CommPtr InitProcess(int rank, int rankSize, const std::string &commId, int domain, int bufferMB, int device)
{
    if (!commId.empty()) setenv("TILEXR_COMM_ID", commId.c_str(), 1);
    if (device >= 0) C10_CUDA_CHECK(cudaSetDevice(device));
    TileXRCommPtr p = nullptr;
    Check(TileXRCommInitRankWithCustDomainSize(domain, bufferMB > 0 ? bufferMB : TILEXR_COMM_BUFFER_SIZE_MB, rankSize, rank, &p),
          "TileXRCommInitRankWithCustDomainSize");
    return std::make_shared<Comm>(p, nullptr);
}

CommPtr InitWithStore(c10::intrusive_ptr<c10d::Store> store, const std::string &prefix, int rank, int rankSize, int domain,
                      int bufferMB, int device, bool hostMemory)
{
    if (device >= 0 && !hostMemory) C10_CUDA_CHECK(cudaSetDevice(device));
    auto ctx = std::make_shared<StoreExchangeCtx>();
    ctx->store = std::move(store);
    ctx->prefix = prefix;
    ctx->rank = rank;
    ctx->rankSize = rankSize;
    TileXRCommPtr p = nullptr;
    if (hostMemory) {
        Check(TileXRCommInitRankHostMemoryWithExchange(StoreAllGather, ctx.get(), domain, bufferMB, rankSize, rank, &p),
              "TileXRCommInitRankHostMemoryWithExchange");
    } else {
        Check(TileXRCommInitRankWithExchange(StoreAllGather, ctx.get(), domain, bufferMB, rankSize, rank, &p),
              "TileXRCommInitRankWithExchange");
    }
    return std::make_shared<Comm>(p, ctx);
}

CommPtr InitHostMemory(int rank, int rankSize, const std::string &commId, int domain, int bufferMB)
{
    if (!commId.empty()) setenv("TILEXR_COMM_ID", commId.c_str(), 1);
    TileXRCommPtr p = nullptr;
    Check(TileXRCommInitRankHostMemory(domain, bufferMB, rankSize, rank, &p), "TileXRCommInitRankHostMemory");
    return std::make_shared<Comm>(p, nullptr);
}

std::vector<CommPtr> InitEmulated(int rankSize, int device, int bufferMB)
{
    std::vector<TileXRCommPtr> raw(rankSize, nullptr);
    Check(TileXRCommInitEmulated(static_cast<uint32_t>(rankSize), device, bufferMB, raw.data()), "TileXRCommInitEmulated");
    std::vector<CommPtr> out;
    for (TileXRCommPtr p : raw) out.push_back(std::make_shared<Comm>(p, nullptr));
    return out;
}

// ---- collectives -------------------------------------------------------------------------------------------

void AllGather(const CommPtr &c, const at::Tensor &in, at::Tensor out)
{
    RequireContiguous(in, "input");
    RequireContiguous(out, "output");
    Keep(in);
    Keep(out);
    TORCH_CHECK(out.numel() == in.numel() * c->rankSize() && out.scalar_type() == in.scalar_type(), "all_gather: bad output");
    Check(TileXRAllGather(in.data_ptr(), out.data_ptr(), in.numel(), ToDtype(in.scalar_type()), c->ptr(), StreamOf(in)),
          "TileXRAllGather");
}

void AllToAll(const CommPtr &c, const at::Tensor &in, at::Tensor out)
{
    RequireContiguous(in, "input");
    RequireContiguous(out, "output");
    Keep(in);
    Keep(out);
    TORCH_CHECK(out.numel() == in.numel() && in.numel() % c->rankSize() == 0 && out.scalar_type() == in.scalar_type(),
                "all_to_all: sizes must match and divide by the rank count");
    Check(TileXRAllToAll(in.data_ptr(), out.data_ptr(), in.numel() / c->rankSize(), ToDtype(in.scalar_type()), c->ptr(),
                         StreamOf(in)),
          "TileXRAllToAll");
}

void AllReduce(const CommPtr &c, const at::Tensor &in, at::Tensor out, int op)
{
    RequireContiguous(in, "input");
    RequireContiguous(out, "output");
    Keep(in);
    Keep(out);
    TORCH_CHECK(out.numel() == in.numel() && out.scalar_type() == in.scalar_type(), "all_reduce: bad output");
    Check(TileXRAllReduce(in.data_ptr(), out.data_ptr(), in.numel(), ToDtype(in.scalar_type()),
                          static_cast<TileXR::TileXRReduceOp>(op), c->ptr(), StreamOf(in)),
          "TileXRAllReduce");
}

void ReduceScatter(const CommPtr &c, const at::Tensor &in, at::Tensor out, int op)
{
    RequireContiguous(in, "input");
    RequireContiguous(out, "output");
    Keep(in);
    Keep(out);
    TORCH_CHECK(in.numel() == out.numel() * c->rankSize() && out.scalar_type() == in.scalar_type(), "reduce_scatter: bad output");
    Check(TileXRReduceScatter(in.data_ptr(), out.data_ptr(), out.numel(), ToDtype(in.scalar_type()),
                              static_cast<TileXR::TileXRReduceOp>(op), c->ptr(), StreamOf(in)),
          "TileXRReduceScatter");
}

void Broadcast(const CommPtr &c, at::Tensor buf, int root)
{
    RequireContiguous(buf, "buffer");
    Keep(buf);
    Check(TileXRBroadcast(buf.data_ptr(), buf.numel(), ToDtype(buf.scalar_type()), root, c->ptr(), StreamOf(buf)),
          "TileXRBroadcast");
}

void ProfileProbe(const CommPtr &c, const at::Tensor &in, at::Tensor out)
{
    RequireContiguous(in, "input");
    RequireContiguous(out, "output");
    Keep(in);
    Keep(out);
    TORCH_CHECK(out.nbytes() >= in.nbytes(), "profile_probe: output too small");
    Check(TileXRProfileProbe(in.data_ptr(), out.data_ptr(), in.numel(), ToDtype(in.scalar_type()), c->ptr(), StreamOf(in)),
          "TileXRProfileProbe");
}

py::dict CollectivePlan(int opType, int64_t count, at::ScalarType dtype, int rankSize, uint64_t dataHalfBytes, unsigned maxGrid)
{
    TileXRCollPlanInfo info;
    Check(TileXRCollectivePlan(opType, count, ToDtype(dtype), rankSize, dataHalfBytes, maxGrid, &info), "TileXRCollectivePlan");
    py::dict d;
    d["kind"] = info.kind;
    d["launches"] = info.launches;
    d["tile_bytes"] = info.tileBytes;
    d["tiles_per_launch"] = info.tilesPerLaunch;
    d["producers"] = info.producers;
    d["reducers"] = info.reducers;
    d["consumers"] = info.consumers;
    d["grid"] = info.grid;
    d["bytes_per_launch"] = info.bytesPerLaunch;
    return d;
}

// ---- expert parallel -------------------------------------------------------------------------------------------

const void *PtrOrNull(const c10::optional<at::Tensor> &t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// Returns (expand_x, dynamic_scales|None, assist, expert_token_nums, send_counts, recv_total, topk_ids, topk_weights,
// route_rows, assist_ext, expand_scales).
py::tuple EpDispatch(const CommPtr &c, const at::Tensor &x, const c10::optional<at::Tensor> &expertIds,
                     const c10::optional<at::Tensor> &gateLogits, const c10::optional<at::Tensor> &selectionBias,
                     const c10::optional<at::Tensor> &activeMask, int64_t topK, int64_t numExperts, int64_t quantMode,
                     int64_t scoreFunc, bool renormalize, double routedScale, int64_t tokenNumsType, int64_t maxRecvRows,
                     const c10::optional<at::Tensor> &expandXOut, const c10::optional<at::Tensor> &expertScales, bool dedup,
                     const c10::optional<at::Tensor> &quantScales, int64_t sharedExpertNum, int64_t sharedExpertRankNum,
                     int64_t tpWorldSize)
{
    RequireContiguous(x, "x");
    const int64_t T = tpWorldSize > 1 ? tpWorldSize : 1;
    Keep(expertScales);
    Keep(quantScales);
    TORCH_CHECK(x.dim() == 2 && x.is_cuda(), "x must be a 2-D CUDA tensor");
    Keep(x);
    Keep(expertIds);
    Keep(gateLogits);
    Keep(selectionBias);
    Keep(activeMask);
    const int64_t bs = x.size(0), h = x.size(1);
    const int R = c->rankSize();
    TORCH_CHECK(sharedExpertRankNum >= 0 && sharedExpertRankNum < R, "shared_expert_rank_num must leave ranks for the routed experts");
    TORCH_CHECK(R % T == 0, "tp_world_size must divide the number of ranks");
    const int64_t localExperts = c->rank() < sharedExpertRankNum ? 1 : numExperts / (R / T - sharedExpertRankNum);
    auto i32 = x.options().dtype(at::kInt);
    const bool mx = quantMode == TileXREp::TILEXR_EP_QUANT_MXFP8_E4M3 || quantMode == TileXREp::TILEXR_EP_QUANT_MXFP8_E5M2;
    const bool int8 = quantMode == TileXREp::TILEXR_EP_QUANT_STATIC_INT8 || quantMode == TileXREp::TILEXR_EP_QUANT_DYNAMIC_INT8;
    const bool quant = mx || int8 || quantMode == TileXREp::TILEXR_EP_QUANT_FP8_1X128;
    const at::ScalarType qType = int8 ? at::kChar
                                 : quantMode == TileXREp::TILEXR_EP_QUANT_MXFP8_E5M2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn;
    at::Tensor expandX = expandXOut.has_value() && expandXOut->defined()
                             ? *expandXOut
                             : at::empty({maxRecvRows, h}, x.options().dtype(quant ? qType : x.scalar_type()));
    TORCH_CHECK(expandX.is_contiguous() && expandX.size(0) >= maxRecvRows && expandX.size(1) == h, "bad expand_x_out");
    const bool hasScales = quant && quantMode != TileXREp::TILEXR_EP_QUANT_STATIC_INT8;
    at::Tensor scales = mx                                                      ? at::empty({maxRecvRows, h / 32}, x.options().dtype(at::kByte))
                        : quantMode == TileXREp::TILEXR_EP_QUANT_DYNAMIC_INT8 ? at::empty({maxRecvRows}, x.options().dtype(at::kFloat))
                        : hasScales                                            ? at::empty({maxRecvRows, h / 128}, x.options().dtype(at::kFloat))
                                                                               : at::Tensor();
    at::Tensor assist = at::empty({maxRecvRows, 4}, i32);
    at::Tensor tokenNums = at::empty({localExperts}, x.options().dtype(at::kLong));
    at::Tensor sendCounts = at::empty({localExperts * R}, i32);
    at::Tensor recvTotal = at::empty({1}, i32);
    at::Tensor topkIds = at::empty({bs, topK}, i32);
    at::Tensor topkWeights = at::empty({bs, topK}, x.options().dtype(at::kFloat));
    at::Tensor routeRows = at::empty({bs, topK * T + sharedExpertNum}, i32);
    at::Tensor assistExt = at::empty({maxRecvRows, 2}, i32);
    at::Tensor expandScales = at::empty({maxRecvRows}, x.options().dtype(at::kFloat));
    at::Tensor tpRecvCounts = at::zeros({T}, i32);
    TileXREpDispatchParams p;
    std::memset(&p, 0, sizeof(p));
    p.tpWorldSize = T;
    p.tpRankId = c->rank() % T;
    p.tpRecvCountsOut = T > 1 ? tpRecvCounts.data_ptr<int32_t>() : nullptr;
    p.x = x.data_ptr();
    if (expertIds.has_value() && expertIds->defined()) {
        TORCH_CHECK(expertIds->scalar_type() == at::kInt && expertIds->is_contiguous(), "expert_ids must be contiguous int32");
        p.expertIds = expertIds->data_ptr<int32_t>();
    }
    if (gateLogits.has_value() && gateLogits->defined()) {
        TORCH_CHECK(gateLogits->scalar_type() == at::kFloat && gateLogits->is_contiguous(), "gate_logits must be contiguous fp32");
        p.gateLogits = gateLogits->data_ptr<float>();
    }
    p.selectionBias = static_cast<const float *>(PtrOrNull(selectionBias));
    if (activeMask.has_value() && activeMask->defined()) {
        TORCH_CHECK(activeMask->scalar_type() == at::kBool && activeMask->is_contiguous(), "active mask must be contiguous bool");
        p.xActiveMask = activeMask->data_ptr<bool>();
        p.activeMaskType = activeMask->dim() == 1 ? TileXREp::TILEXR_EP_ACTIVE_MASK_TOKEN : TileXREp::TILEXR_EP_ACTIVE_MASK_EXPERT;
    }
    p.bs = bs;
    p.h = h;
    p.topK = topK;
    p.moeExpertNum = numExperts;
    p.quantMode = quantMode;
    p.scoreFunc = scoreFunc;
    p.renormalize = renormalize ? 1 : 0;
    p.routedScalingFactor = static_cast<float>(routedScale);
    p.expertTokenNumsType = tokenNumsType;
    p.maxRecvRows = maxRecvRows;
    p.topkIdsOut = topkIds.data_ptr<int32_t>();
    p.topkWeightsOut = topkWeights.data_ptr<float>();
    p.expandXOut = expandX.data_ptr();
    p.dynamicScalesOut = hasScales ? static_cast<float *>(scales.data_ptr()) : nullptr;
    if (quantScales.has_value() && quantScales->defined()) {
        TORCH_CHECK(quantScales->scalar_type() == at::kFloat && quantScales->is_contiguous() && quantScales->numel() == numExperts * h,
                    "scales must be contiguous fp32 [num_experts, h]");
        p.scales = quantScales->data_ptr<float>();
    }
    p.assistInfoForCombineOut = assist.data_ptr<int32_t>();
    p.expertTokenNumsOut = tokenNums.data_ptr<int64_t>();
    p.sendCountsOut = sendCounts.data_ptr<int32_t>();
    p.recvTotalOut = recvTotal.data_ptr<int32_t>();
    p.routeRowsOut = routeRows.data_ptr<int32_t>();
    p.assistExtOut = assistExt.data_ptr<int32_t>();
    p.expandScalesOut = expandScales.data_ptr<float>();
    if (expertScales.has_value() && expertScales->defined()) {
        TORCH_CHECK(expertScales->scalar_type() == at::kFloat && expertScales->is_contiguous() && expertScales->numel() == bs * topK,
                    "expert_scales must be contiguous fp32 [bs, top_k]");
        p.expertScales = expertScales->data_ptr<float>();
    }
    p.dedup = dedup ? 1 : 0;
    p.sharedExpertNum = sharedExpertNum;
    p.sharedExpertRankNum = sharedExpertRankNum;
    p.dtype = ToDtype(x.scalar_type());
    for (const at::Tensor &t : {expandX, scales, assist, tokenNums, sendCounts, recvTotal, topkIds, topkWeights, routeRows,
                                assistExt, expandScales, tpRecvCounts}) {
        Keep(t);
    }
    Check(TileXRMoeEpDispatchFused(&p, c->ptr(), StreamOf(x)), "TileXRMoeEpDispatchFused");
    return py::make_tuple(expandX, hasScales ? py::cast(scales) : py::none(), assist, tokenNums, sendCounts, recvTotal, topkIds,
                          topkWeights, routeRows, assistExt, expandScales, tpRecvCounts);
}

at::Tensor EpCombine(const CommPtr &c, const at::Tensor &expertOut, const at::Tensor &assist, const at::Tensor &sendCounts,
                     const c10::optional<at::Tensor> &expertIds, const c10::optional<at::Tensor> &expertScales,
                     const c10::optional<at::Tensor> &activeMask, const c10::optional<at::Tensor> &sharedExpertX, int64_t bs,
                     int64_t topK, int64_t numExperts, const c10::optional<at::Tensor> &yOut,
                     const c10::optional<at::Tensor> &routeRows, const c10::optional<at::Tensor> &assistExt, bool dedup,
                     int64_t sharedExpertNum, int64_t sharedExpertRankNum, int64_t tpWorldSize)
{
    const int64_t T = tpWorldSize > 1 ? tpWorldSize : 1;
    Keep(assistExt);
    RequireContiguous(expertOut, "expert_out");
    Keep(routeRows);
    TORCH_CHECK(expertOut.dim() == 2 && expertOut.is_cuda(), "expert_out must be a 2-D CUDA tensor");
    Keep(expertOut);
    Keep(assist);
    Keep(sendCounts);
    Keep(expertIds);
    Keep(expertScales);
    Keep(activeMask);
    Keep(sharedExpertX);
    const int64_t h = expertOut.size(1);
    at::Tensor y = yOut.has_value() && yOut->defined() ? *yOut : at::empty({bs, h}, expertOut.options());
    TileXREpCombineParams p;
    std::memset(&p, 0, sizeof(p));
    p.expertOut = expertOut.data_ptr();
    p.assistInfoForCombine = assist.data_ptr<int32_t>();
    p.sendCounts = sendCounts.data_ptr<int32_t>();
    p.expertIds = static_cast<const int32_t *>(PtrOrNull(expertIds));
    p.expertScales = static_cast<const float *>(PtrOrNull(expertScales));
    if (activeMask.has_value() && activeMask->defined()) {
        p.xActiveMask = activeMask->data_ptr<bool>();
        p.activeMaskType = activeMask->dim() == 1 ? TileXREp::TILEXR_EP_ACTIVE_MASK_TOKEN : TileXREp::TILEXR_EP_ACTIVE_MASK_EXPERT;
    }
    p.sharedExpertX = PtrOrNull(sharedExpertX);
    if (routeRows.has_value() && routeRows->defined()) {
        TORCH_CHECK(routeRows->scalar_type() == at::kInt && routeRows->is_contiguous() &&
                        routeRows->numel() == bs * (topK * T + sharedExpertNum),
                    "route_rows must be contiguous int32 [bs, top_k * tp_world_size + shared_expert_num]");
        p.routeRows = routeRows->data_ptr<int32_t>();
    }
    if (assistExt.has_value() && assistExt->defined()) {
        TORCH_CHECK(assistExt->scalar_type() == at::kInt && assistExt->is_contiguous(), "assist_ext must be contiguous int32");
        p.assistExt = assistExt->data_ptr<int32_t>();
    }
    p.dedup = dedup ? 1 : 0;
    p.sharedExpertNum = sharedExpertNum;
    p.sharedExpertRankNum = sharedExpertRankNum;
    p.tpWorldSize = T;
    p.tpRankId = c->rank() % T;
    p.bs = bs;
    p.h = h;
    p.topK = topK;
    p.moeExpertNum = numExperts;
    p.yOut = y.data_ptr();
    p.dtype = ToDtype(expertOut.scalar_type());
    Keep(y);
    Check(TileXRMoeEpCombineFused(&p, c->ptr(), StreamOf(expertOut)), "TileXRMoeEpCombineFused");
    return y;
}

py::tuple RoutingTopK(const at::Tensor &logits, const c10::optional<at::Tensor> &bias, int64_t topK, int64_t scoreFunc,
                      bool renormalize, double routedScale)
{
    TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kFloat && logits.is_contiguous(),
                "gate logits must be a contiguous 2-D fp32 CUDA tensor");
    at::Tensor ids = at::empty({logits.size(0), topK}, logits.options().dtype(at::kInt));
    at::Tensor weights = at::empty({logits.size(0), topK}, logits.options());
    Check(TileXRMoeRoutingTopK(logits.data_ptr<float>(), static_cast<const float *>(PtrOrNull(bias)), logits.size(0),
                               logits.size(1), topK, scoreFunc, renormalize ? 1 : 0, static_cast<float>(routedScale),
                               ids.data_ptr<int32_t>(), weights.data_ptr<float>(), StreamOf(logits)),
          "TileXRMoeRoutingTopK");
    return py::make_tuple(ids, weights);
}

py::tuple Fp8Quant(const at::Tensor &x)
{
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "x must be a contiguous 2-D CUDA tensor");
    at::Tensor y = at::empty(x.sizes(), x.options().dtype(at::kFloat8_e4m3fn));
    at::Tensor s = at::empty({x.size(0), x.size(1) / 128}, x.options().dtype(at::kFloat));
    Check(TileXRFp8Quant1x128(x.data_ptr(), x.size(0), x.size(1), ToDtype(x.scalar_type()), y.data_ptr(), s.data_ptr<float>(),
                              StreamOf(x)),
          "TileXRFp8Quant1x128");
    return py::make_tuple(y, s);
}

at::Tensor Fp8Dequant(const at::Tensor &y, const at::Tensor &scales, at::ScalarType dtype)
{
    TORCH_CHECK(y.is_cuda() && y.dim() == 2 && y.is_contiguous() && scales.is_contiguous(), "bad fp8 input");
    at::Tensor x = at::empty(y.sizes(), y.options().dtype(dtype));
    Check(TileXRFp8Dequant1x128(y.data_ptr(), scales.data_ptr<float>(), y.size(0), y.size(1), ToDtype(dtype), x.data_ptr(),
                                StreamOf(y)),
          "TileXRFp8Dequant1x128");
    return x;
}

py::tuple Mxfp8Quant(const at::Tensor &x, bool e5m2)
{
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "x must be a contiguous 2-D CUDA tensor");
    at::Tensor y = at::empty(x.sizes(), x.options().dtype(e5m2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn));
    at::Tensor s = at::empty({x.size(0), (x.size(1) + 31) / 32}, x.options().dtype(at::kByte));
    Check(TileXRMxfp8Quant(x.data_ptr(), x.size(0), x.size(1), ToDtype(x.scalar_type()),
                           e5m2 ? TileXR::TILEXR_DATA_TYPE_FP8E5M2 : TileXR::TILEXR_DATA_TYPE_FP8E4M3, y.data_ptr(),
                           s.data_ptr<uint8_t>(), StreamOf(x)),
          "TileXRMxfp8Quant");
    return py::make_tuple(y, s);
}

at::Tensor Mxfp8Dequant(const at::Tensor &y, const at::Tensor &scales, at::ScalarType dtype)
{
    at::Tensor x = at::empty(y.sizes(), y.options().dtype(dtype));
    const bool e5m2 = y.scalar_type() == at::kFloat8_e5m2;
    Check(TileXRMxfp8Dequant(y.data_ptr(), scales.data_ptr<uint8_t>(), y.size(0), y.size(1),
                             e5m2 ? TileXR::TILEXR_DATA_TYPE_FP8E5M2 : TileXR::TILEXR_DATA_TYPE_FP8E4M3, ToDtype(dtype),
                             x.data_ptr(), StreamOf(y)),
          "TileXRMxfp8Dequant");
    return x;
}

at::Tensor RmsNorm(const at::Tensor &x, const c10::optional<at::Tensor> &residual, const at::Tensor &gamma, double eps)
{
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && gamma.is_contiguous(), "bad rmsnorm input");
    at::Tensor y = at::empty_like(x);
    void *res = residual.has_value() && residual->defined() ? residual->data_ptr() : nullptr;
    Check(TileXRRmsNorm(x.data_ptr(), res, gamma.data_ptr(), static_cast<float>(eps), x.size(0), x.size(1),
                        ToDtype(x.scalar_type()), y.data_ptr(), StreamOf(x)),
          "TileXRRmsNorm");
    return y;
}

// ---- perf sessions ------------------------------------------------------------------------------------------------

struct PerfSession {
    TileXRCollectivePerfSession s = nullptr;
    std::string dir, cmd;
};

std::shared_ptr<PerfSession> PerfCreate(const std::string &dir, unsigned sampleEveryN, bool aiPrompt, const std::string &aiCommand)
{
    auto ps = std::make_shared<PerfSession>();
    ps->dir = dir;
    ps->cmd = aiCommand;
    TileXRCollectivePerfConfig cfg{1, ps->dir.c_str(), sampleEveryN, aiPrompt ? 1 : 0, ps->cmd.c_str()};
    Check(TileXRCollectivePerfSessionCreate(&cfg, &ps->s), "TileXRCollectivePerfSessionCreate");
    return ps;
}

} // namespace

#include "binding_extras.inc"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.doc() = "TileXR-B200 native binding";
    TORCH_CHECK(TileXREpAbiStamp() == TILEXR_EP_ABI_STAMP,
                "tilexr_b200._C was built against other headers than libtilexr.so; run python -m tilexr_b200._build");
    py::class_<Comm, CommPtr>(m, "Comm")
        .def_property_readonly("rank", &Comm::rank)
        .def_property_readonly("world_size", &Comm::rankSize)
        .def_property_readonly("device", &Comm::device)
        .def_property_readonly("data_half_bytes", &Comm::dataHalfBytes)
        .def_property_readonly("extra_flag", &Comm::ExtraFlag)
        .def_property_readonly("handle", [](const Comm &c) { return reinterpret_cast<uint64_t>(c.ptr()); })
        .def("next_magic", &Comm::NextMagic)
        .def("device_status", &Comm::DeviceStatus)
        .def("dfx", &Comm::Dfx)
        .def("reset_status", &Comm::ResetStatus)
        .def("set_wait_timeout_ms", &Comm::SetWaitTimeoutMs)
        .def("print_dfx", &Comm::PrintDfx)
        .def("barrier", &Comm::Barrier)
        .def("symm_empty", &Comm::SymmEmpty)
        .def("symm_free", &Comm::SymmFree)
        .def("register", &Comm::Register)
        .def("unregister", &Comm::Unregister)
        .def("peer_pointers", &Comm::PeerPointers)
        .def("is_registered", &Comm::IsRegistered)
        .def("multicast_ptr", &Comm::MulticastPtr)
        .def("nvls_available", &Comm::NvlsAvailable)
        .def("physical_info", [](const Comm &c) {
            TileXRPhysicalInfoT ph{};
            Check(TileXRGetPhysicalInfo(c.ptr(), &ph), "TileXRGetPhysicalInfo");
            static const char *links[] = {"reserved", "nvlink", "pcie", "same_device", "host_memory"};
            py::dict d;
            d["link"] = links[ph.link >= 0 && ph.link <= 4 ? ph.link : 0];
            d["compute_capability"] = py::make_tuple(ph.ccMajor, ph.ccMinor);
            d["sm_count"] = ph.smCount;
            d["l2_bytes"] = ph.l2Bytes;
            d["memory_bytes"] = ph.memoryBytes;
            d["p2p_native_atomics"] = ph.p2pNativeAtomics != 0;
            d["p2p_performance_rank"] = ph.p2pPerformanceRank;
            d["multicast_supported"] = ph.multicastSupported != 0;
            d["nvls_bound"] = ph.nvlsBound != 0;
            d["vmm_window"] = ph.vmmWindow != 0;
            return d;
        })
        .def("destroy", &Comm::Destroy);
    m.def("init_process", &InitProcess, py::arg("rank"), py::arg("world_size"), py::arg("comm_id") = "", py::arg("domain") = 0,
          py::arg("buffer_mb") = 0, py::arg("device") = -1);
    m.def("init_with_store", &InitWithStore, py::arg("store"), py::arg("prefix"), py::arg("rank"), py::arg("world_size"),
          py::arg("domain") = 0, py::arg("buffer_mb") = 0, py::arg("device") = -1, py::arg("host_memory") = false);
    m.def("init_host_memory", &InitHostMemory, py::arg("rank"), py::arg("world_size"), py::arg("comm_id") = "",
          py::arg("domain") = 0, py::arg("buffer_mb") = 64);
    m.def("init_emulated", &InitEmulated, py::arg("world_size"), py::arg("device") = 0, py::arg("buffer_mb") = 64);
    m.def("group_start", [] {
        Check(TileXRGroupStart(), "TileXRGroupStart");
        g_groupDepth += 1;
    });
    m.def("group_end", [] {
        if (g_groupDepth > 0) g_groupDepth -= 1;
        const int status = TileXRGroupEnd();
        if (g_groupDepth == 0) g_groupKeep.clear();   // the launches are enqueued: stream order protects the memory now
        Check(status, "TileXRGroupEnd");
    });
    m.def("launch_count", [] { return TileXR::LaunchCount(); });
    m.def("all_gather", &AllGather);
    m.def("all_to_all", &AllToAll);
    m.def("all_reduce", &AllReduce, py::arg("comm"), py::arg("input"), py::arg("output"), py::arg("op") = 0);
    m.def("reduce_scatter", &ReduceScatter, py::arg("comm"), py::arg("input"), py::arg("output"), py::arg("op") = 0);
    m.def("broadcast", &Broadcast);
    m.def("profile_probe", &ProfileProbe);
    m.def("collective_plan", &CollectivePlan);
    m.def("ep_dispatch", &EpDispatch, py::arg("comm"), py::arg("x"), py::arg("expert_ids") = py::none(),
          py::arg("gate_logits") = py::none(), py::arg("selection_bias") = py::none(), py::arg("active_mask") = py::none(),
          py::arg("top_k") = 1, py::arg("num_experts") = 1, py::arg("quant_mode") = 0, py::arg("score_func") = 0,
          py::arg("renormalize") = true, py::arg("routed_scale") = 1.0, py::arg("token_nums_type") = 1,
          py::arg("max_recv_rows") = 0, py::arg("expand_x_out") = py::none(), py::arg("expert_scales") = py::none(),
          py::arg("dedup") = false, py::arg("scales") = py::none(), py::arg("shared_expert_num") = 0,
          py::arg("shared_expert_rank_num") = 0, py::arg("tp_world_size") = 1);
    m.def("ep_combine", &EpCombine, py::arg("comm"), py::arg("expert_out"), py::arg("assist"), py::arg("send_counts"),
          py::arg("expert_ids") = py::none(), py::arg("expert_scales") = py::none(), py::arg("active_mask") = py::none(),
          py::arg("shared_expert_x") = py::none(), py::arg("bs") = 0, py::arg("top_k") = 1, py::arg("num_experts") = 1,
          py::arg("y_out") = py::none(), py::arg("route_rows") = py::none(), py::arg("assist_ext") = py::none(),
          py::arg("dedup") = false, py::arg("shared_expert_num") = 0, py::arg("shared_expert_rank_num") = 0,
          py::arg("tp_world_size") = 1);
    m.def("routing_topk", &RoutingTopK, py::arg("gate_logits"), py::arg("selection_bias") = py::none(), py::arg("top_k") = 1,
          py::arg("score_func") = 0, py::arg("renormalize") = true, py::arg("routed_scale") = 1.0);
    m.def("fp8_quant_1x128", &Fp8Quant);
    m.def("fp8_dequant_1x128", &Fp8Dequant);
    m.def("mxfp8_quant", &Mxfp8Quant, py::arg("x"), py::arg("e5m2") = false);
    m.def("mxfp8_dequant", &Mxfp8Dequant);
    m.def("rmsnorm", &RmsNorm, py::arg("x"), py::arg("residual") = py::none(), py::arg("gamma"), py::arg("eps") = 1e-6);
    py::class_<PerfSession, std::shared_ptr<PerfSession>>(m, "PerfSession")
        .def("activate", [](PerfSession &p) { Check(TileXRCollectivePerfSetActiveSession(p.s), "SetActiveSession"); })
        .def("deactivate", [](PerfSession &) { Check(TileXRCollectivePerfSetActiveSession(nullptr), "SetActiveSession"); })
        .def("write_report", [](PerfSession &p) { Check(TileXRCollectivePerfWriteReport(p.s), "WriteReport"); })
        .def("write_incomplete_report",
             [](PerfSession &p, const std::string &why) { Check(TileXRCollectivePerfWriteIncompleteReport(p.s, why.c_str()), "WriteIncompleteReport"); })
        .def("destroy", [](PerfSession &p) {
            if (p.s != nullptr) TileXRCollectivePerfSessionDestroy(p.s);
            p.s = nullptr;
        });
    m.def("perf_session_create", &PerfCreate, py::arg("output_dir"), py::arg("sample_every_n") = 1, py::arg("ai_prompt") = false,
          py::arg("ai_command") = "");
    BindExtras(m);
}

// torch.ops.tilexr.* : the communicator travels as its integer handle (Comm.handle).
namespace {
TileXRCommPtr FromHandle(int64_t h) { return reinterpret_cast<TileXRCommPtr>(static_cast<uintptr_t>(h)); }

at::Tensor OpAllReduce(const at::Tensor &in, int64_t comm, int64_t op)
{
    at::Tensor out = at::empty_like(in);
    Check(TileXRAllReduce(in.data_ptr(), out.data_ptr(), in.numel(), ToDtype(in.scalar_type()),
                          static_cast<TileXR::TileXRReduceOp>(op), FromHandle(comm), StreamOf(in)),
          "TileXRAllReduce");
    return out;
}
at::Tensor OpAllGather(const at::Tensor &in, int64_t comm, int64_t worldSize)
{
    std::vector<int64_t> shape = in.sizes().vec();
    if (shape.empty()) shape.push_back(1);
    shape[0] *= worldSize;
    at::Tensor out = at::empty(shape, in.options());
    Check(TileXRAllGather(in.data_ptr(), out.data_ptr(), in.numel(), ToDtype(in.scalar_type()), FromHandle(comm), StreamOf(in)),
          "TileXRAllGather");
    return out;
}
at::Tensor OpReduceScatter(const at::Tensor &in, int64_t comm, int64_t worldSize, int64_t op)
{
    std::vector<int64_t> shape = in.sizes().vec();
    TORCH_CHECK(!shape.empty() && shape[0] % worldSize == 0, "reduce_scatter: dim 0 must divide by the world size");
    shape[0] /= worldSize;
    at::Tensor out = at::empty(shape, in.options());
    Check(TileXRReduceScatter(in.data_ptr(), out.data_ptr(), out.numel(), ToDtype(in.scalar_type()),
                              static_cast<TileXR::TileXRReduceOp>(op), FromHandle(comm), StreamOf(in)),
          "TileXRReduceScatter");
    return out;
}
at::Tensor OpAllToAll(const at::Tensor &in, int64_t comm, int64_t worldSize)
{
    at::Tensor out = at::empty_like(in);
    Check(TileXRAllToAll(in.data_ptr(), out.data_ptr(), in.numel() / worldSize, ToDtype(in.scalar_type()), FromHandle(comm),
                         StreamOf(in)),
          "TileXRAllToAll");
    return out;
}
} // namespace

TORCH_LIBRARY(tilexr, m)
{
    m.def("all_reduce(Tensor input, int comm, int op=0) -> Tensor");
    m.def("all_gather(Tensor input, int comm, int world_size) -> Tensor");
    m.def("reduce_scatter(Tensor input, int comm, int world_size, int op=0) -> Tensor");
    m.def("all_to_all(Tensor input, int comm, int world_size) -> Tensor");
}
TORCH_LIBRARY_IMPL(tilexr, CUDA, m)
{
    m.impl("all_reduce", &OpAllReduce);
    m.impl("all_gather", &OpAllGather);
    m.impl("reduce_scatter", &OpReduceScatter);
    m.impl("all_to_all", &OpAllToAll);
}
