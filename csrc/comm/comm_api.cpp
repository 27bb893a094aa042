// C API of the core runtime (tilexr_api.h) on top of TileXRComm.
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <random>
#include <unistd.h>

#include "comm.h"
#include "tilexr_log.h"

using namespace TileXR;

namespace {

// ---- in-process exchange for thread mode ------------------------------------------------------
// Threads of one process that call TileXRCommInitThread with the same uid meet here.
struct ThreadRendezvous {
    std::mutex m;
    std::condition_variable cv;
    int rankSize = 0;
    int arrived = 0;
    uint64_t generation = 0;
    std::vector<uint8_t> buffer;
    std::vector<uint8_t> result;
};

std::mutex g_rendezvousMutex;
std::map<std::string, std::shared_ptr<ThreadRendezvous>> g_rendezvous;

class ThreadExchange : public Exchange {
public:
    ThreadExchange(std::shared_ptr<ThreadRendezvous> rv, int rank, int rankSize)
        : rv_(std::move(rv)), rank_(rank), rankSize_(rankSize)
    {
    }
    int AllGather(const void *send, void *recv, size_t bytes) override
    {
        std::unique_lock<std::mutex> lock(rv_->m);
        if (rv_->arrived == 0) rv_->buffer.assign(bytes * rankSize_, 0);
        if (rv_->buffer.size() != bytes * rankSize_) return TILEXR_ERROR_PARA_CHECK_FAIL;
        std::memcpy(rv_->buffer.data() + rank_ * bytes, send, bytes);
        const uint64_t gen = rv_->generation;
        if (++rv_->arrived == rankSize_) {
            // `result` stays valid until the next gather completes, which needs every rank to
            // have left this one first
            rv_->result = rv_->buffer;
            rv_->arrived = 0;
            rv_->generation += 1;
            rv_->cv.notify_all();
        } else {
            // the reference waits 600 s here (tilexr_comm.cpp:679-746); a minute is plenty in one process
            if (!rv_->cv.wait_for(lock, std::chrono::seconds(60), [&] { return rv_->generation != gen; })) {
                TILEXR_LOG(ERROR) << "thread-mode rendezvous timed out waiting for " << (rankSize_ - rv_->arrived)
                                  << " ranks";
                return TILEXR_ERROR_TIMEOUT;
            }
        }
        std::memcpy(recv, rv_->result.data(), bytes * rankSize_);
        return TILEXR_SUCCESS;
    }

private:
    std::shared_ptr<ThreadRendezvous> rv_;
    int rank_;
    int rankSize_;
};

int BootstrapAddress(int commDomain, std::string *ip, uint16_t *port)
{
    if (!SockExchange::ParseCommId(std::getenv("TILEXR_COMM_ID"), ip, port)) {
        TILEXR_LOG(ERROR) << "TILEXR_COMM_ID must look like 127.0.0.1:10067";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    *port = static_cast<uint16_t>(*port + commDomain);
    return TILEXR_SUCCESS;
}

int InitWithSocket(const InitOptions &opt, int rankSize, int rank, TileXRCommPtr *out)
{
    if (out == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *out = nullptr;
    std::string ip;
    uint16_t port = 0;
    int ret = BootstrapAddress(opt.commDomain, &ip, &port);
    if (ret != TILEXR_SUCCESS) return ret;
    std::unique_ptr<TileXRComm> comm(new TileXRComm(rank, rankSize, opt));
    std::unique_ptr<SockExchange> ex(new SockExchange(rank, rankSize, ip, port));
    ret = comm->Init(std::move(ex));
    if (ret != TILEXR_SUCCESS) return ret;
    *out = comm.release();
    return TILEXR_SUCCESS;
}

TileXRComm *AsComm(TileXRCommPtr p)
{
    TileXRComm *c = static_cast<TileXRComm *>(p);
    return (c != nullptr && c->initialized()) ? c : nullptr;
}

constexpr uint64_t UNIQUE_ID_MAGIC = 0xdddd0000dddd0000ull;
struct UniqueIdBody {
    uint64_t magic;
    char ip[64];
    uint32_t port;
    int32_t domain;
};
static_assert(sizeof(UniqueIdBody) <= TILEXRUNIQUE_ID_BYTES, "unique id body must fit");

} // namespace

extern "C" {

const char *TileXRGetErrorString(int status)
{
    switch (status) {
        case TILEXR_SUCCESS: return "success";
        case TILEXR_ERROR_NOT_INITIALIZED: return "communicator not initialized";
        case TILEXR_ERROR_RUNTIME: return "CUDA runtime call failed";
        case TILEXR_ERROR_PARA_CHECK_FAIL: return "parameter check failed";
        case TILEXR_ERROR_INTERNAL: return "internal error";
        case TILEXR_ERROR_TIMEOUT: return "timeout";
        case TILEXR_ERROR_NOT_SUPPORT: return "not supported";
        case TILEXR_ERROR_NOT_FOUND: return "not found";
        default: return "unknown status";
    }
}

// The id names rank 0's listening address: TILEXR_COMM_ID if set, else loopback with a random
// port, so that two jobs on one host do not collide.
int TileXRGetUniqueId(TileXRUniqueId *uniqueId, int commDomain)
{
    if (uniqueId == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    std::memset(uniqueId, 0, sizeof(*uniqueId));
    UniqueIdBody body{};
    body.magic = UNIQUE_ID_MAGIC;
    std::string ip;
    uint16_t port = 0;
    if (std::getenv("TILEXR_COMM_ID") != nullptr) {
        if (!SockExchange::ParseCommId(std::getenv("TILEXR_COMM_ID"), &ip, &port)) return TILEXR_ERROR_PARA_CHECK_FAIL;
    } else {
        ip = "127.0.0.1";
        std::random_device rd;
        port = static_cast<uint16_t>(20000 + (rd() ^ static_cast<unsigned>(getpid())) % 20000);
    }
    std::strncpy(body.ip, ip.c_str(), sizeof(body.ip) - 1);
    body.port = port;
    body.domain = commDomain;
    std::memcpy(uniqueId->internal, &body, sizeof(body));
    return TILEXR_SUCCESS;
}

int TileXRCommInitRank(TileXRUniqueId commId, int rankSize, int rank, TileXRCommPtr *comm)
{
    if (comm == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *comm = nullptr;
    UniqueIdBody body;
    std::memcpy(&body, commId.internal, sizeof(body));
    if (body.magic != UNIQUE_ID_MAGIC) {
        TILEXR_LOG(ERROR) << "not a TileXR unique id";
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    InitOptions opt;
    opt.commDomain = body.domain;
    std::unique_ptr<TileXRComm> c(new TileXRComm(rank, rankSize, opt));
    std::unique_ptr<SockExchange> ex(
        new SockExchange(rank, rankSize, body.ip, static_cast<uint16_t>(body.port + body.domain)));
    int ret = c->Init(std::move(ex));
    if (ret != TILEXR_SUCCESS) return ret;
    *comm = c.release();
    return TILEXR_SUCCESS;
}

int TileXRCommInitRankLocal(int rankSize, int rank, TileXRCommPtr *comm)
{
    return InitWithSocket(InitOptions(), rankSize, rank, comm);
}

int TileXRCommInit(int rank, int rankSize, TileXRCommPtr *comm)
{
    return InitWithSocket(InitOptions(), rankSize, rank, comm);
}

int TileXRCommInitRankWithDomain(int commDomain, int rankSize, int rank, TileXRCommPtr *comm)
{
    InitOptions opt;
    opt.commDomain = commDomain;
    return InitWithSocket(opt, rankSize, rank, comm);
}

int TileXRCommInitRankWithCustDomainSize(int commDomain, int bufferSizeMB, int rankSize, int rank, TileXRCommPtr *comm)
{
    InitOptions opt;
    opt.commDomain = commDomain;
    opt.bufferMB = bufferSizeMB;
    return InitWithSocket(opt, rankSize, rank, comm);
}

// There are no queue pairs to share between communicators on NVLink; a shared-QP domain is an
// ordinary domain.
int TileXRCommInitRankWithSharedQpDomain(int commDomain, int rankSize, int rank, TileXRCommPtr *comm)
{
    return TileXRCommInitRankWithDomain(commDomain, rankSize, rank, comm);
}

int TileXRCommInitRankMemoryDomain(int commDomain, int rankSize, int rank, TileXRCommPtr *comm)
{
    InitOptions opt;
    opt.commDomain = commDomain;
    opt.bufferMB = TILEXR_MEMORY_DOMAIN_BUFFER_SIZE_MB;
    opt.memoryOnly = true;
    return InitWithSocket(opt, rankSize, rank, comm);
}

int TileXRCommInitRankWithExchange(TileXRAllGatherFn allGather, void *ctx, int commDomain, int bufferSizeMB,
                                   int rankSize, int rank, TileXRCommPtr *comm)
{
    if (comm == nullptr || allGather == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *comm = nullptr;
    InitOptions opt;
    opt.commDomain = commDomain;
    if (bufferSizeMB > 0) opt.bufferMB = bufferSizeMB;
    std::unique_ptr<TileXRComm> c(new TileXRComm(rank, rankSize, opt));
    int ret = c->Init(std::unique_ptr<Exchange>(new CallbackExchange(allGather, ctx)));
    if (ret != TILEXR_SUCCESS) return ret;
    *comm = c.release();
    return TILEXR_SUCCESS;
}

int TileXRCommInitRankHostMemoryWithExchange(TileXRAllGatherFn allGather, void *ctx, int commDomain, int bufferSizeMB,
                                             int rankSize, int rank, TileXRCommPtr *comm)
{
    if (comm == nullptr || allGather == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *comm = nullptr;
    InitOptions opt;
    opt.commDomain = commDomain;
    opt.bufferMB = bufferSizeMB > 0 ? bufferSizeMB : 64;
    opt.mode = CommMode::HOST_MEMORY;
    std::unique_ptr<TileXRComm> c(new TileXRComm(rank, rankSize, opt));
    int ret = c->Init(std::unique_ptr<Exchange>(new CallbackExchange(allGather, ctx)));
    if (ret != TILEXR_SUCCESS) return ret;
    *comm = c.release();
    return TILEXR_SUCCESS;
}

int TileXRCommInitRankHostMemory(int commDomain, int bufferSizeMB, int rankSize, int rank, TileXRCommPtr *comm)
{
    InitOptions opt;
    opt.commDomain = commDomain;
    opt.bufferMB = bufferSizeMB > 0 ? bufferSizeMB : 64;
    opt.mode = CommMode::HOST_MEMORY;
    return InitWithSocket(opt, rankSize, rank, comm);
}

int TileXRCommInitThread(int rank, int rankSize, const char *uid, TileXRCommPtr *comm)
{
    if (comm == nullptr || uid == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *comm = nullptr;
    std::shared_ptr<ThreadRendezvous> rv;
    {
        std::lock_guard<std::mutex> lock(g_rendezvousMutex);
        std::shared_ptr<ThreadRendezvous> &slot = g_rendezvous[uid];
        if (!slot) {
            slot = std::make_shared<ThreadRendezvous>();
            slot->rankSize = rankSize;
        }
        if (slot->rankSize != rankSize) return TILEXR_ERROR_PARA_CHECK_FAIL;
        rv = slot;
    }
    InitOptions opt;
    opt.mode = CommMode::THREAD;
    std::unique_ptr<TileXRComm> c(new TileXRComm(rank, rankSize, opt));
    int ret = c->Init(std::unique_ptr<Exchange>(new ThreadExchange(rv, rank, rankSize)));
    if (ret != TILEXR_SUCCESS) return ret;
    *comm = c.release();
    return TILEXR_SUCCESS;
}

static int InitWorld(uint32_t ndev, const int32_t *devices, int bufferMB, bool emulated, TileXRCommPtr *comms)
{
    if (ndev == 0 || ndev > TILEXR_MAX_RANK_SIZE || comms == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    int previous = 0;
    cudaGetDevice(&previous);
    InitOptions opt;
    opt.mode = CommMode::EMULATED;
    if (bufferMB > 0) opt.bufferMB = bufferMB;
    auto world = std::make_shared<EmulatedWorld>(static_cast<int>(ndev), devices[0]);
    std::vector<std::unique_ptr<TileXRComm>> built;
    for (uint32_t r = 0; r < ndev; ++r) {
        built.emplace_back(new TileXRComm(static_cast<int>(r), static_cast<int>(ndev), opt));
        int ret = built.back()->InitInWorld(world, devices[r]);
        if (ret != TILEXR_SUCCESS) return ret;
    }
    for (auto &c : built) {
        int ret = c->FinishWorldInit();
        if (ret != TILEXR_SUCCESS) return ret;
    }
    (void)emulated;
    for (uint32_t r = 0; r < ndev; ++r) comms[r] = built[r].release();
    cudaSetDevice(previous);
    return TILEXR_SUCCESS;
}

// One communicator per listed device, all driven by the calling thread.  When a device is
// listed more than once its ranks share the GPU, which only works for group launches.
int TileXRCommInitAll(uint32_t ndev, int32_t *devices, TileXRCommPtr *comms)
{
    if (devices == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    for (uint32_t i = 1; i < ndev; ++i) {
        if (devices[i] != devices[0]) {
            TILEXR_LOG(ERROR) << "TileXRCommInitAll drives all ranks from one thread, which needs them on one device "
                              << "(an emulated world); use TileXRCommInitThread with one thread per GPU otherwise";
            return TILEXR_ERROR_NOT_SUPPORT;
        }
    }
    return InitWorld(ndev, devices, 0, true, comms);
}

int TileXRCommInitEmulated(uint32_t rankSize, int32_t device, int bufferSizeMB, TileXRCommPtr *comms)
{
    std::vector<int32_t> devices(rankSize, device);
    return InitWorld(rankSize, devices.data(), bufferSizeMB, true, comms);
}

int TileXRCommDestroy(TileXRCommPtr comm)
{
    TileXRComm *c = static_cast<TileXRComm *>(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    delete c;
    return TILEXR_SUCCESS;
}

int TileXRGetCommArgsDev(TileXRCommPtr comm, GM_ADDR *commArgsPtr)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || commArgsPtr == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    *commArgsPtr = reinterpret_cast<GM_ADDR>(c->isHostMemory() ? c->hostArgs() : c->devArgs());
    return TILEXR_SUCCESS;
}

int TileXRGetCommArgsHost(TileXRCommPtr comm, TileXRCommArgs **commArgsPtr)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || commArgsPtr == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    *commArgsPtr = c->hostArgs();
    return TILEXR_SUCCESS;
}

int TileXRCommNextMagic(TileXRCommPtr comm, int64_t *magic)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || magic == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    *magic = c->NextMagic();
    return TILEXR_SUCCESS;
}

int TileXRUDMARegister(TileXRCommPtr comm, GM_ADDR localPtr, size_t bytes, TileXRUDMAMemHandle *handle)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->Register(localPtr, bytes, false, handle);
}

int TileXRUDMAUnregister(TileXRCommPtr comm, TileXRUDMAMemHandle handle)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->Unregister(handle);
}

int TileXRUDMAProfileRegister(TileXRCommPtr comm, const TileXRUDMAProfileDesc *desc, TileXRUDMAProfileHandle *handle)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (desc == nullptr || handle == nullptr || desc->regionCount == 0 || desc->regionCount > TILEXR_PROFILE_MAX_REGIONS) {
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    uint32_t slot = 0;
    while (slot < c->profiles().size() && c->profiles()[slot].live) ++slot;
    if (slot == c->profiles().size()) return TILEXR_ERROR_INTERNAL;
    ProfileRecord rec;
    rec.live = true;
    rec.view.regionCount = desc->regionCount;
    for (uint32_t i = 0; i < desc->regionCount; ++i) {
        int ret = c->Register(static_cast<uint8_t *>(desc->base[i]), desc->bytes[i], false, &rec.view.handles[i]);
        if (ret != TILEXR_SUCCESS) {
            for (uint32_t j = 0; j < i; ++j) c->Unregister(rec.view.handles[j]);
            return ret;
        }
    }
    rec.view.generation = c->hostArgs()->registrationGeneration;
    c->profiles()[slot] = rec;
    *handle = slot;
    return TILEXR_SUCCESS;
}

int TileXRUDMAProfileUnregister(TileXRCommPtr comm, TileXRUDMAProfileHandle handle)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (handle >= c->profiles().size() || !c->profiles()[handle].live) return TILEXR_ERROR_NOT_FOUND;
    ProfileRecord &rec = c->profiles()[handle];
    for (uint32_t i = 0; i < rec.view.regionCount; ++i) c->Unregister(rec.view.handles[i]);
    rec = ProfileRecord();
    return TILEXR_SUCCESS;
}

int TileXRUDMAProfileQuery(TileXRCommPtr comm, TileXRUDMAProfileHandle handle, TileXRUDMAProfileView *view)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (view == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (handle >= c->profiles().size() || !c->profiles()[handle].live) return TILEXR_ERROR_NOT_FOUND;
    *view = c->profiles()[handle].view;
    return TILEXR_SUCCESS;
}

// Ordering lanes are software constructs here; report the reference's shared-QP count so that
// callers sizing per-QP tables keep working.
int TileXRUDMAGetQpCount(TileXRCommPtr comm, uint32_t *qpCount)
{
    if (AsComm(comm) == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (qpCount == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *qpCount = 32;
    return TILEXR_SUCCESS;
}

int TileXRUDMAFullmeshQuery(TileXRCommPtr comm, TileXRUDMAFullmeshHostView *view)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (view == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    std::memset(view, 0, sizeof(*view));
    view->slotCount = static_cast<uint32_t>(c->rankSize());
    for (int r = 0; r < c->rankSize(); ++r) view->peerMask[r / 64] |= (1ull << (r % 64));
    view->generation = c->hostArgs()->registrationGeneration;
    return TILEXR_SUCCESS;
}

int TileXRGetUDMARegistryDev(TileXRCommPtr comm, GM_ADDR *registryPtr)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || registryPtr == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    *registryPtr = reinterpret_cast<GM_ADDR>(c->isHostMemory() ? c->hostRegistry() : c->devRegistry());
    return TILEXR_SUCCESS;
}

int TileXRGetUDMARegistryHost(TileXRCommPtr comm, const TileXRRegistryT **registry)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || registry == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    *registry = c->hostRegistry();
    return TILEXR_SUCCESS;
}

int TileXRSDMAAvailable(TileXRCommPtr comm, bool *available)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || available == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    *available = (c->hostArgs()->extraFlag & TILEXR_FLAG_LOCAL_COPY) != 0;
    return TILEXR_SUCCESS;
}

int TileXRGetSDMAWorkspaceDev(TileXRCommPtr comm, GM_ADDR *workspace)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || workspace == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    *workspace = static_cast<GM_ADDR>(c->hostArgs()->localCopyWorkspace);
    return TILEXR_SUCCESS;
}

void TileXRPrintDFX2Log(TileXRCommPtr comm)
{
    TileXRComm *c = AsComm(comm);
    if (c != nullptr) c->PrintDfx();
}

int TileXRCommGetDeviceStatus(TileXRCommPtr comm, int *status)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr || status == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->DeviceStatus(status);
}

int TileXRCommResetStatus(TileXRCommPtr comm)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->ResetStatus();
}

int TileXRCommSetWaitTimeoutMs(TileXRCommPtr comm, uint64_t milliseconds)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (milliseconds == 0) return TILEXR_ERROR_PARA_CHECK_FAIL;
    c->hostArgs()->waitTimeoutNs = milliseconds * 1000000ull;
    return c->SyncCommArgs();
}

int TileXRCommHostBarrier(TileXRCommPtr comm)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->HostBarrier();
}

int TileXRCommGetInfo(TileXRCommPtr comm, int *rank, int *rankSize, int *device, uint64_t *dataHalfBytes)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (rank != nullptr) *rank = c->rank();
    if (rankSize != nullptr) *rankSize = c->rankSize();
    if (device != nullptr) *device = c->device();
    if (dataHalfBytes != nullptr) *dataHalfBytes = c->hostArgs()->dataHalfBytes;
    return TILEXR_SUCCESS;
}

int TileXRSymmAlloc(TileXRCommPtr comm, size_t bytes, void **localPtr, TileXRUDMAMemHandle *handle)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (bytes == 0 || localPtr == nullptr || handle == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (c->isHostMemory()) return TILEXR_ERROR_NOT_SUPPORT;
    if (cudaSetDevice(c->device()) != cudaSuccess) return TILEXR_ERROR_RUNTIME;
    void *p = nullptr;
    const size_t rounded = (bytes + 511) & ~static_cast<size_t>(511);
    if (c->usesVmm()) {
        // every rank of the communicator took the same route at bring-up, so all of them are in here
        const int ret = c->SymmAllocVmm(rounded, localPtr, handle);
        if (ret != TILEXR_ERROR_NOT_SUPPORT) return ret;
    }
    if (cudaMalloc(&p, rounded) != cudaSuccess) {
        cudaGetLastError();
        return TILEXR_ERROR_RUNTIME;
    }
    cudaMemset(p, 0, rounded);
    cudaDeviceSynchronize();
    int ret = c->Register(static_cast<uint8_t *>(p), rounded, true, handle);
    if (ret != TILEXR_SUCCESS) {
        cudaFree(p);
        return ret;
    }
    *localPtr = p;
    return TILEXR_SUCCESS;
}

int TileXRSymmFree(TileXRCommPtr comm, TileXRUDMAMemHandle handle)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->Unregister(handle);
}

int TileXRGetMulticastPointer(TileXRCommPtr comm, const void *ptr, size_t bytes, void **mcPtr)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (ptr == nullptr || mcPtr == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *mcPtr = nullptr;
    const uint8_t *p = static_cast<const uint8_t *>(ptr);
    if (c->usesVmm() && p >= c->window() && p + bytes <= c->window() + c->hostArgs()->peerMemBytes) {
        if (c->windowMulticast() != nullptr) *mcPtr = c->windowMulticast() + (p - c->window());
        return TILEXR_SUCCESS;
    }
    for (const RegionRecord &rec : c->regions()) {
        if (!rec.live || !rec.vmm.live) continue;
        if (p >= rec.localBase && p + bytes <= rec.localBase + rec.bytes) {
            if (rec.vmm.multicast != nullptr) *mcPtr = rec.vmm.multicast + (p - rec.localBase);
            return TILEXR_SUCCESS;
        }
    }
    return TILEXR_ERROR_NOT_FOUND;
}

int TileXRNvlsAvailable(TileXRCommPtr comm)
{
    TileXRComm *c = AsComm(comm);
    return (c != nullptr && c->initialized() && (c->hostArgs()->extraFlag & TILEXR_FLAG_NVLS) != 0) ? 1 : 0;
}

int TileXRGetPeerPointers(TileXRCommPtr comm, TileXRUDMAMemHandle handle, void **peerPtrs)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (peerPtrs == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (handle >= c->regions().size() || !c->regions()[handle].live) return TILEXR_ERROR_NOT_FOUND;
    const RegionRecord &rec = c->regions()[handle];
    for (int r = 0; r < c->rankSize(); ++r) peerPtrs[r] = rec.peerBase[r];
    return TILEXR_SUCCESS;
}

int TileXRFindRegistration(TileXRCommPtr comm, const void *ptr, size_t bytes, TileXRUDMAMemHandle *handle,
                           uint64_t *offset)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->FindRegistration(ptr, bytes, handle, offset);
}

int TileXRGetPhysicalInfo(TileXRCommPtr comm, TileXRPhysicalInfoT *info)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (info == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *info = c->physicalInfo();
    return TILEXR_SUCCESS;
}

int TileXRGetOperatorScratch(TileXRCommPtr comm, size_t bytes, void **ptr)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    return c->OperatorScratch(bytes, ptr);
}

int TileXRLocalCopyAsync(TileXRCommPtr comm, void *dst, const void *src, size_t bytes, TileXRStream stream)
{
    TileXRComm *c = AsComm(comm);
    if (c == nullptr) return TILEXR_ERROR_NOT_INITIALIZED;
    if (dst == nullptr || src == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    return c->LocalCopyAsync(dst, src, bytes, static_cast<cudaStream_t>(stream));
}

} // extern "C"
