#include "comm.h"

#include <algorithm>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <fcntl.h>
#include <map>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "tilexr_log.h"

namespace TileXR {

#define TXR_CUDA(call)                                                                              \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess) {                                                                    \
            TILEXR_LOG(ERROR) << #call << " failed: " << cudaGetErrorString(e_);                    \
            return TILEXR_ERROR_RUNTIME;                                                            \
        }                                                                                           \
    } while (0)

namespace {

uint64_t HashString(const std::string &s)
{
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : s) {
        h ^= c;
        h *= 1099511628211ull;
    }
    return h;
}

long EnvLong(const char *name, long fallback)
{
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') return fallback;
    char *end = nullptr;
    const long x = std::strtol(v, &end, 10);
    return (*end == '\0') ? x : fallback;
}

// What every rank tells the others at bring-up.
struct PeerInfo {
    int32_t device;
    int32_t pid;
    uint64_t hostHash;
    uint64_t rawPtr;
    uint64_t windowBytes;
    uint32_t knobs;
    uint32_t bufferMB;
    uint64_t timeoutNs;
    cudaIpcMemHandle_t handle;
};

struct RegionInfo {
    int32_t pid;
    int32_t device;
    uint64_t rawPtr;      // address of the registered range in the owner's address space
    uint64_t offset;      // of the range inside its allocation
    uint64_t bytes;
    uint32_t handleIndex;
    uint32_t valid;
    cudaIpcMemHandle_t handle;
};

typedef int (*CuMemGetAddressRangeFn)(unsigned long long *, size_t *, unsigned long long);

int AllocationBase(const void *ptr, uint8_t **base, size_t *size)
{
    static CuMemGetAddressRangeFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
        return reinterpret_cast<CuMemGetAddressRangeFn>(f);
    }();
    if (fn == nullptr) return TILEXR_ERROR_RUNTIME;
    unsigned long long b = 0;
    size_t s = 0;
    if (fn(&b, &s, reinterpret_cast<unsigned long long>(ptr)) != 0) return TILEXR_ERROR_RUNTIME;
    *base = reinterpret_cast<uint8_t *>(b);
    *size = s;
    return TILEXR_SUCCESS;
}

} // namespace

uint64_t DefaultWaitTimeoutNs()
{
    const long ms = EnvLong("TILEXR_WAIT_TIMEOUT_MS", 10000);
    return static_cast<uint64_t>(ms > 0 ? ms : 10000) * 1000000ull;
}

TileXRComm::TileXRComm(int rank, int rankSize, const InitOptions &opt) : rank_(rank), rankSize_(rankSize), opt_(opt)
{
    waitTimeoutNs_ = DefaultWaitTimeoutNs();
    regions_.resize(TILEXR_MAX_REGISTERED_REGIONS);
    profiles_.resize(16);
    registry_.magic = TILEXR_REGISTRY_MAGIC;
    registry_.version = 1;
    registry_.rankSize = static_cast<uint32_t>(rankSize);
    registry_.regionCount = 0;
    if (std::getenv("LCCL_DETERMINISTIC") != nullptr && EnvLong("LCCL_DETERMINISTIC", 0) != 0) {
        knobFlags_ |= TILEXR_FLAG_DETERMINISTIC;
    }
    if (EnvLong("TILEXR_ENABLE_SDMA", 1) != 0) knobFlags_ |= TILEXR_FLAG_LOCAL_COPY;
    if (EnvLong("TILEXR_ENABLE_UDMA", 1) != 0 && !opt.memoryOnly) knobFlags_ |= TILEXR_FLAG_RMA;
    wantVmm_ = EnvLong("TILEXR_ENABLE_VMM", 1) != 0;
    wantNvls_ = EnvLong("TILEXR_ENABLE_NVLS", 1) != 0;
}

TileXRComm::~TileXRComm()
{
    destroying_ = true;
    const bool gpu = !isHostMemory();
    if (gpu && device_ >= 0) cudaSetDevice(device_);
    if (gpu && windowVmm_.live && initialized_) {
        // Memory bound to a multicast object is let go only after every rank has finished its kernels: all
        // ranks destroy the communicator together, and they meet here once before anybody unbinds anything.
        cudaDeviceSynchronize();
        if (exchange_ != nullptr) exchange_->Barrier();
    }
    for (size_t h = 0; h < regions_.size(); ++h) {
        if (regions_[h].live) Unregister(static_cast<TileXRUDMAMemHandle>(h));
    }
    if (gpu) {
        for (void *p : ipcOpened_) cudaIpcCloseMemHandle(p);
        if (devArgs_ != nullptr) cudaFree(devArgs_);
        if (devRegistry_ != nullptr) cudaFree(devRegistry_);
        if (localCopyWorkspace_ != nullptr) cudaFree(localCopyWorkspace_);
        if (operatorScratch_ != nullptr) cudaFree(operatorScratch_);
        if (windowVmm_.live) {
            VmmFree(nullptr, &windowVmm_);          // the ranks have met above
            window_ = nullptr;
        }
        if (window_ != nullptr) cudaFree(window_);
        if (copyStream_ != nullptr) cudaStreamDestroy(copyStream_);
        if (copyEventIn_ != nullptr) cudaEventDestroy(copyEventIn_);
        if (copyEventOut_ != nullptr) cudaEventDestroy(copyEventOut_);
        delete hostArgs_;
    } else {
        for (int r = 0; r < static_cast<int>(peerWindows_.size()); ++r) {
            if (peerWindows_[r] != nullptr) munmap(peerWindows_[r], windowBytes_);
        }
        if (!shmNames_.empty()) shm_unlink(shmNames_[rank_].c_str());
        delete hostArgs_;
    }
}

int TileXRComm::AllocateWindow()
{
    const size_t dataBytes = static_cast<size_t>(opt_.bufferMB) << 20;
    windowBytes_ = static_cast<size_t>(TILEXR_WIN_DATA_OFFSET) + dataBytes;
    if (isHostMemory()) {
        // every rank derives the segment names from a job id that rank 0 drew
        uint64_t mine = (static_cast<uint64_t>(getpid()) << 32) ^ static_cast<uint64_t>(time(nullptr)) ^
                        reinterpret_cast<uintptr_t>(this);
        std::vector<uint64_t> ids(rankSize_);
        if (exchange_->AllGather(&mine, ids.data(), sizeof(mine)) != TILEXR_SUCCESS) return TILEXR_ERROR_INTERNAL;
        const uint64_t job = ids[0];
        shmNames_.resize(rankSize_);
        for (int r = 0; r < rankSize_; ++r) {
            char name[96];
            std::snprintf(name, sizeof(name), "/tilexr-%016llx-d%d-r%d", static_cast<unsigned long long>(job),
                          opt_.commDomain, r);
            shmNames_[r] = name;
        }
        shm_unlink(shmNames_[rank_].c_str());
        const int fd = shm_open(shmNames_[rank_].c_str(), O_CREAT | O_RDWR | O_EXCL, 0600);
        if (fd < 0) {
            TILEXR_LOG(ERROR) << "shm_open " << shmNames_[rank_] << ": " << std::strerror(errno);
            return TILEXR_ERROR_INTERNAL;
        }
        if (ftruncate(fd, static_cast<off_t>(windowBytes_)) != 0) {
            close(fd);
            return TILEXR_ERROR_INTERNAL;
        }
        void *p = mmap(nullptr, windowBytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        close(fd);
        if (p == MAP_FAILED) return TILEXR_ERROR_INTERNAL;
        window_ = static_cast<uint8_t *>(p);
        // fresh shared memory is zero filled; touch only the control and flag areas
        std::memset(window_, 0, static_cast<size_t>(TILEXR_WIN_DATA_OFFSET));
        return TILEXR_SUCCESS;
    }
    TXR_CUDA(cudaMalloc(reinterpret_cast<void **>(&window_), windowBytes_));
    // flags and control words must start at zero; the data halves need no initial value
    TXR_CUDA(cudaMemset(window_, 0, static_cast<size_t>(TILEXR_WIN_DATA_OFFSET)));
    TXR_CUDA(cudaDeviceSynchronize());
    return TILEXR_SUCCESS;
}

// The window through the virtual-memory API: one collective call allocates, trades POSIX descriptors, maps every
// peer and, where the node has NVSwitch multicast, binds all copies to one multicast object.  Only processes of
// one host can pass descriptors; anything else (or a refusal anywhere) returns NOT_SUPPORT on every rank and the
// caller takes the cudaMalloc + CUDA IPC route.
int TileXRComm::TryVmmWindow()
{
    if (opt_.mode != CommMode::PROCESS || !wantVmm_) return TILEXR_ERROR_NOT_SUPPORT;
    struct Probe {
        uint64_t hostHash;
        uint64_t job;
    } mine{HashString(SockExchange::ReadBootId()),
           (static_cast<uint64_t>(getpid()) << 32) ^ static_cast<uint64_t>(time(nullptr)) ^ reinterpret_cast<uintptr_t>(this)};
    std::vector<Probe> all(rankSize_);
    int ret = exchange_->AllGather(&mine, all.data(), sizeof(Probe));
    if (ret != TILEXR_SUCCESS) return ret;
    for (const Probe &p : all) {
        if (p.hostHash != mine.hostHash) return TILEXR_ERROR_NOT_SUPPORT;
    }
    vmmTag_ = all[0].job ^ (static_cast<uint64_t>(opt_.commDomain) << 48);
    const size_t dataBytes = static_cast<size_t>(opt_.bufferMB) << 20;
    windowBytes_ = static_cast<size_t>(TILEXR_WIN_DATA_OFFSET) + dataBytes;
    ret = VmmAllocate(*exchange_, rank_, rankSize_, device_, windowBytes_, wantNvls_, vmmTag_ + vmmSeq_++, &windowVmm_);
    if (ret != TILEXR_SUCCESS) return ret;
    window_ = windowVmm_.local;
    peerWindows_ = windowVmm_.peers;
    TXR_CUDA(cudaMemset(window_, 0, static_cast<size_t>(TILEXR_WIN_DATA_OFFSET)));
    TXR_CUDA(cudaDeviceSynchronize());
    return exchange_->Barrier();
}

int TileXRComm::AgreeOnKnobs()
{
    struct Knobs {
        uint32_t flags;
        uint32_t bufferMB;
        uint64_t timeoutNs;
        int32_t memoryOnly;
        int32_t domain;
        int32_t vmm;
        int32_t nvls;
    } mine{knobFlags_, static_cast<uint32_t>(opt_.bufferMB), waitTimeoutNs_, opt_.memoryOnly ? 1 : 0, opt_.commDomain,
           wantVmm_ ? 1 : 0, wantNvls_ ? 1 : 0};
    std::vector<Knobs> all(rankSize_);
    int ret = exchange_->AllGather(&mine, all.data(), sizeof(Knobs));
    if (ret != TILEXR_SUCCESS) return ret;
    for (int r = 0; r < rankSize_; ++r) {
        if (std::memcmp(&all[r], &mine, sizeof(Knobs)) != 0) {
            TILEXR_LOG(ERROR) << "rank " << r << " was started with different TILEXR_*/LCCL_* settings or buffer size "
                              << "than rank " << rank_ << "; every rank must agree";
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
    }
    return TILEXR_SUCCESS;
}

int TileXRComm::MapHostMemoryWindows()
{
    int ret = exchange_->Barrier();   // every rank created its segment
    if (ret != TILEXR_SUCCESS) return ret;
    peerWindows_.assign(rankSize_, nullptr);
    for (int r = 0; r < rankSize_; ++r) {
        if (r == rank_) {
            peerWindows_[r] = window_;
            continue;
        }
        const int fd = shm_open(shmNames_[r].c_str(), O_RDWR, 0600);
        if (fd < 0) {
            TILEXR_LOG(ERROR) << "cannot open window of rank " << r << ": " << std::strerror(errno);
            return TILEXR_ERROR_INTERNAL;
        }
        void *p = mmap(nullptr, windowBytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        close(fd);
        if (p == MAP_FAILED) return TILEXR_ERROR_INTERNAL;
        peerWindows_[r] = static_cast<uint8_t *>(p);
    }
    return exchange_->Barrier();
}

// What this device is and how it reaches its peers.  Read-only queries; nothing is configured.  Device ordinals of
// peers in other processes are theirs, which equals ours when the processes see the same devices (the usual
// one-process-per-GPU launch); an ordinal this process does not have is skipped.
void TileXRComm::DetectTopology(const std::vector<int> &peerDevices)
{
    TileXRPhysicalInfo &ph = physical_;
    ph = TileXRPhysicalInfo{};
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device_) == cudaSuccess) {
        ph.ccMajor = prop.major;
        ph.ccMinor = prop.minor;
        ph.smCount = static_cast<uint32_t>(prop.multiProcessorCount);
        ph.l2Bytes = static_cast<uint32_t>(prop.l2CacheSize);
        ph.memoryBytes = prop.totalGlobalMem;
    }
    int deviceCount = 0;
    cudaGetDeviceCount(&deviceCount);
    bool anyPeer = false, allAtomics = true, anyPcie = false;
    int worstRank = 0;
    for (int r = 0; r < static_cast<int>(peerDevices.size()); ++r) {
        const int d = peerDevices[r];
        if (r == rank_ || d == device_ || d < 0 || d >= deviceCount) continue;
        int access = 0, atomics = 0, perf = 0;
        if (cudaDeviceGetP2PAttribute(&access, cudaDevP2PAttrAccessSupported, device_, d) != cudaSuccess || access == 0) {
            cudaGetLastError();
            continue;
        }
        anyPeer = true;
        cudaDeviceGetP2PAttribute(&atomics, cudaDevP2PAttrNativeAtomicSupported, device_, d);
        cudaDeviceGetP2PAttribute(&perf, cudaDevP2PAttrPerformanceRank, device_, d);
        cudaGetLastError();
        if (atomics == 0) {
            allAtomics = false;
            anyPcie = true;
        }
        worstRank = std::max(worstRank, perf);
    }
    ph.link = !anyPeer ? TILEXR_LINK_SAME_DEVICE : anyPcie ? TILEXR_LINK_PCIE : TILEXR_LINK_NVLINK;
    ph.p2pNativeAtomics = anyPeer && allAtomics ? 1 : 0;
    ph.p2pPerformanceRank = worstRank;
    bool vmm = false, multicast = false;
    if (VmmDeviceSupport(device_, &vmm, &multicast) == TILEXR_SUCCESS) ph.multicastSupported = multicast ? 1 : 0;
}

int TileXRComm::ExchangeWindows()
{
    PeerInfo mine{};
    mine.device = device_;
    mine.pid = static_cast<int32_t>(getpid());
    mine.hostHash = HashString(SockExchange::ReadBootId());
    mine.rawPtr = reinterpret_cast<uint64_t>(window_);
    mine.windowBytes = windowBytes_;
    if (opt_.mode == CommMode::PROCESS) {
        TXR_CUDA(cudaIpcGetMemHandle(&mine.handle, window_));
    }
    std::vector<PeerInfo> all(rankSize_);
    int ret = exchange_->AllGather(&mine, all.data(), sizeof(PeerInfo));
    if (ret != TILEXR_SUCCESS) return ret;
    peerWindows_.assign(rankSize_, nullptr);
    for (int i = 0; i < rankSize_; ++i) {
        const int r = (rank_ + i) % rankSize_;
        const PeerInfo &p = all[r];
        if (r == rank_) {
            peerWindows_[r] = window_;
            continue;
        }
        if (p.hostHash != mine.hostHash) {
            TILEXR_LOG(ERROR) << "rank " << r << " runs on another host; this build maps peers inside one NVSwitch "
                              << "node only";
            return TILEXR_ERROR_NOT_SUPPORT;
        }
        if (p.windowBytes != windowBytes_) return TILEXR_ERROR_PARA_CHECK_FAIL;
        if (p.pid == mine.pid) {
            if (p.device != device_) {
                int can = 0;
                TXR_CUDA(cudaDeviceCanAccessPeer(&can, device_, p.device));
                if (!can) {
                    TILEXR_LOG(ERROR) << "device " << device_ << " cannot access device " << p.device;
                    return TILEXR_ERROR_NOT_SUPPORT;
                }
                cudaError_t e = cudaDeviceEnablePeerAccess(p.device, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
                    TILEXR_LOG(ERROR) << "cudaDeviceEnablePeerAccess: " << cudaGetErrorString(e);
                    return TILEXR_ERROR_RUNTIME;
                }
                cudaGetLastError();
            }
            peerWindows_[r] = reinterpret_cast<uint8_t *>(p.rawPtr);
        } else {
            void *mapped = nullptr;
            TXR_CUDA(cudaIpcOpenMemHandle(&mapped, p.handle, cudaIpcMemLazyEnablePeerAccess));
            ipcOpened_.push_back(mapped);
            peerWindows_[r] = static_cast<uint8_t *>(mapped);
        }
    }
    return exchange_->Barrier();
}

void TileXRComm::FillCommArgs()
{
    CommArgs &a = *hostArgs_;
    std::memset(&a, 0, sizeof(a));
    a.rank = rank_;
    a.localRank = rank_;
    a.rankSize = rankSize_;
    a.localRankSize = rankSize_;
    a.commDomain = opt_.commDomain;
    a.peerMemBytes = windowBytes_;
    a.dataHalfBytes = ((static_cast<uint64_t>(opt_.bufferMB) << 20) / 2) & ~static_cast<uint64_t>(255);
    a.waitTimeoutNs = waitTimeoutNs_;
    a.extraFlag = knobFlags_ | TILEXR_FLAG_P2P;
    if (opt_.memoryOnly) a.extraFlag |= TILEXR_FLAG_MEMORY_ONLY;
    if (opt_.mode == CommMode::THREAD || opt_.mode == CommMode::EMULATED) a.extraFlag |= TILEXR_FLAG_SAME_PROCESS;
    if (opt_.mode == CommMode::EMULATED) a.extraFlag |= TILEXR_FLAG_EMULATED;
    if (opt_.mode == CommMode::HOST_MEMORY) {
        a.extraFlag |= TILEXR_FLAG_HOST_MEMORY;
        a.extraFlag &= ~static_cast<uint32_t>(TILEXR_FLAG_LOCAL_COPY);
    }
    for (int r = 0; r < rankSize_; ++r) {
        a.peerMems[r] = peerWindows_[r];
        a.signalMems[r] = peerWindows_[r] + TILEXR_CTRL_SIGNAL_OFFSET;
    }
    a.localCopyWorkspace = localCopyWorkspace_;
    a.registryPtr = devRegistry_;
    if (windowVmm_.live && windowVmm_.multicast != nullptr) {
        a.multicastMem = windowVmm_.multicast;
        a.extraFlag |= TILEXR_FLAG_NVLS;
        physical_.nvlsBound = 1;
    }
    if (!isHostMemory() && physical_.smCount == 0) DetectTopology(std::vector<int>());     // worlds that exchange no peer records
    physical_.vmmWindow = windowVmm_.live ? 1 : 0;
    if (opt_.mode == CommMode::HOST_MEMORY) physical_.link = TILEXR_LINK_HOST_MEMORY;
    else if (opt_.mode == CommMode::EMULATED || rankSize_ == 1) physical_.link = TILEXR_LINK_SAME_DEVICE;
    if (physical_.link == TILEXR_LINK_NVLINK) a.extraFlag |= TILEXR_FLAG_TOPO_NVLINK;
    if (physical_.link == TILEXR_LINK_PCIE) a.extraFlag |= TILEXR_FLAG_TOPO_PCIE;
}

int TileXRComm::SyncCommArgs()
{
    if (isHostMemory()) return TILEXR_SUCCESS;   // hostArgs_ is what the CPU kernels read
    TXR_CUDA(cudaMemcpy(devArgs_, hostArgs_, offsetof(CommArgs, dfx), cudaMemcpyHostToDevice));
    return TILEXR_SUCCESS;
}

int TileXRComm::Init(std::unique_ptr<Exchange> exchange)
{
    if (rankSize_ <= 0 || rankSize_ > TILEXR_MAX_RANK_SIZE || rank_ < 0 || rank_ >= rankSize_ || opt_.bufferMB < 2) {
        TILEXR_LOG(ERROR) << "bad communicator shape rank=" << rank_ << " rankSize=" << rankSize_
                          << " bufferMB=" << opt_.bufferMB;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    exchange_ = std::move(exchange);
    int ret = AgreeOnKnobs();
    if (ret != TILEXR_SUCCESS) return ret;
    hostArgs_ = new CommArgs();
    if (isHostMemory()) {
        ret = AllocateWindow();
        if (ret != TILEXR_SUCCESS) return ret;
        ret = MapHostMemoryWindows();
        if (ret != TILEXR_SUCCESS) return ret;
        FillCommArgs();
        devArgs_ = nullptr;
        initialized_ = true;
        return TILEXR_SUCCESS;
    }
    TXR_CUDA(cudaGetDevice(&device_));
    TXR_CUDA(cudaFree(nullptr));             // the device's context exists before any driver call
    {
        // which device every rank sits on, for the link description (both window paths below need it)
        std::vector<int32_t> devices(rankSize_);
        const int32_t mine = device_;
        ret = exchange_->AllGather(&mine, devices.data(), sizeof(int32_t));
        if (ret != TILEXR_SUCCESS) return ret;
        DetectTopology(std::vector<int>(devices.begin(), devices.end()));
    }
    ret = TryVmmWindow();
    if (ret == TILEXR_ERROR_NOT_SUPPORT) {
        ret = AllocateWindow();
        if (ret != TILEXR_SUCCESS) return ret;
        ret = ExchangeWindows();
    }
    if (ret != TILEXR_SUCCESS) return ret;
    TXR_CUDA(cudaMalloc(reinterpret_cast<void **>(&devArgs_), sizeof(CommArgs)));
    TXR_CUDA(cudaMemset(devArgs_, 0, sizeof(CommArgs)));
    TXR_CUDA(cudaMalloc(reinterpret_cast<void **>(&devRegistry_), sizeof(TileXRRegistry)));
    TXR_CUDA(cudaMemcpy(devRegistry_, &registry_, sizeof(TileXRRegistry), cudaMemcpyHostToDevice));
    TXR_CUDA(cudaMalloc(&localCopyWorkspace_, 4096));
    TXR_CUDA(cudaStreamCreateWithFlags(&copyStream_, cudaStreamNonBlocking));
    TXR_CUDA(cudaEventCreateWithFlags(&copyEventIn_, cudaEventDisableTiming));
    TXR_CUDA(cudaEventCreateWithFlags(&copyEventOut_, cudaEventDisableTiming));
    FillCommArgs();
    ret = SyncCommArgs();
    if (ret != TILEXR_SUCCESS) return ret;
    initialized_ = true;
    TILEXR_LOG(INFO) << "rank " << rank_ << "/" << rankSize_ << " ready on device " << device_ << ", window "
                     << (windowBytes_ >> 20) << " MiB, "
                     << (windowVmm_.live ? (windowVmm_.multicast != nullptr ? "virtual-memory API with NVLink multicast" : "virtual-memory API")
                                         : "cudaMalloc + CUDA IPC");
    return exchange_->Barrier();
}

int TileXRComm::InitInWorld(std::shared_ptr<EmulatedWorld> world, int device)
{
    world_ = std::move(world);
    device_ = device;
    hostArgs_ = new CommArgs();
    TXR_CUDA(cudaSetDevice(device_));
    int ret = AllocateWindow();
    if (ret != TILEXR_SUCCESS) return ret;
    world_->comms[rank_] = this;
    return TILEXR_SUCCESS;
}

int TileXRComm::FinishWorldInit()
{
    TXR_CUDA(cudaSetDevice(device_));
    peerWindows_.assign(rankSize_, nullptr);
    for (int r = 0; r < rankSize_; ++r) {
        TileXRComm *peer = world_->comms[r];
        if (peer == nullptr || peer->window_ == nullptr) return TILEXR_ERROR_INTERNAL;
        if (peer->device_ != device_) {
            cudaError_t e = cudaDeviceEnablePeerAccess(peer->device_, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return TILEXR_ERROR_RUNTIME;
            cudaGetLastError();
        }
        peerWindows_[r] = peer->window_;
    }
    TXR_CUDA(cudaMalloc(reinterpret_cast<void **>(&devArgs_), sizeof(CommArgs)));
    TXR_CUDA(cudaMemset(devArgs_, 0, sizeof(CommArgs)));
    TXR_CUDA(cudaMalloc(reinterpret_cast<void **>(&devRegistry_), sizeof(TileXRRegistry)));
    TXR_CUDA(cudaMemcpy(devRegistry_, &registry_, sizeof(TileXRRegistry), cudaMemcpyHostToDevice));
    TXR_CUDA(cudaMalloc(&localCopyWorkspace_, 4096));
    TXR_CUDA(cudaStreamCreateWithFlags(&copyStream_, cudaStreamNonBlocking));
    TXR_CUDA(cudaEventCreateWithFlags(&copyEventIn_, cudaEventDisableTiming));
    TXR_CUDA(cudaEventCreateWithFlags(&copyEventOut_, cudaEventDisableTiming));
    FillCommArgs();
    int ret = SyncCommArgs();
    if (ret != TILEXR_SUCCESS) return ret;
    initialized_ = true;
    return TILEXR_SUCCESS;
}

// ---- registry -------------------------------------------------------------------------------

int TileXRComm::UploadRegistry()
{
    uint32_t count = 0;
    for (uint32_t h = 0; h < regions_.size(); ++h) {
        const RegionRecord &rec = regions_[h];
        registry_.regions[h].bytes = rec.live ? rec.bytes : 0;
        registry_.regions[h].localBase = rec.live ? rec.localBase : nullptr;
        registry_.regions[h].peerBase = rec.live ? rec.devPeerBase : nullptr;
        registry_.regions[h].mcBase = (rec.live && rec.vmm.live) ? rec.vmm.multicast : nullptr;
        if (rec.live) count = h + 1;
    }
    registry_.regionCount = count;
    hostArgs_->registrationGeneration += 1;
    if (isHostMemory()) return TILEXR_SUCCESS;
    TXR_CUDA(cudaMemcpy(devRegistry_, &registry_, sizeof(TileXRRegistry), cudaMemcpyHostToDevice));
    return SyncCommArgs();
}

int EmulatedWorld::TryFinalizeRegion(TileXRUDMAMemHandle handle)
{
    for (TileXRComm *c : comms) {
        if (c == nullptr || !c->regions()[handle].live) return TILEXR_SUCCESS;   // not everyone yet
    }
    const size_t bytes = comms[0]->regions()[handle].bytes;
    for (TileXRComm *c : comms) {
        if (c->regions()[handle].bytes != bytes) {
            TILEXR_LOG(ERROR) << "ranks registered different sizes under handle " << handle;
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
    }
    for (TileXRComm *c : comms) {
        RegionRecord &rec = c->regions()[handle];
        rec.peerBase.resize(rankSize);
        for (int r = 0; r < rankSize; ++r) rec.peerBase[r] = comms[r]->regions()[handle].localBase;
        if (cudaMemcpy(rec.devPeerBase, rec.peerBase.data(), sizeof(uint8_t *) * rankSize, cudaMemcpyHostToDevice) !=
            cudaSuccess) {
            return TILEXR_ERROR_RUNTIME;
        }
        int ret = c->UploadRegistry();
        if (ret != TILEXR_SUCCESS) return ret;
    }
    return TILEXR_SUCCESS;
}

int TileXRComm::Register(uint8_t *ptr, size_t bytes, bool owned, TileXRUDMAMemHandle *handle)
{
    if (!initialized_) return TILEXR_ERROR_NOT_INITIALIZED;
    if (ptr == nullptr || bytes == 0 || handle == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if ((hostArgs_->extraFlag & TILEXR_FLAG_RMA) == 0) return TILEXR_ERROR_NOT_SUPPORT;
    uint32_t h = 0;
    while (h < regions_.size() && regions_[h].live) ++h;
    if (h == regions_.size()) {
        TILEXR_LOG(ERROR) << "all " << regions_.size() << " registration slots are in use";
        return TILEXR_ERROR_INTERNAL;
    }
    RegionRecord rec;
    rec.live = true;
    rec.ownedAllocation = owned;
    rec.localBase = ptr;
    rec.bytes = bytes;
    rec.peerBase.assign(rankSize_, nullptr);
    rec.peerBase[rank_] = ptr;

    if (isHostMemory()) {
        TILEXR_LOG(ERROR) << "host-memory communicators register only memory from TileXRSymmAlloc";
        return TILEXR_ERROR_NOT_SUPPORT;
    }
    TXR_CUDA(cudaSetDevice(device_));
    TXR_CUDA(cudaMalloc(reinterpret_cast<void **>(&rec.devPeerBase), sizeof(uint8_t *) * rankSize_));

    if (isEmulated()) {
        regions_[h] = rec;
        *handle = h;
        return world_->TryFinalizeRegion(h);
    }

    RegionInfo mine{};
    mine.pid = static_cast<int32_t>(getpid());
    mine.device = device_;
    mine.rawPtr = reinterpret_cast<uint64_t>(ptr);
    mine.bytes = bytes;
    mine.handleIndex = h;
    mine.valid = 1;
    if (opt_.mode == CommMode::PROCESS) {
        uint8_t *base = nullptr;
        size_t allocBytes = 0;
        if (AllocationBase(ptr, &base, &allocBytes) != TILEXR_SUCCESS) {
            mine.valid = 0;
        } else {
            mine.offset = static_cast<uint64_t>(ptr - base);
            if (cudaIpcGetMemHandle(&mine.handle, base) != cudaSuccess) {
                cudaGetLastError();
                mine.valid = 0;
            }
        }
    }
    std::vector<RegionInfo> all(rankSize_);
    int ret = exchange_->AllGather(&mine, all.data(), sizeof(RegionInfo));
    if (ret != TILEXR_SUCCESS) return ret;
    for (int r = 0; r < rankSize_; ++r) {
        if (!all[r].valid || all[r].bytes != bytes || all[r].handleIndex != h) {
            TILEXR_LOG(ERROR) << "registration mismatch with rank " << r << " (valid=" << all[r].valid
                              << " bytes=" << all[r].bytes << " slot=" << all[r].handleIndex << ")";
            cudaFree(rec.devPeerBase);
            return TILEXR_ERROR_PARA_CHECK_FAIL;
        }
    }
    for (int r = 0; r < rankSize_; ++r) {
        if (r == rank_) continue;
        if (all[r].pid == mine.pid) {
            rec.peerBase[r] = reinterpret_cast<uint8_t *>(all[r].rawPtr);
        } else {
            void *mapped = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&mapped, all[r].handle, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                TILEXR_LOG(ERROR) << "cannot map region of rank " << r << ": " << cudaGetErrorString(e);
                for (void *p : rec.ipcOpened) cudaIpcCloseMemHandle(p);
                cudaFree(rec.devPeerBase);
                return TILEXR_ERROR_RUNTIME;
            }
            rec.ipcOpened.push_back(mapped);
            rec.peerBase[r] = static_cast<uint8_t *>(mapped) + all[r].offset;
        }
    }
    TXR_CUDA(cudaMemcpy(rec.devPeerBase, rec.peerBase.data(), sizeof(uint8_t *) * rankSize_, cudaMemcpyHostToDevice));
    regions_[h] = rec;
    *handle = h;
    ret = UploadRegistry();
    if (ret != TILEXR_SUCCESS) return ret;
    return exchange_->Barrier();
}

int TileXRComm::SymmAllocVmm(size_t bytes, void **localPtr, TileXRUDMAMemHandle *handle)
{
    if (!initialized_) return TILEXR_ERROR_NOT_INITIALIZED;
    if (!windowVmm_.live || (hostArgs_->extraFlag & TILEXR_FLAG_RMA) == 0) return TILEXR_ERROR_NOT_SUPPORT;
    uint32_t h = 0;
    while (h < regions_.size() && regions_[h].live) ++h;
    if (h == regions_.size()) {
        TILEXR_LOG(ERROR) << "all " << regions_.size() << " registration slots are in use";
        return TILEXR_ERROR_INTERNAL;
    }
    TXR_CUDA(cudaSetDevice(device_));
    RegionRecord rec;
    int ret = VmmAllocate(*exchange_, rank_, rankSize_, device_, bytes, wantNvls_, vmmTag_ + vmmSeq_++, &rec.vmm);
    if (ret != TILEXR_SUCCESS) return ret;
    rec.live = true;
    rec.ownedAllocation = true;
    rec.localBase = rec.vmm.local;
    rec.bytes = bytes;
    rec.peerBase = rec.vmm.peers;
    TXR_CUDA(cudaMemset(rec.localBase, 0, bytes));
    TXR_CUDA(cudaMalloc(reinterpret_cast<void **>(&rec.devPeerBase), sizeof(uint8_t *) * rankSize_));
    TXR_CUDA(cudaMemcpy(rec.devPeerBase, rec.peerBase.data(), sizeof(uint8_t *) * rankSize_, cudaMemcpyHostToDevice));
    TXR_CUDA(cudaDeviceSynchronize());
    regions_[h] = rec;
    *handle = h;
    *localPtr = rec.localBase;
    ret = UploadRegistry();
    if (ret != TILEXR_SUCCESS) return ret;
    return exchange_->Barrier();
}

int TileXRComm::Unregister(TileXRUDMAMemHandle handle)
{
    if (handle >= regions_.size() || !regions_[handle].live) return TILEXR_ERROR_NOT_FOUND;
    RegionRecord &rec = regions_[handle];
    if (!isHostMemory()) {
        cudaSetDevice(device_);
        for (void *p : rec.ipcOpened) cudaIpcCloseMemHandle(p);
        if (rec.devPeerBase != nullptr) cudaFree(rec.devPeerBase);
        if (rec.vmm.live) {
            // a collective free while the communicator is up (TileXRSymmFree is collective, like the allocation)
            VmmFree(initialized_ && !destroying_ ? exchange_.get() : nullptr, &rec.vmm);
        } else if (rec.ownedAllocation && rec.localBase != nullptr) {
            cudaFree(rec.localBase);
        }
    }
    rec = RegionRecord();
    if (initialized_) UploadRegistry();
    return TILEXR_SUCCESS;
}

int TileXRComm::FindRegistration(const void *ptr, size_t bytes, TileXRUDMAMemHandle *handle, uint64_t *offset) const
{
    const uint8_t *p = static_cast<const uint8_t *>(ptr);
    for (uint32_t h = 0; h < regions_.size(); ++h) {
        const RegionRecord &rec = regions_[h];
        if (!rec.live || rec.peerBase.empty() || rec.peerBase[(rank_ + 1) % rankSize_] == nullptr) continue;
        if (p >= rec.localBase && p + bytes <= rec.localBase + rec.bytes) {
            if (handle != nullptr) *handle = h;
            if (offset != nullptr) *offset = static_cast<uint64_t>(p - rec.localBase);
            return TILEXR_SUCCESS;
        }
    }
    return TILEXR_ERROR_NOT_FOUND;
}

// ---- status ---------------------------------------------------------------------------------

int TileXRComm::DeviceStatus(int *status)
{
    if (!initialized_) return TILEXR_ERROR_NOT_INITIALIZED;
    if (!isHostMemory()) {
        TXR_CUDA(cudaSetDevice(device_));
        TXR_CUDA(cudaMemcpy(hostArgs_->dfx, devArgs_->dfx, sizeof(hostArgs_->dfx), cudaMemcpyDeviceToHost));
    }
    *status = static_cast<int>(hostArgs_->dfx[TILEXR_DFX_FAIL_CODE]);
    return TILEXR_SUCCESS;
}

int TileXRComm::ResetStatus()
{
    if (!initialized_) return TILEXR_ERROR_NOT_INITIALIZED;
    // Cleared: the failure record, the abort word, the grid-barrier pairs with the exit counter, and the
    // operator scratch words (work cursors that a launch returns to zero only when it ends normally).
    // NOT cleared: the launch epoch word.  Flags and the done-epoch table are never reset, they stay valid
    // only as long as the epoch keeps growing; a rank that restarted at epoch 1 would find every flag of
    // its earlier launches already "raised".
    const size_t headBytes = TILEXR_CTRL_EPOCH_WORD * 8;
    const size_t scratchOff = TILEXR_CTRL_SCRATCH_WORD * 8;
    const size_t scratchBytes = TILEXR_CTRL_SCRATCH_WORDS * 8;
    if (isHostMemory()) {
        std::memset(hostArgs_->dfx, 0, sizeof(hostArgs_->dfx));
        std::memset(window_, 0, headBytes);
        std::memset(window_ + scratchOff, 0, scratchBytes);
    } else {
        TXR_CUDA(cudaSetDevice(device_));
        TXR_CUDA(cudaDeviceSynchronize());
        TXR_CUDA(cudaMemset(devArgs_->dfx, 0, sizeof(hostArgs_->dfx)));
        TXR_CUDA(cudaMemset(window_, 0, headBytes));
        TXR_CUDA(cudaMemset(window_ + scratchOff, 0, scratchBytes));
        TXR_CUDA(cudaDeviceSynchronize());
    }
    return isEmulated() ? TILEXR_SUCCESS : HostBarrier();
}

int TileXRComm::HostBarrier()
{
    if (exchange_ == nullptr) return TILEXR_SUCCESS;
    return exchange_->Barrier();
}

void TileXRComm::PrintDfx()
{
    int status = 0;
    if (DeviceStatus(&status) != TILEXR_SUCCESS) return;
    const int64_t *d = hostArgs_->dfx;
    const char *run = d[TILEXR_DFX_RUN_STATUS] == TILEXR_RUN_STARTED    ? "running"
                      : d[TILEXR_DFX_RUN_STATUS] == TILEXR_RUN_FINISHED ? "finished"
                      : d[TILEXR_DFX_RUN_STATUS] == TILEXR_RUN_FAILED   ? "FAILED"
                                                                        : "idle";
    std::ostringstream os;
    os << "DFX rank " << rank_ << ": last op " << TileXROpName(static_cast<int>(d[TILEXR_DFX_OP])) << " magic "
       << d[TILEXR_DFX_MAGIC] << " count " << d[TILEXR_DFX_COUNT_ARG] << " state " << run << " launches "
       << d[TILEXR_DFX_LAUNCHES];
    if (d[TILEXR_DFX_FAIL_CODE] != 0) {
        os << " | failure code " << d[TILEXR_DFX_FAIL_CODE] << " block " << d[TILEXR_DFX_FAIL_BLOCK] << " peer "
           << d[TILEXR_DFX_FAIL_PEER] << " slot " << d[TILEXR_DFX_FAIL_SLOT] << " expected 0x" << std::hex
           << d[TILEXR_DFX_FAIL_EXPECTED] << " observed 0x" << d[TILEXR_DFX_FAIL_OBSERVED];
    }
    // DFX is asked for explicitly, so it is printed at any log level
    std::lock_guard<std::mutex> lock(LogMutex());
    std::fprintf(stdout, "[TileXR] %s\n", os.str().c_str());
    std::fflush(stdout);
}

// Operators whose host side has to stage small per-call arrays on the device (the widened route arrays of EP x TP)
// take them from here instead of allocating per call.  Growing the buffer frees the old one, which waits for the
// device: it happens on the first call of a larger shape only.
int TileXRComm::OperatorScratch(size_t bytes, void **ptr)
{
    if (ptr == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    if (isHostMemory()) return TILEXR_ERROR_NOT_SUPPORT;
    if (bytes > operatorScratchBytes_) {
        TXR_CUDA(cudaSetDevice(device_));
        if (operatorScratch_ != nullptr) {
            TXR_CUDA(cudaDeviceSynchronize());
            TXR_CUDA(cudaFree(operatorScratch_));
            operatorScratch_ = nullptr;
            operatorScratchBytes_ = 0;
        }
        const size_t want = (bytes + (1u << 20) - 1) & ~static_cast<size_t>((1u << 20) - 1);
        TXR_CUDA(cudaMalloc(&operatorScratch_, want));
        operatorScratchBytes_ = want;
    }
    *ptr = operatorScratch_;
    return TILEXR_SUCCESS;
}

int TileXRComm::LocalCopyAsync(void *dst, const void *src, size_t bytes, cudaStream_t stream)
{
    if (!initialized_) return TILEXR_ERROR_NOT_INITIALIZED;
    if (isHostMemory()) {
        std::memcpy(dst, src, bytes);
        return TILEXR_SUCCESS;
    }
    if ((hostArgs_->extraFlag & TILEXR_FLAG_LOCAL_COPY) == 0) {
        TXR_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream));
        return TILEXR_SUCCESS;
    }
    TXR_CUDA(cudaEventRecord(copyEventIn_, stream));
    TXR_CUDA(cudaStreamWaitEvent(copyStream_, copyEventIn_, 0));
    TXR_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, copyStream_));
    TXR_CUDA(cudaEventRecord(copyEventOut_, copyStream_));
    TXR_CUDA(cudaStreamWaitEvent(stream, copyEventOut_, 0));
    return TILEXR_SUCCESS;
}

} // namespace TileXR
