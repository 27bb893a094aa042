// Internal communicator object behind TileXRCommPtr.
//
// One TileXRComm = one rank.  It owns the rank's window, the mappings of every peer's window,
// the host and device copies of CommArgs, the launch-epoch counter and the registry of
// peer-visible user regions.  Operator libraries never include this header: they go through
// the C API (TileXRGetCommArgsDev/Host, TileXRCommNextMagic) and launch.h, the same ownership
// rule the reference keeps between libtile-comm and its operator libraries
// (reference README.md:197-201).
#ifndef TILEXR_COMM_INTERNAL_H
#define TILEXR_COMM_INTERNAL_H

#include <atomic>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "sock_exchange.h"
#include "tilexr_api.h"
#include "vmm.h"

namespace TileXR {

enum class CommMode {
    PROCESS,      // one process per GPU, windows shared through CUDA IPC
    THREAD,       // one thread per GPU inside one process
    EMULATED,     // several ranks on one GPU inside one process (test worlds)
    HOST_MEMORY,  // windows in POSIX shared memory, kernels on CPU threads
};

struct InitOptions {
    int commDomain = 0;
    int bufferMB = TILEXR_COMM_BUFFER_SIZE_MB;
    bool memoryOnly = false;
    CommMode mode = CommMode::PROCESS;
};

struct RegionRecord {
    bool live = false;
    bool ownedAllocation = false;          // TileXRSymmAlloc: freed by TileXRSymmFree/Destroy
    uint8_t *localBase = nullptr;
    size_t bytes = 0;
    std::vector<uint8_t *> peerBase;       // [rankSize], as mapped in this process
    std::vector<void *> ipcOpened;         // bases returned by cudaIpcOpenMemHandle, to close
    uint8_t **devPeerBase = nullptr;       // device copy of peerBase
    VmmAllocation vmm;                     // TileXRSymmAlloc through the virtual-memory API (live when used)
};

struct ProfileRecord {
    bool live = false;
    TileXRUDMAProfileView view{};
};

class EmulatedWorld;

class TileXRComm {
public:
    TileXRComm(int rank, int rankSize, const InitOptions &opt);
    ~TileXRComm();

    int Init(std::unique_ptr<Exchange> exchange);      // PROCESS / THREAD / HOST_MEMORY
    int InitInWorld(std::shared_ptr<EmulatedWorld> world, int device);   // EMULATED
    int FinishWorldInit();                              // after every rank of the world allocated

    int64_t NextMagic() { return magic_.fetch_add(1); }
    int SyncCommArgs();                                 // host copy -> device copy

    int Register(uint8_t *ptr, size_t bytes, bool owned, TileXRUDMAMemHandle *handle);
    // Collective allocation of `bytes` per rank that every rank maps, with a multicast alias where the node
    // offers one; registered like any region.  TILEXR_ERROR_NOT_SUPPORT when this communicator cannot (the
    // caller then allocates with cudaMalloc and registers).
    int SymmAllocVmm(size_t bytes, void **localPtr, TileXRUDMAMemHandle *handle);
    bool usesVmm() const { return windowVmm_.live; }
    uint8_t *windowMulticast() const { return windowVmm_.live ? windowVmm_.multicast : nullptr; }
    int Unregister(TileXRUDMAMemHandle handle);
    int FindRegistration(const void *ptr, size_t bytes, TileXRUDMAMemHandle *handle, uint64_t *offset) const;
    int UploadRegistry();

    int DeviceStatus(int *status);
    int ResetStatus();
    void PrintDfx();
    int HostBarrier();
    int LocalCopyAsync(void *dst, const void *src, size_t bytes, cudaStream_t stream);
    int OperatorScratch(size_t bytes, void **ptr);
    const TileXRPhysicalInfo &physicalInfo() const { return physical_; }      // device memory that lives as long as the communicator, grown on demand

    int rank() const { return rank_; }
    int rankSize() const { return rankSize_; }
    int device() const { return device_; }
    CommMode mode() const { return opt_.mode; }
    bool isHostMemory() const { return opt_.mode == CommMode::HOST_MEMORY; }
    bool isEmulated() const { return opt_.mode == CommMode::EMULATED; }
    CommArgs *hostArgs() { return hostArgs_; }
    CommArgs *devArgs() { return devArgs_; }
    TileXRRegistry *hostRegistry() { return &registry_; }
    TileXRRegistry *devRegistry() { return devRegistry_; }
    EmulatedWorld *world() { return world_.get(); }
    std::vector<RegionRecord> &regions() { return regions_; }
    std::vector<ProfileRecord> &profiles() { return profiles_; }
    uint8_t *window() { return window_; }
    bool initialized() const { return initialized_; }

private:
    int AllocateWindow();
    int TryVmmWindow();
    int ExchangeWindows();
    int MapHostMemoryWindows();
    void FillCommArgs();
    int AgreeOnKnobs();

    int rank_;
    int rankSize_;
    InitOptions opt_;
    int device_ = -1;
    bool initialized_ = false;
    std::unique_ptr<Exchange> exchange_;
    std::shared_ptr<EmulatedWorld> world_;

    size_t windowBytes_ = 0;
    uint8_t *window_ = nullptr;
    std::vector<uint8_t *> peerWindows_;
    std::vector<void *> ipcOpened_;
    std::vector<std::string> shmNames_;
    VmmAllocation windowVmm_;             // live when the window came from the virtual-memory API
    uint64_t vmmTag_ = 0;                 // names the descriptor sockets of this communicator's allocations
    uint32_t vmmSeq_ = 0;
    bool wantVmm_ = true;
    bool wantNvls_ = true;
    bool destroying_ = false;             // regions released by the destructor do not meet the peers one by one

    CommArgs *hostArgs_ = nullptr;
    CommArgs *devArgs_ = nullptr;
    TileXRRegistry registry_{};
    TileXRRegistry *devRegistry_ = nullptr;
    std::vector<RegionRecord> regions_;
    std::vector<ProfileRecord> profiles_;
    void *localCopyWorkspace_ = nullptr;
    void DetectTopology(const std::vector<int> &peerDevices);
    TileXRPhysicalInfo physical_{};
    void *operatorScratch_ = nullptr;
    size_t operatorScratchBytes_ = 0;
    cudaStream_t copyStream_ = nullptr;
    cudaEvent_t copyEventIn_ = nullptr;
    cudaEvent_t copyEventOut_ = nullptr;
    std::atomic<int64_t> magic_{1};
    uint64_t waitTimeoutNs_ = 0;
    uint32_t knobFlags_ = 0;
    friend class EmulatedWorld;
};

// The ranks of an emulated world share one device; this object lets their single-threaded
// "collective" host calls (registration) complete without a blocking exchange, and gathers
// their kernel launches into one cooperative launch (see launch.h).
class EmulatedWorld {
public:
    EmulatedWorld(int rankSize, int device) : rankSize(rankSize), device(device), comms(rankSize, nullptr) {}
    int rankSize;
    int device;
    std::vector<TileXRComm *> comms;
    // Completes region `handle` once every rank has registered it.
    int TryFinalizeRegion(TileXRUDMAMemHandle handle);
};

uint64_t DefaultWaitTimeoutNs();

} // namespace TileXR

#endif
