#include "vmm.h"

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <poll.h>
#include <string>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cuda.h>
#include <cuda_runtime_api.h>

#include "sock_exchange.h"
#include "tilexr_log.h"
#include "tilexr_types.h"

namespace TileXR {

namespace {

// ---- driver entry points -------------------------------------------------------------------------------------
// The library does not link libcuda (it must load on machines without a driver, for the CPU plumbing mode); the
// runtime hands out the driver's entry points.

struct Driver {
    CUresult (*memCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long) = nullptr;
    CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*memAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*memAddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t) = nullptr;
    CUresult (*memExport)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*memImport)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType) = nullptr;
    CUresult (*memGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*mcCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *) = nullptr;
    CUresult (*mcAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
    CUresult (*mcBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
    CUresult (*mcUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
    CUresult (*mcGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags) = nullptr;
    CUresult (*deviceGet)(CUdevice *, int) = nullptr;
    CUresult (*deviceGetAttribute)(int *, CUdevice_attribute, CUdevice) = nullptr;
    bool core = false;        // everything but the multicast calls
    bool multicast = false;
};

template <typename Fn>
bool Resolve(const char *name, Fn *out)
{
    void *f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess || f == nullptr ||
        q != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        *out = nullptr;
        return false;
    }
    *out = reinterpret_cast<Fn>(f);
    return true;
}

const Driver &Drv()
{
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        bool ok = true;
        ok &= Resolve("cuMemCreate", &d.memCreate);
        ok &= Resolve("cuMemRelease", &d.memRelease);
        ok &= Resolve("cuMemAddressReserve", &d.memAddressReserve);
        ok &= Resolve("cuMemAddressFree", &d.memAddressFree);
        ok &= Resolve("cuMemMap", &d.memMap);
        ok &= Resolve("cuMemUnmap", &d.memUnmap);
        ok &= Resolve("cuMemSetAccess", &d.memSetAccess);
        ok &= Resolve("cuMemExportToShareableHandle", &d.memExport);
        ok &= Resolve("cuMemImportFromShareableHandle", &d.memImport);
        ok &= Resolve("cuMemGetAllocationGranularity", &d.memGranularity);
        ok &= Resolve("cuDeviceGet", &d.deviceGet);
        ok &= Resolve("cuDeviceGetAttribute", &d.deviceGetAttribute);
        d.core = ok;
        bool mc = ok;
        mc &= Resolve("cuMulticastCreate", &d.mcCreate);
        mc &= Resolve("cuMulticastAddDevice", &d.mcAddDevice);
        mc &= Resolve("cuMulticastBindMem", &d.mcBindMem);
        mc &= Resolve("cuMulticastUnbind", &d.mcUnbind);
        mc &= Resolve("cuMulticastGetGranularity", &d.mcGranularity);
        d.multicast = mc;
    });
    return d;
}

// ---- descriptors over Unix domain sockets ----------------------------------------------------------------------
// A POSIX descriptor only means something inside its process; SCM_RIGHTS over a Unix socket is how the kernel
// copies one into another process.  Abstract socket names (leading NUL) need no file and vanish with the socket.

struct FdMessage {
    int32_t srcRank;
    int32_t kind;        // 0: a rank's memory, 1: the multicast object
};

socklen_t AbstractAddress(uint64_t tag, int rank, sockaddr_un *addr)
{
    std::memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    const int n = std::snprintf(addr->sun_path + 1, sizeof(addr->sun_path) - 1, "tilexr-vmm-%016llx-%d",
                                static_cast<unsigned long long>(tag), rank);
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int Listen(uint64_t tag, int rank, int backlog)
{
    const int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    sockaddr_un addr;
    const socklen_t len = AbstractAddress(tag, rank, &addr);
    if (bind(fd, reinterpret_cast<sockaddr *>(&addr), len) != 0 || listen(fd, backlog) != 0) {
        close(fd);
        return -1;
    }
    return fd;
}

bool SendFd(uint64_t tag, int dstRank, int fdToSend, int srcRank, int kind)
{
    const int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) return false;
    sockaddr_un addr;
    const socklen_t len = AbstractAddress(tag, dstRank, &addr);
    if (connect(s, reinterpret_cast<sockaddr *>(&addr), len) != 0) {
        close(s);
        return false;
    }
    FdMessage body{srcRank, kind};
    iovec iov{&body, sizeof(body)};
    alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
    std::memset(control, 0, sizeof(control));
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = control;
    msg.msg_controllen = sizeof(control);
    cmsghdr *c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fdToSend, sizeof(int));
    const bool ok = sendmsg(s, &msg, 0) == static_cast<ssize_t>(sizeof(body));
    close(s);
    return ok;
}

// One message from whoever connects next; gives up after `timeoutMs`.
bool RecvFd(int listenFd, int timeoutMs, int *fdOut, FdMessage *body)
{
    pollfd p{listenFd, POLLIN, 0};
    if (poll(&p, 1, timeoutMs) <= 0) return false;
    const int s = accept4(listenFd, nullptr, nullptr, SOCK_CLOEXEC);
    if (s < 0) return false;
    iovec iov{body, sizeof(*body)};
    alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = control;
    msg.msg_controllen = sizeof(control);
    pollfd ps{s, POLLIN, 0};
    bool ok = poll(&ps, 1, timeoutMs) > 0 && recvmsg(s, &msg, MSG_CMSG_CLOEXEC) == static_cast<ssize_t>(sizeof(*body));
    close(s);
    if (!ok) return false;
    cmsghdr *c = CMSG_FIRSTHDR(&msg);
    if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return false;
    std::memcpy(fdOut, CMSG_DATA(c), sizeof(int));
    return true;
}

// Every rank learns whether every rank is still fine; the verdict is the same everywhere.
bool AllOk(Exchange &ex, int rankSize, bool mine)
{
    int32_t v = mine ? 1 : 0;
    std::vector<int32_t> all(rankSize, 0);
    if (ex.AllGather(&v, all.data(), sizeof(v)) != TILEXR_SUCCESS) return false;
    for (int32_t x : all) {
        if (x == 0) return false;
    }
    return true;
}

size_t RoundUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

CUmemAllocationProp DeviceProp(int ordinal)
{
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = ordinal;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

// Reserves an address range and maps `handle` into it with read/write access for `ordinal`.
uint8_t *MapHandle(const Driver &d, CUmemGenericAllocationHandle handle, size_t bytes, size_t align, int ordinal)
{
    CUdeviceptr va = 0;
    if (d.memAddressReserve(&va, bytes, align, 0, 0) != CUDA_SUCCESS) return nullptr;
    if (d.memMap(va, bytes, 0, handle, 0) != CUDA_SUCCESS) {
        d.memAddressFree(va, bytes);
        return nullptr;
    }
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = ordinal;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (d.memSetAccess(va, bytes, &access, 1) != CUDA_SUCCESS) {
        d.memUnmap(va, bytes);
        d.memAddressFree(va, bytes);
        return nullptr;
    }
    return reinterpret_cast<uint8_t *>(va);
}

void Unmap(const Driver &d, uint8_t *p, size_t bytes)
{
    if (p == nullptr) return;
    d.memUnmap(reinterpret_cast<CUdeviceptr>(p), bytes);
    d.memAddressFree(reinterpret_cast<CUdeviceptr>(p), bytes);
}

// Lets go of everything `a` holds on this rank (no meeting with the peers).
void ReleaseLocal(VmmAllocation *a)
{
    const Driver &d = Drv();
    if (!d.core) return;
    if (a->multicast != nullptr) Unmap(d, a->multicast, a->mappedBytes);
    a->multicast = nullptr;
    if (a->mcHandle != 0) {
        if (a->mcBound) {
            CUdevice dev = 0;
            if (d.deviceGet(&dev, a->device) == CUDA_SUCCESS) d.mcUnbind(a->mcHandle, dev, 0, a->mappedBytes);
            a->mcBound = false;
        }
        d.memRelease(a->mcHandle);
        a->mcHandle = 0;
    }
    for (size_t r = 0; r < a->peers.size(); ++r) {
        if (a->peers[r] != nullptr && a->peers[r] != a->local) Unmap(d, a->peers[r], a->mappedBytes);
        if (r < a->peerHandles.size() && a->peerHandles[r] != 0) d.memRelease(a->peerHandles[r]);
    }
    a->peers.clear();
    a->peerHandles.clear();
    if (a->local != nullptr) Unmap(d, a->local, a->mappedBytes);
    a->local = nullptr;
    if (a->memHandle != 0) d.memRelease(a->memHandle);
    a->memHandle = 0;
    a->live = false;
}

} // namespace

int VmmDeviceSupport(int device, bool *vmm, bool *multicast)
{
    *vmm = false;
    *multicast = false;
    const Driver &d = Drv();
    if (!d.core) return TILEXR_SUCCESS;
    CUdevice dev = 0;
    if (d.deviceGet(&dev, device) != CUDA_SUCCESS) return TILEXR_ERROR_RUNTIME;
    int v = 0;
    if (d.deviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev) == CUDA_SUCCESS && v != 0) {
        int fdOk = 0;
        d.deviceGetAttribute(&fdOk, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
        *vmm = fdOk != 0;
    }
    if (*vmm && d.multicast) {
        int m = 0;
        if (d.deviceGetAttribute(&m, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) *multicast = m != 0;
    }
    return TILEXR_SUCCESS;
}

int VmmAllocate(Exchange &ex, int rank, int rankSize, int device, size_t bytes, bool wantMulticast, uint64_t tag,
                VmmAllocation *out)
{
    const Driver &d = Drv();
    *out = VmmAllocation();
    out->device = device;
    out->bytes = bytes;
    constexpr int TIMEOUT_MS = 30000;

    // ---- phase 0: does everybody have the API, and the multicast object if it is wanted? -----------------------
    bool vmm = false, mcOk = false;
    const bool probed = VmmDeviceSupport(device, &vmm, &mcOk) == TILEXR_SUCCESS;
    if (!AllOk(ex, rankSize, probed && vmm)) return TILEXR_ERROR_NOT_SUPPORT;
    const bool multicast = wantMulticast && rankSize > 1 && AllOk(ex, rankSize, mcOk);

    // ---- phase 1: sizes, own memory, listening socket ------------------------------------------------------------
    CUmemAllocationProp prop = DeviceProp(device);
    size_t gran = 0;
    bool ok = d.memGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && gran != 0;
    CUmulticastObjectProp mcProp{};
    if (ok && multicast) {
        mcProp.numDevices = static_cast<unsigned int>(rankSize);
        mcProp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        mcProp.size = RoundUp(bytes, gran);
        size_t mcGran = 0;
        ok = d.mcGranularity(&mcGran, &mcProp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mcGran != 0;
        if (ok) gran = gran > mcGran ? RoundUp(gran, mcGran) : RoundUp(mcGran, gran);
    }
    const size_t mapped = ok ? RoundUp(bytes, gran) : 0;
    out->mappedBytes = mapped;
    mcProp.size = mapped;
    int myFd = -1;
    int listenFd = -1;
    if (ok) {
        CUmemGenericAllocationHandle h = 0;
        ok = d.memCreate(&h, mapped, &prop, 0) == CUDA_SUCCESS;
        if (ok) {
            out->memHandle = h;
            ok = d.memExport(&myFd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS && myFd >= 0;
        }
        if (ok) {
            out->local = MapHandle(d, h, mapped, gran, device);
            ok = out->local != nullptr;
        }
        if (ok && rankSize > 1) {
            listenFd = Listen(tag, rank, rankSize + 1);
            ok = listenFd >= 0;
        }
    }
    if (!AllOk(ex, rankSize, ok)) {      // also the meeting after which every rank is listening
        if (myFd >= 0) close(myFd);
        if (listenFd >= 0) close(listenFd);
        ReleaseLocal(out);
        TILEXR_LOG(INFO) << "rank " << rank << ": symmetric memory through the virtual-memory API is not available here";
        return TILEXR_ERROR_NOT_SUPPORT;
    }

    // ---- phase 2: trade descriptors, map the peers -----------------------------------------------------------------
    out->peers.assign(rankSize, nullptr);
    out->peerHandles.assign(rankSize, 0);
    out->peers[rank] = out->local;
    for (int i = 1; ok && i < rankSize; ++i) {
        const int peer = (rank + i) % rankSize;
        ok = SendFd(tag, peer, myFd, rank, 0);
    }
    for (int i = 1; ok && i < rankSize; ++i) {
        int fd = -1;
        FdMessage m{};
        ok = RecvFd(listenFd, TIMEOUT_MS, &fd, &m) && m.kind == 0 && m.srcRank >= 0 && m.srcRank < rankSize && m.srcRank != rank &&
             out->peerHandles[m.srcRank] == 0;
        if (ok) {
            CUmemGenericAllocationHandle h = 0;
            ok = d.memImport(&h, reinterpret_cast<void *>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
            if (ok) {
                out->peerHandles[m.srcRank] = h;
                out->peers[m.srcRank] = MapHandle(d, h, mapped, gran, device);
                ok = out->peers[m.srcRank] != nullptr;
            }
        }
        if (fd >= 0) close(fd);
    }
    if (myFd >= 0) close(myFd);
    if (!AllOk(ex, rankSize, ok)) {
        if (listenFd >= 0) close(listenFd);
        ReleaseLocal(out);
        TILEXR_LOG(WARN) << "rank " << rank << ": the exchange of memory descriptors failed";
        return TILEXR_ERROR_NOT_SUPPORT;
    }

    // ---- phase 3: the multicast object (optional; a refusal leaves the peer mappings in place) ----------------------
    if (multicast) {
        bool mc = true;
        CUdevice dev = 0;
        mc = d.deviceGet(&dev, device) == CUDA_SUCCESS;
        if (rank == 0) {
            CUmemGenericAllocationHandle h = 0;
            mc = mc && d.mcCreate(&h, &mcProp) == CUDA_SUCCESS;
            int mcFd = -1;
            if (mc) {
                out->mcHandle = h;
                mc = d.memExport(&mcFd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS && mcFd >= 0;
            }
            // the others wait for a message in any case: a failed root says so with kind 2
            for (int peer = 1; peer < rankSize; ++peer) {
                int sendFd = mc ? mcFd : listenFd;
                if (!SendFd(tag, peer, sendFd, 0, mc ? 1 : 2)) mc = false;
            }
            if (mcFd >= 0) close(mcFd);
        } else {
            int fd = -1;
            FdMessage m{};
            mc = RecvFd(listenFd, TIMEOUT_MS, &fd, &m) && mc;
            if (mc && m.kind == 1) {
                CUmemGenericAllocationHandle h = 0;
                mc = d.memImport(&h, reinterpret_cast<void *>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
                if (mc) out->mcHandle = h;
            } else {
                mc = false;
            }
            if (fd >= 0) close(fd);
        }
        mc = mc && d.mcAddDevice(out->mcHandle, dev) == CUDA_SUCCESS;
        mc = AllOk(ex, rankSize, mc);                 // every device has joined before anybody binds
        if (mc) {
            const bool bound = d.mcBindMem(out->mcHandle, 0, out->memHandle, 0, mapped, 0) == CUDA_SUCCESS;
            out->mcBound = bound;
            mc = AllOk(ex, rankSize, bound);
        }
        if (mc) {
            out->multicast = MapHandle(d, out->mcHandle, mapped, gran, device);
            mc = AllOk(ex, rankSize, out->multicast != nullptr);
        }
        if (!mc) {
            // keep the unicast mappings, drop what exists of the multicast side
            if (out->multicast != nullptr) Unmap(d, out->multicast, mapped);
            out->multicast = nullptr;
            if (out->mcHandle != 0) {
                if (out->mcBound) d.mcUnbind(out->mcHandle, dev, 0, mapped);
                out->mcBound = false;
                d.memRelease(out->mcHandle);
                out->mcHandle = 0;
            }
            TILEXR_LOG(INFO) << "rank " << rank << ": no NVLink multicast object for this allocation; collectives use peer-to-peer kernels";
        }
    }
    if (listenFd >= 0) close(listenFd);
    out->live = true;
    return TILEXR_SUCCESS;
}

int VmmFree(Exchange *ex, VmmAllocation *a)
{
    if (a == nullptr || !a->live) return TILEXR_SUCCESS;
    // nobody unbinds while a peer may still run a kernel that uses the alias
    cudaDeviceSynchronize();
    if (ex != nullptr) ex->Barrier();
    ReleaseLocal(a);
    return TILEXR_SUCCESS;
}

} // namespace TileXR

// ---- host-side self tests (no GPU involved) ------------------------------------------------------------------------------

extern "C" {

// What this host offers the symmetric allocator: *vmm / *multicast are 0 on a machine without a CUDA driver (the library
// resolves the driver's entry points at run time and loads anywhere), and the caller then takes cudaMalloc + CUDA IPC.
int TileXRVmmQuerySupport(int device, int *vmm, int *multicast)
{
    if (vmm == nullptr || multicast == nullptr) return TileXR::TILEXR_ERROR_PARA_CHECK_FAIL;
    bool v = false, m = false;
    const int ret = TileXR::VmmDeviceSupport(device, &v, &m);
    *vmm = v ? 1 : 0;
    *multicast = m ? 1 : 0;
    return ret;
}

// The descriptor hand-over that carries a rank's memory to its peers, run inside one process: a listener named after
// (tag, rank), a sender that passes `fd` with the (source rank, kind) header, and the received descriptor written to
// *received (the caller closes it).  Returns 0, or which step failed (1 listen, 2 send, 3 receive, 4 header).  A second
// listener on the same name must be refused (5 when it is not): the name is the rendezvous.
int TileXRVmmDescriptorSelfTest(uint64_t tag, int rank, int fd, int srcRank, int kind, int *received)
{
    using namespace TileXR;
    if (received == nullptr) return TILEXR_ERROR_PARA_CHECK_FAIL;
    *received = -1;
    const int listener = Listen(tag, rank, 4);
    if (listener < 0) return 1;
    const int second = Listen(tag, rank, 4);
    if (second >= 0) {
        close(second);
        close(listener);
        return 5;
    }
    int step = 0;
    if (!SendFd(tag, rank, fd, srcRank, kind)) {
        step = 2;
    } else {
        FdMessage body{-1, -1};
        int got = -1;
        if (!RecvFd(listener, 2000, &got, &body)) {
            step = 3;
        } else if (body.srcRank != srcRank || body.kind != kind) {
            close(got);
            step = 4;
        } else {
            *received = got;
        }
    }
    close(listener);
    return step;
}

// Nobody listens on (tag, rank): the send must fail at once instead of blocking, and a receive must give up after its budget.
int TileXRVmmDescriptorNobodyThere(uint64_t tag, int rank, int fd)
{
    using namespace TileXR;
    if (SendFd(tag, rank, fd, 0, 0)) return 1;
    const int listener = Listen(tag, rank, 1);
    if (listener < 0) return 2;
    FdMessage body{-1, -1};
    int got = -1;
    const bool received = RecvFd(listener, 50, &got, &body);
    close(listener);
    if (received) {
        close(got);
        return 3;
    }
    return 0;
}

} // extern "C"
