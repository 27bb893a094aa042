// Portability layer under every TileXR device header.
//
// Compiled by nvcc for sm_100a the primitives below are inline PTX with system scope
// (a peer GPU behind NVSwitch is "system" to the memory model).  Compiled by a host
// compiler the same names are implemented with GCC atomics, so that the flag, registry and
// data-as-flag logic can be unit-tested on a CPU and reused by the host-memory communicator
// (windows in POSIX shared memory, "blocks" as threads).  The reference tests its device
// headers the same way with a stub kernel_operator.h (tests/udma/unit/stubs/kernel_operator.h).
#ifndef TILEXR_PLATFORM_CUH
#define TILEXR_PLATFORM_CUH

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define TXR_HD __host__ __device__ __forceinline__
#define TXR_D __device__ __forceinline__
#else
#define TXR_HD inline
#define TXR_D inline
#include <time.h>
#endif

#if defined(__CUDA_ARCH__)
#define TXR_ON_DEVICE 1
#else
#define TXR_ON_DEVICE 0
#endif

namespace tilexr {

// ---- host builds only: observation points for a protocol trace --------------------------------
// When the flag and window primitives below run on a CPU (the host-memory communicator), a recorder can watch
// them: every flag store, every wait that ends, every copy into a window and every read out of one.  The protocol
// checker analyses what the PRODUCTION code did, not a model of it (the reference replays its kernel headers through
// shims for the same purpose: tools/checker/shim/tilexr/checker/collective_trace_shim.h).  A null slot costs one
// thread-local load per call; device code has none of this.
#if !TXR_ON_DEVICE
struct HostTraceHooks {
    void (*onFlagStore)(void *ctx, const void *addr, uint64_t value);                  // BEFORE the store is performed
    void (*onFlagWait)(void *ctx, const void *addr, uint64_t want, uint64_t seen, int peer, int satisfied);   // when the wait ends
    void (*onCopy)(void *ctx, const void *dst, const void *src, uint64_t bytes);       // BEFORE a copy into a window
    void (*onRead)(void *ctx, const void *src, uint64_t bytes);                        // a read out of a window
    void *ctx;
    uint64_t epoch;                                                                    // of the launch that is running (set by its prologue)
};
inline HostTraceHooks *&HostTraceSlot()
{
    static thread_local HostTraceHooks *hooks = nullptr;
    return hooks;
}
#endif

// ---- 64-bit flag words --------------------------------------------------------------------

TXR_D void st_release_sys_u64(uint64_t *p, uint64_t v)
{
#if TXR_ON_DEVICE
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
    if (HostTraceHooks *h = HostTraceSlot()) h->onFlagStore(h->ctx, p, v);
    __atomic_store_n(p, v, __ATOMIC_RELEASE);
#endif
}

TXR_D void st_relaxed_sys_u64(uint64_t *p, uint64_t v)
{
#if TXR_ON_DEVICE
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
    if (HostTraceHooks *h = HostTraceSlot()) h->onFlagStore(h->ctx, p, v);
    __atomic_store_n(p, v, __ATOMIC_RELAXED);
#endif
}

TXR_D uint64_t ld_acquire_sys_u64(const uint64_t *p)
{
#if TXR_ON_DEVICE
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
#else
    return __atomic_load_n(p, __ATOMIC_ACQUIRE);
#endif
}

TXR_D uint64_t ld_relaxed_sys_u64(const uint64_t *p)
{
#if TXR_ON_DEVICE
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
#else
    return __atomic_load_n(p, __ATOMIC_RELAXED);
#endif
}

TXR_D uint32_t ld_acquire_sys_u32(const uint32_t *p)
{
#if TXR_ON_DEVICE
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
#else
    return __atomic_load_n(p, __ATOMIC_ACQUIRE);
#endif
}

TXR_D void st_release_sys_u32(uint32_t *p, uint32_t v)
{
#if TXR_ON_DEVICE
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
#else
    __atomic_store_n(p, v, __ATOMIC_RELEASE);
#endif
}

TXR_D uint32_t ld_acquire_gpu_u32(const uint32_t *p)
{
#if TXR_ON_DEVICE
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
#else
    return __atomic_load_n(p, __ATOMIC_ACQUIRE);
#endif
}

TXR_D void st_release_gpu_u32(uint32_t *p, uint32_t v)
{
#if TXR_ON_DEVICE
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
#else
    __atomic_store_n(p, v, __ATOMIC_RELEASE);
#endif
}

// add with release semantics at system scope, result discarded ("signal add")
TXR_D void red_release_sys_add_u64(uint64_t *p, uint64_t v)
{
#if TXR_ON_DEVICE
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
    __atomic_fetch_add(p, v, __ATOMIC_RELEASE);
#endif
}

TXR_D uint32_t atom_add_acq_rel_gpu_u32(uint32_t *p, uint32_t v)
{
#if TXR_ON_DEVICE
    uint32_t old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
#else
    return __atomic_fetch_add(p, v, __ATOMIC_ACQ_REL);
#endif
}

TXR_D uint64_t atom_cas_sys_u64(uint64_t *p, uint64_t expected, uint64_t desired)
{
#if TXR_ON_DEVICE
    uint64_t old;
    asm volatile("atom.acq_rel.sys.global.cas.b64 %0, [%1], %2, %3;"
                 : "=l"(old) : "l"(p), "l"(expected), "l"(desired) : "memory");
    return old;
#else
    __atomic_compare_exchange_n(p, &expected, desired, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE);
    return expected;
#endif
}

TXR_D void fence_acq_rel_sys()
{
#if TXR_ON_DEVICE
    asm volatile("fence.acq_rel.sys;" ::: "memory");
#else
    __atomic_thread_fence(__ATOMIC_SEQ_CST);
#endif
}

// Makes earlier generic-proxy writes visible to the async proxy (TMA) and vice versa.
TXR_D void fence_proxy_async()
{
#if TXR_ON_DEVICE
    asm volatile("fence.proxy.async;" ::: "memory");
#endif
}

// ---- time ---------------------------------------------------------------------------------

TXR_D uint64_t now_ns()
{
#if TXR_ON_DEVICE
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
#else
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
#endif
}

TXR_D void spin_pause()
{
#if TXR_ON_DEVICE
    __nanosleep(20);
#else
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
#endif
}

// ---- 16-byte data movement ------------------------------------------------------------------

struct alignas(16) Vec16 {
    uint32_t x, y, z, w;
};

TXR_D Vec16 ld_vec16(const void *p)
{
#if TXR_ON_DEVICE
    Vec16 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
#else
    Vec16 v;
    memcpy(&v, p, 16);
    return v;
#endif
}

// Streaming load: data that is read once (a peer window, a ring slot) should not displace
// the reusable working set from L1.
TXR_D Vec16 ld_vec16_stream(const void *p)
{
#if TXR_ON_DEVICE
    Vec16 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
#else
    return ld_vec16(p);
#endif
}

// Load that must observe another GPU's latest stores without an acquire on the same
// address (data-as-flag polling): relaxed at system scope, never served from L1.
TXR_D Vec16 ld_vec16_volatile(const void *p)
{
#if TXR_ON_DEVICE
    Vec16 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
#else
    Vec16 v;
    const uint64_t *q = reinterpret_cast<const uint64_t *>(p);
    uint64_t hi = __atomic_load_n(q + 1, __ATOMIC_ACQUIRE);   // epoch word lives in the upper half
    uint64_t lo = __atomic_load_n(q, __ATOMIC_RELAXED);
    memcpy(&v, &lo, 8);
    memcpy(reinterpret_cast<char *>(&v) + 8, &hi, 8);
    return v;
#endif
}

TXR_D void st_vec16(void *p, const Vec16 &v)
{
#if TXR_ON_DEVICE
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
#else
    memcpy(p, &v, 16);
#endif
}

// One 16-byte store whose last word is a flag/epoch.  On the GPU a 16-byte aligned vector
// store is performed as a single transaction, which is what lets a reader treat the epoch
// word as proof that the other twelve bytes arrived (the LL protocol of NCCL relies on the
// same property).  On the host the payload is written first and the epoch half released last.
TXR_D void st_vec16_flagged(void *p, const Vec16 &v)
{
#if TXR_ON_DEVICE
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
#else
    uint64_t lo, hi;
    memcpy(&lo, &v, 8);
    memcpy(&hi, reinterpret_cast<const char *>(&v) + 8, 8);
    uint64_t *q = reinterpret_cast<uint64_t *>(p);
    __atomic_store_n(q, lo, __ATOMIC_RELAXED);
    __atomic_store_n(q + 1, hi, __ATOMIC_RELEASE);
#endif
}

} // namespace tilexr

#endif // TILEXR_PLATFORM_CUH
