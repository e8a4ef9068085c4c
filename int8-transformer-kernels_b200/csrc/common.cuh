// Shared host/device helpers for the i8tk kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/i8tk.h"

namespace i8tk {

// ---- host-side error plumbing -------------------------------------------
void set_error(const char* fmt, ...);   // defined in status.cu (thread-local buffer)

#define I8TK_REQUIRE(cond, code, ...)            \
    do {                                          \
        if (!(cond)) {                            \
            ::i8tk::set_error(__VA_ARGS__);       \
            return (code);                        \
        }                                         \
    } while (0)

#define I8TK_CUDA(call)                                                        \
    do {                                                                       \
        cudaError_t e__ = (call);                                              \
        if (e__ != cudaSuccess) {                                              \
            ::i8tk::set_error("%s failed: %s", #call, cudaGetErrorString(e__)); \
            return I8TK_ERR_CUDA;                                              \
        }                                                                      \
    } while (0)

inline bool aligned_to(const void* p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Status block at the start of every workspace (two 32-bit words):
//   word 0  receives this magic value when a bounded wait of the CURRENT call runs out; the
//           first kernel of every call clears it, so what it shows belongs to the last call
//   word 1  counts such give-ups and is never cleared by a kernel: a caller that zeroes it
//           once can look at it as rarely as it likes and still learn that some call failed
constexpr uint32_t kDeviceTimeoutMagic = 0xD1E7E0u;
// Same two words, other cause: an index read on the device (a page id) lay outside the bound
// the caller gave; the kernel used a valid one in its place so that nothing is read out of range.
constexpr uint32_t kDeviceBadIndexMagic = 0xBAD1D0u;

// ---- device helpers -----------------------------------------------------
#ifdef __CUDACC__

// A bounded wait gave up: mark the call and bump the sticky count (see kDeviceTimeoutMagic).
__device__ __forceinline__ void note_timeout(uint32_t* status) {
    atomicExch(status, kDeviceTimeoutMagic);
    atomicAdd(status + 1, 1u);
}
__device__ __forceinline__ void note_bad_index(uint32_t* status) {
    atomicExch(status, kDeviceBadIndexMagic);
    atomicAdd(status + 1, 1u);
}
// Run by one thread of the first kernel of a call, before anything of that call can give up.
__device__ __forceinline__ void clear_call_status(uint32_t* status) { *status = 0u; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// 16-byte asynchronous copy global -> shared (LSU path, not the bulk engine), and the hook that
// makes an mbarrier wait for this thread's copies issued so far: the barrier's pending count goes
// up by one now and down by one when they have landed.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// One poll of the barrier phase.  `suspend_ns` lets the hardware park the
// thread until the phase completes or that much time has passed, instead of
// burning issue slots in a spin loop.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity,
                                              uint32_t suspend_ns = 20000u) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(suspend_ns)
        : "memory");
    return ok != 0;
}

// Bounded wait: returns false (after `limit` polls, each parked for at most
// the suspend hint -- about a second in total) instead of waiting forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  uint32_t limit = (1u << 16)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Latency-critical variant: polls without a suspend hint (the hinted form backs
// off with nanosleep, which adds wake-up latency to every wait).  Still bounded.
__device__ __forceinline__ bool mbar_wait_spin_bounded(uint32_t bar, uint32_t parity,
                                                       uint32_t limit = (1u << 24)) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// 1-D bulk async copy global -> shared, completion counted on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// The same copy with an L2 eviction-priority hint (a policy from l2_policy_evict_first()).
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// ---- thread-block clusters ---------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// every thread of every CTA of the cluster
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}

// Programmatic dependent launch: a kernel launched with launch_after() may start while the
// kernel before it in the stream is still running; it must call pdl_wait() before it touches
// anything that kernel writes (the wait returns once that grid has completed and its writes
// are visible; it returns at once in a kernel launched the ordinary way).  The earlier kernel
// calls pdl_launch_dependents() to let the later one be scheduled as SMs become free.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Packed fp32x2 arithmetic (one instruction for two lanes of a register pair), through the
// float2 intrinsics of sm_100: as a typed pair the compiler keeps the two halves in an aligned
// register pair from where they are produced, which the same instructions written as inline
// PTX on 64-bit operands did not always manage (2-4 % of an MLP forward went into moves).
typedef float2 f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 unpack2(f32x2 v) { return v; }

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { return __fmul2_rn(a, b); }

// The same operations as inline PTX on 64-bit operands, for the one kernel family that is
// faster with them (the LayerNorm + quantiser pass holds a whole row in such pairs: with the
// typed form its 2048-column variant went from 67 to 115 us on 65536 rows).
namespace asm2 {
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    float2 t = make_float2(a, b);
    return *reinterpret_cast<f32x2*>(&t);
}
__device__ __forceinline__ float2 unpack2(f32x2 v) { return *reinterpret_cast<float2*>(&v); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
}  // namespace asm2

#endif  // __CUDACC__

#ifdef __CUDACC__
// Launch `kernel` so that it may overlap the tail of the previous kernel in `st`
// (programmatic stream serialisation); see pdl_wait().
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the CTAs of the grid grouped into clusters of `cluster_x` along x (1: no clusters).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                          int cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
    if (cluster_x > 1) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)cluster_x;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

}  // namespace i8tk
