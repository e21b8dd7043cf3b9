// Device-side building blocks shared by the sm_100a kernels: mbarrier, TMA copies
// (tiled tensor form and untiled bulk form) and bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nmspmm {

constexpr int kVecLen = 32;     // columns of B that share one index list (VEC_LEN of the reference API)

// Status word values written by kernels whose bounded waits gave up.
constexpr int kDevOk = 0;
constexpr int kDevTimeoutFull = 1;    // a consumer never saw its stage filled
constexpr int kDevTimeoutEmpty = 2;   // the producer never saw its stage released
constexpr int kDevTimeoutMma = 3;     // the epilogue never saw the tensor core finish

// Upper bound of one wait, in SM clock cycles (about a second).
constexpr long long kWaitCycleLimit = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Whole (converged) warp: true in exactly one thread.  The branch it guards is the place
// for instructions one thread issues on the warp's behalf (TMA copies, tcgen05.mma,
// tcgen05.commit): the compiler knows the elected branch to be warp-uniform and keeps their
// descriptor operands in uniform registers.  The same instructions under `lane == 0` cost
// about 200 cycles each on sm_100a, against 25 here (measured on a chain of tcgen05.mma).
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .b32 rx;\n"
        ".reg .pred px;\n"
        "elect.sync rx|px, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, px;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

// Makes freshly initialised barriers visible to the asynchronous proxy.
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later
// asynchronous-proxy (TMA) accesses.
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ int lds_volatile_s32(uint32_t addr)
{
    int v;
    asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void sts_volatile_s32(uint32_t addr, int v)
{
    asm volatile("st.volatile.shared.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Waits for the phase with the given parity to complete.  Gives up after
// kWaitCycleLimit cycles, or as soon as another thread of the CTA has given up (the
// word at shared address abort_word is non-zero); returns false in both cases and
// raises the word.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t abort_word)
{
    if (mbar_try_wait(bar, parity)) return true;
    if (lds_volatile_s32(abort_word)) return false;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0u) {
            if (lds_volatile_s32(abort_word)) return false;
            if (clock64() - t0 > kWaitCycleLimit) {
                sts_volatile_s32(abort_word, 1);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Same contract as mbar_wait_bounded, but polls without letting the hardware suspend the
// thread: for hand-offs that are expected within a few hundred cycles, where the wake-up
// latency of a suspended wait would dominate.
__device__ __forceinline__ bool mbar_spin_bounded(uint32_t bar, uint32_t parity, uint32_t abort_word)
{
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!mbar_test_wait(bar, parity)) {
        if ((++spins & 1023u) == 0u) {
            if (lds_volatile_s32(abort_word)) return false;
            if (clock64() - t0 > kWaitCycleLimit) {
                sts_volatile_s32(abort_word, 1);
                return false;
            }
        }
    }
    return true;
}

// Untiled bulk copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src_gmem, uint32_t bytes, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(src_gmem), "r"(bytes), "r"(bar)
        : "memory");
}

// Tiled 2-D tensor copy global -> shared through a tensor map ({x, y} = element
// coordinates of the box corner, x innermost and a multiple of 4 floats).
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tensor_map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Programmatic dependent launch.  grid_dependency_wait: returns once the kernel ahead of this
// one on the stream has completed and its writes are visible (at once when this launch has
// no such dependency).  grid_launch_dependents: this CTA no longer stands in the way of the
// next kernel's CTAs being scheduled (they still wait, as above, for this grid to complete).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Starts fetching a tensor map (kernel parameter) into the TMA unit's descriptor cache.
__device__ __forceinline__ void prefetch_tensor_map(const void* tensor_map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensor_map)) : "memory");
}

// Tiled 3-D tensor copy global -> shared ({x, y, z} = element coordinates of the box corner).
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tensor_map, int x, int y, int z, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// One thread's asynchronous 4-byte copy global -> shared (cp.async groups of the issuing thread).
__device__ __forceinline__ void cp_async_4(uint32_t dst_smem, const void* src_gmem)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void sts_f32(uint32_t addr, float v)
{
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_s32(uint32_t addr, int v)
{
    asm volatile("st.shared.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_f4(uint32_t addr, float4 v)
{
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Shared-memory loads by 32-bit shared address.  volatile: they stay behind the
// mbarrier wait that guards the stage they read.
__device__ __forceinline__ float4 lds_f4(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ float2 lds_f2(uint32_t addr)
{
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ int4 lds_i4(uint32_t addr)
{
    int4 v;
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ int lds_s32(uint32_t addr)
{
    int v;
    asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

}  // namespace nmspmm
