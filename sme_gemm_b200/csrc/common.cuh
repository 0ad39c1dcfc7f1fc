// Shared device helpers for the sm_100a kernels: mbarrier + bulk-copy (TMA)
// wrappers with bounded waits, 16-bit float conversions, the status word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace smeg {

// Error bits written to the library's device status word by a kernel that gave
// up on a bounded wait.  The host entry point turns a non-zero word into rc != 0.
enum : unsigned {
    STATUS_MBAR_TIMEOUT = 1u,   // a shared-memory barrier never completed
    STATUS_TMEM_TIMEOUT = 2u,   // a tensor-memory pipeline barrier never completed
    STATUS_PEER_TIMEOUT = 4u,   // a peer flag never arrived (multi-GPU reduce)
};

// Wall-clock bound of one wait (nanoseconds of the global timer).  Never reached
// unless a copy or an arrival was lost; a wait that does reach it raises the
// status word and every later wait of the CTA returns at once.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Same, letting the hardware suspend the thread for up to `ns` nanoseconds while the phase is
// pending (it resumes at once when the phase completes): a waiting warp then issues a handful
// of instructions per microsecond instead of competing with the working warps for issue slots.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t* bar, unsigned parity, unsigned ns) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises `status`) if the barrier never
// flipped; `abort_flag` in shared memory then short-circuits every later wait
// of the CTA so the kernel still ends quickly.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag,
                                          unsigned* status, unsigned code = STATUS_MBAR_TIMEOUT) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (*abort_flag) return false;
        if (mbar_try_wait_suspend(bar, parity, 4000u)) return true;
        if (global_ns() - t0 > kWaitLimitNs) break;
    }
    *abort_flag = 1;
    if (status) atomicOr(status, code);
    return false;
}

// Bounded wait for the hand-offs of a fine-grained pipeline (a stage every few hundred cycles): polls
// with the plain try_wait, whose own suspension is short, so the waiter resumes as soon as the
// phase completes.
__device__ __forceinline__ bool mbar_wait_poll(uint64_t* bar, unsigned parity, volatile int* abort_flag,
                                               unsigned* status, unsigned code = STATUS_MBAR_TIMEOUT) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (unsigned spins = 0;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 63u) == 63u) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitLimitNs) break;
        }
    }
    *abort_flag = 1;
    if (status) atomicOr(status, code);
    return false;
}

// One contiguous global -> shared copy on the bulk-copy (TMA) engine.  Both
// addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue / wait for the previous kernel's memory to be visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- 16-bit element helpers (T = 0: f16, 1: bf16), bit patterns in uint16 ----
template <int BF16>
__device__ __forceinline__ float t_to_f32(uint16_t v) {
    if (BF16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
    return __half2float(__ushort_as_half(v));
}
template <int BF16>
__device__ __forceinline__ uint16_t f32_to_t(float x) {
    if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(x));
    return __half_as_ushort(__float2half_rn(x));
}

// Two f32 values rounded to T and back (one packed conversion each way), and two f32 values rounded to a pair of T bits.
template <int BF16>
__device__ __forceinline__ float2 round2_t(float a, float b) {
    if (BF16) return __bfloat1622float2(__floats2bfloat162_rn(a, b));
    return __half22float2(__floats2half2_rn(a, b));
}
template <int BF16>
__device__ __forceinline__ uint32_t pack2_t(float a, float b) {
    if (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}

}  // namespace smeg
