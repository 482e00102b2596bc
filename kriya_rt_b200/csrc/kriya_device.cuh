// Device-side helpers shared by the kernels: 16-bit storage conversion, mbarrier and bulk-copy PTX.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kriya_internal.h"

namespace kriya {

struct Bf16 {
    static constexpr uint32_t kDtype = KRIYA_DTYPE_BF16;
    // bf16 -> f32 is a 16-bit shift (paged_gqa_and_deltanet.metal:95-97)
    __device__ __forceinline__ static float load(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }
    // round to nearest even on the bit pattern, no NaN special case (paged_gqa_and_deltanet.metal:99-103)
    __device__ __forceinline__ static uint16_t store(float v) {
        const uint32_t u = __float_as_uint(v);
        return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
    }
    // two packed values (low half = element 0)
    __device__ __forceinline__ static float2 load2(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    }
    // two finite values rounded to nearest even and packed (low half = lo): one instruction; equal to store() on
    // every finite input, used for probabilities
    __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
        uint32_t w;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
        return w;
    }
};

struct Fp16 {
    static constexpr uint32_t kDtype = KRIYA_DTYPE_FP16;
    __device__ __forceinline__ static float load(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    __device__ __forceinline__ static uint16_t store(float v) { return __half_as_ushort(__float2half_rn(v)); }
    __device__ __forceinline__ static float2 load2(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
    __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
        uint32_t w;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
        return w;
    }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: polls until the phase completes or `limit_ns` of wall time have passed (default kWaitNs; a context may
// set its own, see kriya_cuda_set_wait_limit_us), so a lost copy or a missing arrival can never hang the GPU.  Returns
// false on expiry.  Callers that go on to use warp-synchronous primitives must agree on the outcome first (see warp_wait).
constexpr uint64_t kWaitNs = 2000000000ull;
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// The polling loop is a function of its own: dozens of inlined copies of it would be most of a kernel's code, and code
// that is executed once per CTA is paid for in instruction-cache misses.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = kWaitNs) {
    if (mbar_try_wait(bar, parity)) return true;
#ifdef KRIYA_INLINE_WAITS  // kernels that move registers between warpgroups (setmaxnreg) cannot call functions
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
#else
    return mbar_wait_slow(bar, parity, limit_ns);
#endif
}
// All 32 lanes wait, then agree: true only if every lane saw the phase complete.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = kWaitNs) {
    const bool ok = mbar_wait(bar, parity, limit_ns);
    return __all_sync(0xFFFFFFFFu, ok);
}

// ---- bulk async copy global -> shared, completion on an mbarrier ------------------------------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace kriya
