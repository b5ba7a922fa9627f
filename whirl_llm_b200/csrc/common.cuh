// Device-side building blocks shared by the sampling kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace wb {

constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------------------------------
// ordering
// ---------------------------------------------------------------------------------------------------------------

// Order-preserving 32-bit key of a logit.  -0.0 and +0.0 share one key (the host comparators compare floats, so the
// two are equal there); NaN maps to key 0, below -inf, so a NaN logit is never preferred to a number.
__device__ __forceinline__ uint32_t key_of(float f) {
    if (f != f) return 0u;
    const uint32_t u = __float_as_uint(f + 0.0f);  // -0 + +0 = +0
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float float_of_key(uint32_t k) {
    const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}
// Candidate = (key << 32) | ~id : larger composite <=> (logit desc, id asc) earlier.  Composites of one row are distinct.
__device__ __forceinline__ uint64_t make_cand(uint32_t key, uint32_t id) { return (uint64_t(key) << 32) | uint32_t(~id); }
__device__ __forceinline__ uint32_t cand_key(uint64_t c) { return uint32_t(c >> 32); }
__device__ __forceinline__ uint32_t cand_id(uint64_t c) { return ~uint32_t(c); }

__device__ __forceinline__ float bf16_to_f32(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }

// ---------------------------------------------------------------------------------------------------------------
// warp helpers
// ---------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ uint64_t warp_max(uint64_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint64_t t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}
// inclusive prefix sum over the warp
__device__ __forceinline__ uint32_t warp_scan_incl(uint32_t v) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane_id() >= o) v += t;
    }
    return v;
}

// A group of NT threads (a multiple of 32) inside a CTA that synchronises on its own hardware barrier.
// id 0 is __syncthreads' barrier; groups that are not the whole CTA use ids 1..15.
template <int NT>
struct Group {
    static constexpr int size = NT;
    int tid;  // 0..NT-1 within the group
    int bar;  // hardware barrier id
    __device__ __forceinline__ void sync() const {
        if (NT == 32) __syncwarp();
        else asm volatile("bar.sync %0, %1;" ::"r"(bar), "n"(NT) : "memory");
    }
    // barrier + OR-reduction of a predicate over the group
    __device__ __forceinline__ bool sync_or(bool p) const {
        if (NT == 32) return __any_sync(0xffffffffu, p);
        uint32_t r;
        asm volatile(
            "{\n .reg .pred p, q;\n setp.ne.u32 p, %1, 0;\n bar.red.or.pred q, %2, %3, p;\n selp.u32 %0, 1, 0, q;\n}\n"
            : "=r"(r)
            : "r"(uint32_t(p)), "r"(bar), "n"(NT)
            : "memory");
        return r != 0;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// mbarrier + bulk async copy (TMA, untiled) wrappers.  Every wait is bounded: a wait that runs out sets *err and the
// caller unwinds, so a lost copy can never hang the device.
// ---------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same, letting the hardware keep the thread suspended for up to `ns` nanoseconds while the phase is not complete
// (a waiting warp that keeps asking takes issue slots from the warps that work).
__device__ __forceinline__ bool mbar_try_wait_for(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// One look at the barrier, never suspending the thread (for a loop that polls several barriers in turn).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: up to `limit` suspensions of about a microsecond each (the default is about a second).  false = gave up.
constexpr uint32_t kWaitLimit = 1u << 20;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = kWaitLimit) {
    if (mbar_try_wait(bar, parity)) return true;
#pragma unroll 1
    for (uint32_t it = 0; it < limit; ++it)
        if (mbar_try_wait_for(bar, parity, 1000u)) return true;
    return false;
}
// global -> shared bulk copy, 16-byte aligned addresses, size a multiple of 16, completion on an mbarrier
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// The same with an L2 policy for data that is read once (it should not push out what other warps keep reading: their
// parameters, their code).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_once(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace wb
