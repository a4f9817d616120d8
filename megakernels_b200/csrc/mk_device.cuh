// PTX wrappers and small math helpers for the decode kernel (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "mk_common.h"

namespace mk {

typedef unsigned long long u64;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- race-detection build ------------------------------------------------------------------------
// With -DMK_CHAOS every publish (a flag-in-data word, a counter increment, a barrier arrival, a ring-slot release)
// is preceded, for about one call in eight, by a pseudo-random pause of up to four microseconds.  The results
// of a correct protocol do not depend on when a publish happens, so a test requires the bits of this build's
// outputs to equal those of the normal build.  What the reference's `chaos` sleeps do for its stage flags
// (`common/mkcore/dev.py:394-416`).
#ifdef MK_CHAOS
__device__ __forceinline__ void chaos_delay() {
    unsigned t;
    asm volatile("mov.u32 %0, %%clock;" : "=r"(t));
    const unsigned h = (t ^ (threadIdx.x * 2654435761u) ^ (blockIdx.x * 40503u)) * 2246822519u;
    if ((h >> 29) == 0u) __nanosleep((h >> 8) & 4095u);
}
#else
__device__ __forceinline__ void chaos_delay() {}
#endif

// ---- mbarrier + bulk copy ----------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    chaos_delay();
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ u64 policy_evict_first() {
    u64 p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.  Both addresses and the
// size must be multiples of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar, u64 policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}
// 16-byte asynchronous copy global -> shared (bypasses L1), and the wait for all of this thread's copies.
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ u64 globaltimer() {
    u64 t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- named barriers over the consumer warps (the producer warp never joins) ---------------------
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }
// Barrier plus OR-reduction: every consumer thread gets the same answer.
__device__ __forceinline__ bool consumer_any(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n .reg .pred p, q;\n"
        " setp.ne.u32 q, %1, 0;\n"
        " bar.red.or.pred p, 1, %2, q;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(r) : "r"((uint32_t)pred), "n"(NCT) : "memory");
    return r != 0;
}

// ---- flag-in-data words: (epoch << 32) | fp32 bits ---------------------------------------------
__device__ __forceinline__ void ll_store(u64* p, uint32_t epoch, float v) {
    chaos_delay();
    const u64 w = ((u64)epoch << 32) | __float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_store_bits(u64* p, uint32_t epoch, uint32_t bits) {
    chaos_delay();
    const u64 w = ((u64)epoch << 32) | bits;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ u64 ll_load(const u64* p) {
    u64 w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ void ll_load2(const u64* p, u64& a, u64& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_u32(const unsigned* p) {
    uint32_t w;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ void st_relaxed_u32(unsigned* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_i32(const int* p) {
    int w;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(w) : "l"(p) : "memory");
    return w;
}

// ---- math ------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ u64 warp_max_u64(u64 v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const u64 t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Order-preserving float -> uint, so that an unsigned compare orders scores; the low word holds
// ~index so that equal scores resolve to the smallest index.
__device__ __forceinline__ uint32_t ordered_bits(float s) {
    const uint32_t b = __float_as_uint(s);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ u64 score_key(float s, int idx) {
    return ((u64)ordered_bits(s) << 32) | (0xFFFFFFFFu - (uint32_t)idx);
}
__device__ __forceinline__ int key_index(u64 k) { return (int)(0xFFFFFFFFu - (uint32_t)k); }

// 32-bit hash of (seed, position, token id) behind the sampling noise.
__host__ __device__ __forceinline__ uint32_t mk_mix32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t h = a * 0x9E3779B9u + 0x7F4A7C15u;
    h ^= b * 0x85EBCA6Bu + 0x165667B1u;
    h = (h ^ (h >> 15)) * 0x2C1B3C6Du;
    h ^= c * 0xC2B2AE35u + 0x27D4EB2Fu;
    h = (h ^ (h >> 13)) * 0x297A2D39u;
    h = (h ^ (h >> 16)) * 0x7FEB352Du;
    h = (h ^ (h >> 15)) * 0x846CA68Bu;
    return h ^ (h >> 16);
}

}  // namespace mk
