// Shared device helpers for the Q4 linear kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lattice_q4.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "this library is written for sm_100a only"
#endif

namespace lq4 {

constexpr int kBlockBytes = 20;     // one Q4 block: f16 scale, f16 bias, 16 nibble bytes
constexpr int kBlockWeights = 32;

// Bits of the device status word (set by kernels, read by lq4_ctx_check).
constexpr int kDevErrBarrierTimeout = 1;   // an mbarrier wait hit its time limit
constexpr int kDevErrGridWaitTimeout = 2;  // waiting for other CTAs' LoRA partials timed out
constexpr int kDevErrTmem = 4;

// Every device-side wait gives up after this many SM clock cycles (about two seconds).  The
// SM-local %clock64 is used because it is cheap to read inside a polling loop.
constexpr long long kWaitLimitCycles = 4000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ long long wait_clock() { return clock64(); }
__device__ __forceinline__ bool wait_expired(long long t0) { return clock64() - t0 > kWaitLimitCycles; }

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait: returns false (and the caller records an error) once the time limit passes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = wait_clock();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (wait_expired(t0)) return false;
    }
}

// ---- bulk async copy global -> shared, completion on an mbarrier ---------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// SwiGLU gating as the reference's silu_mul_fused computes it: gate / (1 + exp(-gate)) * up
// (crates/inference/src/forward/shaders/qwen35.metal:712-722).
__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + expf(-gate)) * up; }

// ---- programmatic dependent launch ----------------------------------------------
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- arrivals of a fused all-gather ----------------------------------------------------
// Waits (bounded) until every peer's results of all gathered launches this rank has issued so far
// have arrived: each such launch of a peer adds 256 to `arrive[0]`, each of this rank's own adds
// 256 to `arrive[1]`.  Called by ONE thread of a warp or CTA after the previous launch is known to be
// complete; the others follow through a warp or CTA barrier.  Returns false on timeout.
__device__ __forceinline__ bool wait_gather_arrivals(const unsigned long long* arrive, uint32_t world) {
    unsigned long long seq, v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(seq) : "l"(arrive + 1) : "memory");
    const unsigned long long need = (seq >> 8) * 256ull * (world - 1);
    const long long t0 = wait_clock();
    for (;;) {
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(arrive) : "memory");
        if (v >= need) return true;
        if (wait_expired(t0)) return false;
    }
}

// ---- named barriers (subsets of a CTA) ----------------------------------------------
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- nibble word -> exact f16 integers ------------------------------------------------
// A 32-bit word holds nibbles n0..n7 (n_i at bits 4i).  OR-ing a nibble into the
// mantissa of 1024.0 (0x6400, ulp 1) or of 64.0 (0x5400, ulp 1/16 so bits 4..7 count
// units) and subtracting the base gives the integer exactly, two at a time.
//   q04 = (n0, n4)  q15 = (n1, n5)  q26 = (n2, n6)  q37 = (n3, n7)
__device__ __forceinline__ void nibbles_to_h2(uint32_t w, uint32_t& q04, uint32_t& q15, uint32_t& q26,
                                              uint32_t& q37) {
    const uint32_t w8 = w >> 8;
    uint32_t lo0 = (w & 0x000F000Fu) | 0x64006400u;
    uint32_t hi0 = (w & 0x00F000F0u) | 0x54005400u;
    uint32_t lo1 = (w8 & 0x000F000Fu) | 0x64006400u;
    uint32_t hi1 = (w8 & 0x00F000F0u) | 0x54005400u;
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6400));
    const __half2 k64 = __half2half2(__ushort_as_half((unsigned short)0x5400));
    __half2 r;
    r = __hsub2(*reinterpret_cast<__half2*>(&lo0), k1024); q04 = *reinterpret_cast<uint32_t*>(&r);
    r = __hsub2(*reinterpret_cast<__half2*>(&hi0), k64);   q15 = *reinterpret_cast<uint32_t*>(&r);
    r = __hsub2(*reinterpret_cast<__half2*>(&lo1), k1024); q26 = *reinterpret_cast<uint32_t*>(&r);
    r = __hsub2(*reinterpret_cast<__half2*>(&hi1), k64);   q37 = *reinterpret_cast<uint32_t*>(&r);
}

// f16 bit pattern -> f32, exact (including subnormals).
__device__ __forceinline__ float h2f_bits(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

// bf16 bits -> f32 (exact widening).
__device__ __forceinline__ float bf16_to_f32(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

__device__ __forceinline__ float load_act(const void* x, int dtype, size_t idx) {
    return dtype == LQ4_DTYPE_BF16 ? bf16_to_f32(static_cast<const uint16_t*>(x)[idx])
                                   : static_cast<const float*>(x)[idx];
}

// Splits v into an f16 "hi" (round to nearest) and an f16 "lo" holding the residual,
// so hi + lo carries about 22 significant bits of v.
__device__ __forceinline__ void split_f16(float v, __half& hi, __half& lo) {
    hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
}

}  // namespace lq4
