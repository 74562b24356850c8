// Device helpers shared by the decode kernels (lq4_decode.cu, lq4_gemv.cu).
#pragma once

#include "lq4_kernels.cuh"

namespace lq4 {
namespace gemv {

constexpr uint32_t kFull = 0xffffffffu;
constexpr int kConsumerThreads = 256;
constexpr int kBarConsumers = 1;   // named barrier id used by the 8 consumer warps

__device__ __forceinline__ uint64_t range_begin(uint64_t c, uint64_t total, uint64_t grid) {
    return (c * total) / grid;
}

// CTA whose range contains position `pos` (every CTA owns at least one granule).
__device__ __forceinline__ uint32_t owner_of(uint64_t pos, uint64_t total, uint64_t grid) {
    uint64_t c = (pos * grid) / total;
    while (c + 1 < grid && range_begin(c + 1, total, grid) <= pos) ++c;
    return (uint32_t)c;
}

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}

// Loads eight consecutive activations (16-byte aligned) as f32.
__device__ __forceinline__ void load8(const void* x, int dtype, size_t idx, float (&v)[8]) {
    if (dtype == LQ4_DTYPE_BF16) {
        const uint4 r = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + idx);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
        const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + idx);
        const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + idx + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// Turns eight activations k = 8o .. 8o+7 of one token into the two 16-byte B-operand
// fragments (hi limb, lo limb) the consumer threads load, and returns their sum.
// Fragment order {(k0,k4), (k1,k5), (k2,k6), (k3,k7)} mirrors nibbles_to_h2().
__device__ __forceinline__ float make_fragments(const float (&v)[8], uint4& fh, uint4& fl) {
    __half h[8], l[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) split_f16(v[i], h[i], l[i]);
    fh = make_uint4(pack_h2(h[0], h[4]), pack_h2(h[1], h[5]), pack_h2(h[2], h[6]), pack_h2(h[3], h[7]));
    fl = make_uint4(pack_h2(l[0], l[4]), pack_h2(l[1], l[5]), pack_h2(l[2], l[6]), pack_h2(l[3], l[7]));
    return ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
}

// Writes fragments and block sums of token slot `mp` for octet `o` (8 activations).
// Layout: fragments [kb][nt][gmax columns][4 quads][16 B]; sums [kb][nt][4 tokens].
// `sx_stride` floats separate consecutive blocks' sums (NT * 4 in the staged layout, the token
// count in the compact resident layout).
__device__ __forceinline__ void store_fragments(uint8_t* xs, float* sx, uint32_t NT, uint32_t gmax, uint32_t mp,
                                                uint32_t o, bool active, const float (&v)[8],
                                                uint32_t sx_stride) {
    uint4 fh, fl;
    float s = make_fragments(v, fh, fl);
    s += __shfl_xor_sync(kFull, s, 1);
    s += __shfl_xor_sync(kFull, s, 2);
    if (!active) return;
    const uint32_t kbi = o >> 2, tt = o & 3, ntile = mp >> 2, ghi = (mp & 3) * 2;
    uint8_t* dst = xs + ((size_t)(kbi * NT + ntile) * gmax + ghi) * 64 + tt * 16;
    *reinterpret_cast<uint4*>(dst) = fh;
    *reinterpret_cast<uint4*>(dst + 64) = fl;
    if (tt == 0) sx[(size_t)kbi * sx_stride + ntile * 4 + (mp & 3)] = s;
}

}  // namespace gemv
}  // namespace lq4
