// Device helpers shared by the decode kernels (lq4_decode.cu, lq4_dense.cu) and the generic kernel.
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

}  // namespace gemv
}  // namespace lq4
