// Generic Q4 linear kernel (any k % 32 == 0, any alignment) and the plain LoRA projection used
// with it; both are fallbacks for shapes the TMA-based decode kernels do not take.
#include "lq4_gemv_common.cuh"

namespace lq4 {

using namespace gemv;

bool gemv_resident_fits(uint32_t m, uint32_t k, bool rot) {
    if (m == 0 || m > 4 || k % 128 != 0) return false;
    GemvParams q{};
    q.m = m; q.n = 1u << 20; q.k = k; q.kb = k / 32; q.rank = kGemvMaxRank;
    q.tiles = q.n / kGemvTileRows;
    static float dummy;
    q.signs = rot ? &dummy : nullptr;
    return decode_plan_smem(q) != 0;
}

// t[tok][j] = sum_k A[j][k] * x[tok][k]; one warp per (tok, j), fixed reduction tree.
__global__ void __launch_bounds__(256) lora_t_kernel(const void* __restrict__ x, int x_dtype, uint32_t m, uint32_t k,
                                                     const float* __restrict__ la, uint32_t rank,
                                                     float* __restrict__ t) {
    const uint32_t pr = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (pr >= m * rank) return;
    const uint32_t tok = pr / rank, j = pr - tok * rank;
    const float* arow = la + (size_t)j * k;
    float s0 = 0.0f, s1 = 0.0f;
    uint32_t kk = lane;
    for (; kk + 32 < k; kk += 64) {
        s0 = fmaf(__ldg(arow + kk), load_act(x, x_dtype, (size_t)tok * k + kk), s0);
        s1 = fmaf(__ldg(arow + kk + 32), load_act(x, x_dtype, (size_t)tok * k + kk + 32), s1);
    }
    for (; kk < k; kk += 32) s0 = fmaf(__ldg(arow + kk), load_act(x, x_dtype, (size_t)tok * k + kk), s0);
    float sum = s0 + s1;
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
    if (lane == 0) t[pr] = sum;
}

void launch_lora_t(const void* x, int x_dtype, uint32_t m, uint32_t k, const float* la, uint32_t rank, float* t,
                   cudaStream_t s) {
    const uint32_t pairs = m * rank;
    if (pairs == 0) return;
    lora_t_kernel<<<(pairs + 7) / 8, 256, 0, s>>>(x, x_dtype, m, k, la, rank, t);
}

// ---------------------------------------------------------------------------
// Generic kernel: any k % 32 == 0, 4-byte aligned payload, any m.  One warp per
// output row and token; lanes stride over nibble words.  Also serves the
// standalone LoRA accumulate (base term skipped).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gemv_generic_kernel(const void* __restrict__ x, int x_dtype,
                                                           const uint8_t* __restrict__ w, float* __restrict__ y,
                                                           uint64_t ldy, uint32_t m, uint32_t n, uint32_t k,
                                                           const float* __restrict__ t, const float* __restrict__ lb,
                                                           uint32_t rank, float lscale, int accumulate_only) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= n) return;
    const uint32_t kb = k / 32, nwords = k / 8;
    const uint8_t* wrow = w ? w + (size_t)row * kb * kBlockBytes : nullptr;
    for (uint32_t tok = blockIdx.y; tok < m; tok += gridDim.y) {
        float acc = 0.0f;
        if (!accumulate_only) {
            for (uint32_t wi = lane; wi < nwords; wi += 32) {
                const uint32_t* bp = reinterpret_cast<const uint32_t*>(wrow + (size_t)(wi >> 2) * kBlockBytes);
                const uint32_t meta = __ldg(bp), q = __ldg(bp + 1 + (wi & 3));
                const float d = h2f_bits(meta & 0xffffu), b = h2f_bits(meta >> 16);
                const size_t xb = (size_t)tok * k + (size_t)wi * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float wv = __fmaf_rn((float)((q >> (4 * i)) & 15u), d, b);
                    acc = fmaf(wv, load_act(x, x_dtype, xb + i), acc);
                }
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
        }
        if (lane == 0) {
            float out = accumulate_only ? y[(size_t)tok * ldy + row] : acc;
            if (rank) {
                float dsum = 0.0f;
                for (uint32_t j = 0; j < rank; ++j) dsum = fmaf(lb[(size_t)row * rank + j], t[(size_t)tok * rank + j], dsum);
                out += lscale * dsum;
            }
            y[(size_t)tok * ldy + row] = out;
        }
    }
}

void launch_gemv_generic(const void* x, int x_dtype, const uint8_t* w, float* y, uint64_t ldy, uint32_t m,
                         uint32_t n, uint32_t k, const float* t, const float* lb, uint32_t rank, float lscale,
                         int accumulate_only, cudaStream_t s) {
    if (m == 0 || n == 0) return;
    dim3 grid((n + 7) / 8, m < 65535u ? m : 65535u);
    gemv_generic_kernel<<<grid, 256, 0, s>>>(x, x_dtype, w, y, ldy, m, n, k, t, lb, rank, lscale, accumulate_only);
}

}  // namespace lq4
