// Dequantizer, quantizer, Hadamard rotation and sign generation kernels.
// These are the byte/integer side of the path: results are bit-identical to the
// reference's CPU code, so every floating-point step below is written as the single
// IEEE operation the reference performs (no contraction across statements).
#include "lq4_kernels.cuh"

namespace lq4 {

// ---------------------------------------------------------------------------
// Dequantize: one thread per nibble word (8 weights).  HBM-bound on the f32
// writes (4 B per weight against 0.625 B read).
// q * scale is exact in f32 (q <= 15 has 4 bits, scale has an 11-bit significand),
// so the fused multiply-add below rounds exactly like "multiply, then add".
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ payload, uint64_t n_words,
                                                      float* __restrict__ out) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t wi = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; wi < n_words; wi += stride) {
        const uint64_t blk = wi >> 2;
        const uint32_t il = (uint32_t)(wi & 3);
        const uint32_t* bp = reinterpret_cast<const uint32_t*>(payload + blk * kBlockBytes);
        const uint32_t meta = __ldg(bp);
        const uint32_t w = __ldg(bp + 1 + il);
        const float scale = h2f_bits(meta & 0xffffu);
        const float bias = h2f_bits(meta >> 16);
        float4 lo, hi;
        lo.x = __fmaf_rn((float)(w & 15u), scale, bias);
        lo.y = __fmaf_rn((float)((w >> 4) & 15u), scale, bias);
        lo.z = __fmaf_rn((float)((w >> 8) & 15u), scale, bias);
        lo.w = __fmaf_rn((float)((w >> 12) & 15u), scale, bias);
        hi.x = __fmaf_rn((float)((w >> 16) & 15u), scale, bias);
        hi.y = __fmaf_rn((float)((w >> 20) & 15u), scale, bias);
        hi.z = __fmaf_rn((float)((w >> 24) & 15u), scale, bias);
        hi.w = __fmaf_rn((float)(w >> 28), scale, bias);
        float4* o = reinterpret_cast<float4*>(out + wi * 8);
        __stcs(o, lo);
        __stcs(o + 1, hi);
    }
}

void launch_dequant(const uint8_t* payload, uint64_t n_blocks, float* out, int sm_count, cudaStream_t s) {
    const uint64_t n_words = n_blocks * 4;
    uint64_t blocks = (n_words + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return;
    dequant_kernel<<<(unsigned)blocks, 256, 0, s>>>(payload, n_words, out);
}

// ---------------------------------------------------------------------------
// Quantize: one warp per block of 32 values, lane i holds value i.
// Follows quantize_block_with_mode_len step by step; min/max/abs-max are exact
// whatever the reduction order, every other step is one rounded f32 operation.
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool scale_survives_f16(float s) {
    const float r = __half2float(__float2half_rn(s));
    return isfinite(r) && r > 0.0f;
}

__global__ void __launch_bounds__(256) quantize_kernel(const float* __restrict__ data, uint64_t len,
                                                       int symmetric, uint8_t* __restrict__ payload,
                                                       int32_t* __restrict__ status) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t n_blocks = (len + 31) / 32;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t blk = (((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5); blk < n_blocks; blk += warps) {
        const uint64_t idx = blk * 32 + lane;
        const bool real = idx < len;
        const float v = real ? data[idx] : 0.0f;       // padding slots hold zero
        const bool finite = isfinite(v);
        float scale, bias, sub;
        if (symmetric) {
            float a = fabsf(v);                        // folds over the padded block
            for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            float cand = __fdiv_rn(a, 7.0f);
            scale = (cand < 1.0f && !scale_survives_f16(cand)) ? 1.0f : cand;
            bias = __fmul_rn(-8.0f, scale);
            sub = 0.0f;
        } else {
            float mn = real ? v : INFINITY, mx = real ? v : -INFINITY;   // real elements only
            for (int o = 16; o; o >>= 1) {
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
            float cand = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
            scale = (cand < 1.0f && !scale_survives_f16(cand)) ? 1.0f : cand;
            bias = mn;
            sub = mn;
        }
        const __half sh = __float2half_rn(scale), bh = __float2half_rn(bias);
        const bool ok = __all_sync(0xffffffffu, finite) && scale_survives_f16(scale) &&
                        isfinite(__half2float(bh));
        const float inv = __fdiv_rn(1.0f, scale);
        float t;
        if (symmetric) t = __fadd_rn(roundf(__fmul_rn(v, inv)), 8.0f);
        else t = roundf(__fmul_rn(__fsub_rn(v, sub), inv));
        t = fminf(fmaxf(t, 0.0f), 15.0f);
        uint32_t q = ok ? (uint32_t)t : 0u;
        // pack: byte b = q[2b+1] << 4 | q[2b]; lane 8j assembles word j
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t qi = __shfl_sync(0xffffffffu, q, (lane & 24) + i);
            word |= qi << (4 * i);
        }
        uint32_t* bp = reinterpret_cast<uint32_t*>(payload + blk * kBlockBytes);
        if ((lane & 7) == 0) bp[1 + (lane >> 3)] = word;
        if (lane == 1) bp[0] = (uint32_t)__half_as_ushort(sh) | ((uint32_t)__half_as_ushort(bh) << 16);
        if (!ok && lane == 0 && status) atomicExch(status, LQ4_ERR_BAD_BLOCK);
    }
}

void launch_quantize(const float* data, uint64_t len, int symmetric, uint8_t* payload, int32_t* status,
                     int sm_count, cudaStream_t s) {
    const uint64_t n_blocks = (len + 31) / 32;
    uint64_t blocks = (n_blocks + 7) / 8;
    const uint64_t cap = (uint64_t)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return;
    quantize_kernel<<<(unsigned)blocks, 256, 0, s>>>(data, len, symmetric, payload, status);
}

// ---------------------------------------------------------------------------
// Randomized Hadamard rotation of activation rows: x' = H (D x), one CTA per
// row, the row staged in shared memory.  Radix-2 butterflies in the reference's
// stage order (h = 1, 2, 4, ...): every output of a stage is a single add or
// subtract of two values of the previous stage, so running the butterflies of
// one stage in parallel reproduces the sequential result bit for bit.
// ---------------------------------------------------------------------------
// A block-diagonal rotation is the same kernel over rows of one block each: row r of the launch is block
// r % sign_rows of its vector and takes that block's signs (sign_rows = 1: one diagonal for every row).
__global__ void __launch_bounds__(512) hadamard_rows_kernel(const void* __restrict__ x, int x_dtype,
                                                            const float* __restrict__ signs, uint32_t dim,
                                                            uint32_t sign_rows, float* __restrict__ out) {
    extern __shared__ float row[];
    const size_t base = (size_t)blockIdx.x * dim;
    signs += (size_t)(blockIdx.x % sign_rows) * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x)
        row[i] = __fmul_rn(load_act(x, x_dtype, base + i), signs[i]);
    __syncthreads();
    for (uint32_t h = 1; h < dim; h <<= 1) {
        for (uint32_t b = threadIdx.x; b < dim / 2; b += blockDim.x) {
            const uint32_t j = ((b / h) * 2 * h) + (b % h);
            const float p = row[j], q = row[j + h];
            row[j] = __fadd_rn(p, q);
            row[j + h] = __fsub_rn(p, q);
        }
        __syncthreads();
    }
    const float sc = __fdiv_rn(1.0f, __fsqrt_rn((float)dim));
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) out[base + i] = __fmul_rn(row[i], sc);
}

cudaError_t launch_hadamard_rows(const void* x, int x_dtype, const float* signs, uint32_t dim, uint32_t rows,
                                 float* out, cudaStream_t s, uint32_t sign_rows) {
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(hadamard_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    if (rows == 0) return cudaSuccess;
    hadamard_rows_kernel<<<rows, dim >= 1024 ? 512 : (dim >= 128 ? dim / 2 : 64), smem, s>>>(x, x_dtype, signs, dim, sign_rows ? sign_rows : 1, out);
    return cudaGetLastError();
}

// The cross-head rotation H_NH (x) I_head_dim of an activation [NH * head_dim] ("Hadamard heads", the R3
// rotation in front of o_proj): one thread per (row, within-head channel) gathers the NH values of its
// channel across the heads, applies signs and the butterflies in the sequential order (bit-identical to
// the scalar loop), scales and scatters.  Neighbouring threads take neighbouring channels: coalesced.
template <int NH>
__global__ void __launch_bounds__(128) cross_head_rows_kernel(const float* __restrict__ x, const float* __restrict__ signs,
                                                              uint32_t head_dim, uint64_t total, float* __restrict__ out) {
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const uint64_t row = idx / head_dim, base = row * NH * head_dim + (idx - row * head_dim);
    float v[NH];
#pragma unroll
    for (int h = 0; h < NH; ++h) v[h] = __fmul_rn(x[base + (uint64_t)h * head_dim], signs[h]);
#pragma unroll
    for (int hh = 1; hh < NH; hh <<= 1)
#pragma unroll
        for (int i = 0; i < NH; i += 2 * hh)
#pragma unroll
            for (int j = i; j < i + hh; ++j) {
                const float p = v[j], q = v[j + hh];
                v[j] = __fadd_rn(p, q);
                v[j + hh] = __fsub_rn(p, q);
            }
    const float sc = __fdiv_rn(1.0f, __fsqrt_rn((float)NH));
#pragma unroll
    for (int h = 0; h < NH; ++h) out[base + (uint64_t)h * head_dim] = __fmul_rn(v[h], sc);
}

cudaError_t launch_cross_head_rows(const float* x, const float* signs, uint32_t num_heads, uint32_t head_dim,
                                   uint32_t rows, float* out, cudaStream_t s) {
    const uint64_t total = (uint64_t)rows * head_dim;
    if (total == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((total + 127) / 128);
    switch (num_heads) {
#define LQ4_CH_CASE(NH) case NH: cross_head_rows_kernel<NH><<<grid, 128, 0, s>>>(x, signs, head_dim, total, out); break;
        LQ4_CH_CASE(1) LQ4_CH_CASE(2) LQ4_CH_CASE(4) LQ4_CH_CASE(8) LQ4_CH_CASE(16) LQ4_CH_CASE(32) LQ4_CH_CASE(64)
        LQ4_CH_CASE(128)
#undef LQ4_CH_CASE
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// h[row][i] = silu(gate_up[row][i]) * gate_up[row][inter + i]: the gating between the merged gate||up
// projection and down_proj, for the shapes whose down_proj kernel does not gate its own input.
__global__ void __launch_bounds__(256) silu_mul_rows_kernel(const float* __restrict__ gate_up, uint32_t inter,
                                                            uint64_t total, float* __restrict__ h) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint64_t row = i / inter, c = i - row * inter;
        const float* g = gate_up + row * 2 * inter;
        h[i] = silu_mul(g[c], g[inter + c]);
    }
}

cudaError_t launch_silu_mul_rows(const float* gate_up, uint32_t rows, uint32_t inter, float* h, int sm_count,
                                 cudaStream_t s) {
    const uint64_t total = (uint64_t)rows * inter;
    if (total == 0) return cudaSuccess;
    const uint64_t want = (total + 255) / 256, cap = (uint64_t)sm_count * 8;
    silu_mul_rows_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, s>>>(gate_up, inter, total, h);
    return cudaGetLastError();
}

// splitmix64 sign stream: state_i = seed + (i + 2) * gamma, sign = +1 when the mixed low bit is 0.
__global__ void rot_signs_kernel(uint64_t seed, uint32_t dim, float* __restrict__ signs) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    const uint64_t gamma = 0x9E3779B97F4A7C15ull;
    uint64_t z = seed + gamma * (uint64_t)(i + 2);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    signs[i] = (z & 1ull) ? -1.0f : 1.0f;
}

// Block i of a block-diagonal rotation draws its signs from the stream seeded with
// mix(seed + i * gamma) (derive_block_seed of the reference).
__global__ void block_rot_signs_kernel(uint64_t seed, uint32_t n, uint32_t block, float* __restrict__ signs) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t gamma = 0x9E3779B97F4A7C15ull;
    auto mix = [](uint64_t z) {
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    };
    const uint64_t bseed = mix(seed + gamma * (uint64_t)(i / block));
    signs[i] = (mix(bseed + gamma * (uint64_t)(i % block + 2)) & 1ull) ? -1.0f : 1.0f;
}

void launch_block_rot_signs(uint64_t seed, uint32_t n, uint32_t block, float* signs, cudaStream_t s) {
    if (n == 0) return;
    block_rot_signs_kernel<<<(n + 255) / 256, 256, 0, s>>>(seed, n, block, signs);
}

void launch_rot_signs(uint64_t seed, uint32_t dim, float* signs, cudaStream_t s) {
    if (dim == 0) return;
    rot_signs_kernel<<<(dim + 255) / 256, 256, 0, s>>>(seed, dim, signs);
}

}  // namespace lq4
