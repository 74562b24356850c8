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

// Input element `idx` as the f32 the reference's block quantizer sees: f32 as is, bf16 widened
// (quantize_bf16_to_q4), f64 narrowed with round-to-nearest-even like Rust's `as f32`
// (quantize_f64_to_q4_mode); an f64 beyond the f32 range becomes infinite and is refused below.
template <typename T>
__device__ __forceinline__ float quant_input(const T* data, uint64_t idx);
template <>
__device__ __forceinline__ float quant_input<float>(const float* data, uint64_t idx) { return data[idx]; }
template <>
__device__ __forceinline__ float quant_input<uint16_t>(const uint16_t* data, uint64_t idx) { return bf16_to_f32(data[idx]); }
template <>
__device__ __forceinline__ float quant_input<double>(const double* data, uint64_t idx) { return __double2float_rn(data[idx]); }

// `row_len` elements form one run of blocks: the whole flattened tensor for the flat entry points
// (blocks cross row ends), one row for quantize_tensor_q4_0 (every row ends in its own padded block).
template <typename T>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ data, uint64_t rows, uint64_t row_len,
                                                       int symmetric, uint8_t* __restrict__ payload,
                                                       int32_t* __restrict__ status) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t bpr = (row_len + 31) / 32;
    const uint64_t n_blocks = rows * bpr;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t blk = (((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5); blk < n_blocks; blk += warps) {
        const uint64_t r = blk / bpr, col = (blk - r * bpr) * 32 + lane;
        const bool real = col < row_len;
        const float v = real ? quant_input<T>(data, r * row_len + col) : 0.0f;       // padding slots hold zero
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

void launch_quantize(const void* data, int dtype, uint64_t rows, uint64_t row_len, int symmetric, uint8_t* payload,
                     int32_t* status, int sm_count, cudaStream_t s) {
    const uint64_t n_blocks = rows * ((row_len + 31) / 32);
    uint64_t blocks = (n_blocks + 7) / 8;
    const uint64_t cap = (uint64_t)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return;
    if (dtype == LQ4_DTYPE_BF16)
        quantize_kernel<uint16_t><<<(unsigned)blocks, 256, 0, s>>>(static_cast<const uint16_t*>(data), rows, row_len, symmetric, payload, status);
    else if (dtype == LQ4_DTYPE_F64)
        quantize_kernel<double><<<(unsigned)blocks, 256, 0, s>>>(static_cast<const double*>(data), rows, row_len, symmetric, payload, status);
    else
        quantize_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(static_cast<const float*>(data), rows, row_len, symmetric, payload, status);
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

// ---------------------------------------------------------------------------
// Rotation absorption into weights (offline conversion), f32 or f64, in place.
// Input side, W <- W R^T: R applied to every ROW (one CTA per row, the row in shared memory).
// Output side, W <- R W: R applied to every COLUMN; the butterflies of a stage pair whole rows, so
// they run over the matrix in place, three stages per pass, a thread per (column, group of 8 rows).
// Every value is produced by the same single IEEE operation, on the same operands, as in the
// reference's sequential loops, so the result is bit-identical.
// ---------------------------------------------------------------------------
template <typename T> struct Ieee;
template <> struct Ieee<float> {
    static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
    static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
    static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
    static __device__ __forceinline__ float inv_sqrt(uint32_t n) { return __fdiv_rn(1.0f, __fsqrt_rn((float)n)); }
};
template <> struct Ieee<double> {
    static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
    static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
    static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
    static __device__ __forceinline__ double inv_sqrt(uint32_t n) { return __ddiv_rn(1.0, __dsqrt_rn((double)n)); }
};

template <typename T>
__global__ void __launch_bounds__(512) absorb_rows_kernel(T* __restrict__ w, const float* __restrict__ signs, uint32_t dim) {
    extern __shared__ __align__(16) unsigned char absorb_smem[];
    T* row = reinterpret_cast<T*>(absorb_smem);
    T* g = w + (size_t)blockIdx.x * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) row[i] = Ieee<T>::mul(g[i], (T)signs[i]);
    __syncthreads();
    for (uint32_t h = 1; h < dim; h <<= 1) {
        for (uint32_t b = threadIdx.x; b < dim / 2; b += blockDim.x) {
            const uint32_t j = ((b / h) * 2 * h) + (b % h);
            const T p = row[j], q = row[j + h];
            row[j] = Ieee<T>::add(p, q);
            row[j + h] = Ieee<T>::sub(p, q);
        }
        __syncthreads();
    }
    const T sc = Ieee<T>::inv_sqrt(dim);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) g[i] = Ieee<T>::mul(row[i], sc);
}

// One pass of the output-side transform: `stages` (1..3) butterfly levels starting at row distance h.
// first: multiply by the signs on the way in; last: scale on the way out.
template <typename T, int ST>
__global__ void __launch_bounds__(256) absorb_cols_kernel(T* __restrict__ w, const float* __restrict__ signs, uint32_t dim,
                                                          uint64_t cols, uint32_t h, int first, int last) {
    constexpr uint32_t span = 1u << ST;                       // rows a thread combines
    const uint64_t groups = dim / span;
    const uint64_t total = groups * cols;
    const T sc = Ieee<T>::inv_sqrt(dim);
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t gi = idx / cols, c = idx - gi * cols;
        // group gi: rows base + i * h, i < span, where base keeps the bits below h and those above h * span
        const uint64_t lowbits = gi % h, high = gi / h;
        const uint64_t base = high * h * span + lowbits;
        T v[span];
#pragma unroll
        for (uint32_t i = 0; i < span; ++i) {
            const uint64_t r = base + (uint64_t)i * h;
            T t = w[r * cols + c];
            if (first) t = Ieee<T>::mul(t, (T)signs[r]);
            v[i] = t;
        }
#pragma unroll
        for (uint32_t hh = 1; hh < span; hh <<= 1)
#pragma unroll
            for (uint32_t i = 0; i < span; ++i) {
                if (i & hh) continue;
                const T p = v[i], q = v[i + hh];
                v[i] = Ieee<T>::add(p, q);
                v[i + hh] = Ieee<T>::sub(p, q);
            }
#pragma unroll
        for (uint32_t i = 0; i < span; ++i) {
            const uint64_t r = base + (uint64_t)i * h;
            w[r * cols + c] = last ? Ieee<T>::mul(v[i], sc) : v[i];
        }
    }
}

template <typename T>
static cudaError_t absorb_input_t(T* w, uint64_t rows, uint32_t dim, const float* signs, cudaStream_t s) {
    const size_t smem = (size_t)dim * sizeof(T);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(absorb_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const unsigned threads = dim >= 1024 ? 512 : (dim >= 128 ? dim / 2 : 64);
    // the grid's x extent is a 31-bit count: rows beyond that go in further launches
    for (uint64_t r0 = 0; r0 < rows; r0 += 0x40000000ull) {
        const uint64_t nr = rows - r0 < 0x40000000ull ? rows - r0 : 0x40000000ull;
        absorb_rows_kernel<T><<<(unsigned)nr, threads, smem, s>>>(w + r0 * dim, signs, dim);
    }
    return cudaGetLastError();
}

template <typename T>
static cudaError_t absorb_output_t(T* w, uint32_t dim, uint64_t cols, const float* signs, int sm_count, cudaStream_t s) {
    uint32_t levels = 0;
    while ((1u << levels) < dim) ++levels;
    auto grid_for = [&](uint32_t st) {
        const uint64_t total = (uint64_t)(dim >> st) * cols;
        const uint64_t want = (total + 255) / 256, cap = (uint64_t)sm_count * 16;
        return (unsigned)(want < cap ? want : cap);
    };
    if (levels == 0) {          // dim == 1: x * sign * 1
        absorb_cols_kernel<T, 0><<<grid_for(0), 256, 0, s>>>(w, signs, dim, cols, 1, 1, 1);
        return cudaGetLastError();
    }
    for (uint32_t l = 0; l < levels;) {
        const uint32_t st = levels - l >= 3 ? 3 : levels - l;
        const int first = l == 0, last = l + st == levels;
        if (st == 3) absorb_cols_kernel<T, 3><<<grid_for(3), 256, 0, s>>>(w, signs, dim, cols, 1u << l, first, last);
        else if (st == 2) absorb_cols_kernel<T, 2><<<grid_for(2), 256, 0, s>>>(w, signs, dim, cols, 1u << l, first, last);
        else absorb_cols_kernel<T, 1><<<grid_for(1), 256, 0, s>>>(w, signs, dim, cols, 1u << l, first, last);
        l += st;
    }
    return cudaGetLastError();
}

cudaError_t launch_absorb_input(void* w, int dtype, uint64_t rows, uint32_t dim, const float* signs, cudaStream_t s) {
    if (rows == 0) return cudaSuccess;
    return dtype == LQ4_DTYPE_F64 ? absorb_input_t(static_cast<double*>(w), rows, dim, signs, s)
                                  : absorb_input_t(static_cast<float*>(w), rows, dim, signs, s);
}
cudaError_t launch_absorb_output(void* w, int dtype, uint32_t dim, uint64_t cols, const float* signs, int sm_count,
                                 cudaStream_t s) {
    if (cols == 0) return cudaSuccess;
    return dtype == LQ4_DTYPE_F64 ? absorb_output_t(static_cast<double*>(w), dim, cols, signs, sm_count, s)
                                  : absorb_output_t(static_cast<float*>(w), dim, cols, signs, sm_count, s);
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
