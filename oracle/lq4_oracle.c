/*
 * CPU oracle for the Q4(+LoRA, +QuaRot) linear path of ohdearquant/lattice.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's CPU arithmetic; it is the checker the CUDA path is compared
 * against and the CPU baseline that gets timed.  Nothing in the shipped
 * library links, loads or calls it.
 *
 * Parity status: PINNED by the reference's own golden vectors and known-answer
 * tests (the two committed `.q4` byte-identity fixtures, the quantizer, f16,
 * Walsh-Hadamard and LoRA known answers, and the composed QuaRot+Q4 gate); the
 * reference itself is Rust and cannot be compiled in this environment.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project root).  Build with -ffp-contract=off: the Rust
 * reference never contracts a*b+c into an FMA unless it says so explicitly.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define ORC_OK 0
#define ORC_ERR_NONFINITE 1   /* source weight is NaN/inf */
#define ORC_ERR_SCALE 2       /* scale not finite-positive once stored as f16 */
#define ORC_ERR_BIAS 3        /* bias not finite once stored as f16 */
#define ORC_ERR_SHAPE 4       /* shape / length mismatch */
#define ORC_ERR_POW2 5        /* Hadamard length not a power of two */
#define ORC_ERR_IO 6
#define ORC_ERR_FORMAT 7
#define ORC_ERR_VALID_LEN 8

#define Q4_BLOCK_BYTES 20
#define Q4_BLOCK_WEIGHTS 32

static inline uint32_t f32_bits(float v) { uint32_t u; memcpy(&u, &v, 4); return u; }
static inline float bits_f32(uint32_t u) { float v; memcpy(&v, &u, 4); return v; }

/* ------------------------------------------------------------------------
 * f16 / bf16 bit conversions.
 * crates/inference/src/weights/f16_encode.rs:4-85  (f32 -> f16, RNE)
 * crates/inference/src/weights/half_bits.rs:24-63  (f16 -> f32, bf16 -> f32)
 * ---------------------------------------------------------------------- */

/* Shift right by `shift` bits rounding to nearest, ties to even. */
static uint32_t shr_rne(uint32_t value, uint32_t shift) {
    if (shift == 0) return value;
    if (shift >= 32) return 0;
    uint32_t kept = value >> shift;
    uint32_t lost = value & ((1u << shift) - 1u);
    uint32_t tie = 1u << (shift - 1);
    if (lost > tie || (lost == tie && (kept & 1u))) kept += 1;
    return kept;
}

uint16_t orc_f32_to_f16_bits(float v) {
    uint32_t bits = f32_bits(v);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int32_t e = (int32_t)((bits >> 23) & 0xffu);
    uint32_t frac = bits & 0x007fffffu;

    if (e == 0xff) {                       /* inf / NaN */
        if (frac == 0) return (uint16_t)(sign | 0x7c00u);
        uint16_t payload = (uint16_t)(frac >> 13);
        if (payload == 0) payload = 1;
        payload |= 0x0200u;
        return (uint16_t)(sign | 0x7c00u | (payload & 0x03ffu));
    }
    if (e == 0) return sign;               /* f32 zero and subnormals flush to signed zero */

    int32_t ue = e - 127;                  /* unbiased exponent */
    if (ue > 15) return (uint16_t)(sign | 0x7c00u);
    if (ue >= -14) {                       /* f16 normal range */
        uint16_t e16 = (uint16_t)(ue + 15);
        uint16_t f16 = (uint16_t)shr_rne(frac, 13);
        if (f16 == 0x0400u) {              /* mantissa carried out */
            f16 = 0;
            e16 += 1;
            if (e16 >= 0x1f) return (uint16_t)(sign | 0x7c00u);
        }
        return (uint16_t)(sign | (uint16_t)(e16 << 10) | f16);
    }
    /* f16 subnormal range: shift the 24-bit significand down */
    uint32_t mant = frac | 0x00800000u;
    uint32_t shift = (uint32_t)(-ue - 1);
    if (shift >= 32) return sign;
    uint16_t f16 = (uint16_t)shr_rne(mant, shift);
    if (f16 == 0) return sign;
    if (f16 == 0x0400u) return (uint16_t)(sign | 0x0400u);
    return (uint16_t)(sign | f16);
}

float orc_f16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) & 1u;
    uint32_t e = (uint32_t)(h >> 10) & 0x1fu;
    uint32_t frac = (uint32_t)h & 0x03ffu;
    uint32_t out;
    if (e == 0) {
        if (frac == 0) {
            out = sign << 31;
        } else {                           /* subnormal: renormalise */
            int32_t ue = -14;
            while ((frac & 0x0400u) == 0) { frac <<= 1; ue -= 1; }
            frac &= 0x03ffu;
            out = (sign << 31) | ((uint32_t)(ue + 127) << 23) | (frac << 13);
        }
    } else if (e == 0x1f) {
        out = (sign << 31) | 0x7f800000u | (frac << 13);
    } else {
        out = (sign << 31) | ((e + 112u) << 23) | (frac << 13);
    }
    return bits_f32(out);
}

float orc_bf16_bits_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

/* bf16 narrowing, RNE.  Not in the reference hot path (its fixtures truncate);
 * used only by the synthetic-input generator for the bf16-activation config. */
uint16_t orc_f32_to_bf16_bits_rne(float v) {
    uint32_t u = f32_bits(v);
    if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0xffffu) ? 0x40u : 0u));
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* ------------------------------------------------------------------------
 * Block quantizer.
 * crates/inference/src/weights/q4_weights.rs:161-216 (scale survivability,
 *   metadata bits, degenerate-safe scale)
 * crates/inference/src/weights/q4_weights.rs:239-295 (quantize_block_with_mode_len)
 * ---------------------------------------------------------------------- */

static int scale_survives_f16(float scale) {
    float s = orc_f16_bits_to_f32(orc_f32_to_f16_bits(scale));
    return isfinite(s) && s > 0.0f;
}

static float degenerate_safe_scale(float candidate) {
    if (candidate < 1.0f && !scale_survives_f16(candidate)) return 1.0f;
    return candidate;
}

static int metadata_bits(float scale, float bias, uint16_t* sb, uint16_t* bb) {
    *sb = orc_f32_to_f16_bits(scale);
    *bb = orc_f32_to_f16_bits(bias);
    if (!scale_survives_f16(scale)) return ORC_ERR_SCALE;
    if (!isfinite(orc_f16_bits_to_f32(*bb))) return ORC_ERR_BIAS;
    return ORC_OK;
}

static inline float clamp015(float v) { return v < 0.0f ? 0.0f : (v > 15.0f ? 15.0f : v); }

/* Rust `as u8` on a float saturates and maps NaN to 0. */
static inline uint8_t f32_as_u8(float v) {
    if (!(v == v)) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 255.0f) return 255;
    return (uint8_t)v;
}

int orc_quantize_block(const float vals[32], int valid_len, int symmetric, uint8_t out[20]) {
    if (valid_len < 1 || valid_len > 32) return ORC_ERR_VALID_LEN;
    for (int i = 0; i < 32; ++i)
        if (!isfinite(vals[i])) return ORC_ERR_NONFINITE;

    float scale, bias, sub;
    if (symmetric) {
        /* abs-max folds over the whole padded array, starting from 0.0 */
        float abs_max = 0.0f;
        for (int i = 0; i < 32; ++i) { float a = fabsf(vals[i]); if (a > abs_max) abs_max = a; }
        scale = degenerate_safe_scale(abs_max / 7.0f);
        bias = -8.0f * scale;
        sub = 0.0f;
    } else {
        /* min/max only over the real elements: padding must not widen the range */
        float mn = INFINITY, mx = -INFINITY;
        for (int i = 0; i < valid_len; ++i) {
            if (vals[i] < mn) mn = vals[i];
            if (vals[i] > mx) mx = vals[i];
        }
        scale = degenerate_safe_scale((mx - mn) / 15.0f);
        bias = mn;
        sub = mn;
    }
    uint16_t sb, bb;
    int rc = metadata_bits(scale, bias, &sb, &bb);
    if (rc) return rc;
    /* codes are chosen with the UNROUNDED f32 scale (and unrounded min) */
    float inv = 1.0f / scale;
    memcpy(out, &sb, 2);
    memcpy(out + 2, &bb, 2);
    for (int b = 0; b < 16; ++b) {
        uint8_t q0, q1;
        if (symmetric) {
            q0 = f32_as_u8(clamp015(roundf(vals[2 * b] * inv) + 8.0f));
            q1 = f32_as_u8(clamp015(roundf(vals[2 * b + 1] * inv) + 8.0f));
        } else {
            q0 = f32_as_u8(clamp015(roundf((vals[2 * b] - sub) * inv)));
            q1 = f32_as_u8(clamp015(roundf((vals[2 * b + 1] - sub) * inv)));
        }
        out[4 + b] = (uint8_t)((q1 << 4) | (q0 & 0x0f));
    }
    return ORC_OK;
}

/* quantize_f32_to_q4: flat 32-element chunks of the flattened tensor, last one
 * zero padded.  crates/inference/src/weights/q4_weights.rs:470-487.
 * `symmetric` = 0 is the reference entry point; 1 is exposed for the f64 path. */
int orc_quantize_f32_to_q4(const float* data, size_t len, int symmetric, uint8_t* out) {
    size_t nb = (len + 31) / 32;
    for (size_t blk = 0; blk < nb; ++blk) {
        float vals[32];
        size_t have = len - blk * 32; if (have > 32) have = 32;
        memset(vals, 0, sizeof vals);
        memcpy(vals, data + blk * 32, have * sizeof(float));
        int rc = orc_quantize_block(vals, (int)have, symmetric, out + blk * Q4_BLOCK_BYTES);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* quantize_tensor_q4_0 / quantize_row_q4_0: each row quantized on its own, so a
 * row whose length is not a multiple of 32 ends in its own padded block.
 * crates/inference/src/weights/q4_weights.rs:312-328, 364-388. */
int orc_quantize_tensor_q4_0(const float* src, size_t rows, size_t cols, uint8_t* out) {
    size_t bpr = (cols + 31) / 32;
    for (size_t r = 0; r < rows; ++r) {
        int rc = orc_quantize_f32_to_q4(src + r * cols, cols, 0, out + r * bpr * Q4_BLOCK_BYTES);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* quantize_bf16_to_q4 / stream_quantize_shard: widen bf16, flat chunks, asymmetric.
 * crates/inference/src/weights/q4_weights.rs:428-447, 580-606. */
int orc_quantize_bf16_to_q4(const uint16_t* data, size_t len, uint8_t* out) {
    size_t nb = (len + 31) / 32;
    for (size_t blk = 0; blk < nb; ++blk) {
        float vals[32];
        size_t have = len - blk * 32; if (have > 32) have = 32;
        memset(vals, 0, sizeof vals);
        for (size_t i = 0; i < have; ++i) vals[i] = orc_bf16_bits_to_f32(data[blk * 32 + i]);
        int rc = orc_quantize_block(vals, (int)have, 0, out + blk * Q4_BLOCK_BYTES);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* quantize_f64_to_q4_mode: per-element f64 -> f32 cast, then the f32 block
 * quantizer.  quantize_f64_to_q4 is this with symmetric = 1.
 * crates/inference/src/weights/q4_weights.rs:514-553. */
int orc_quantize_f64_to_q4(const double* data, size_t len, int symmetric, uint8_t* out) {
    size_t nb = (len + 31) / 32;
    for (size_t blk = 0; blk < nb; ++blk) {
        float vals[32];
        size_t have = len - blk * 32; if (have > 32) have = 32;
        memset(vals, 0, sizeof vals);
        for (size_t i = 0; i < have; ++i) vals[i] = (float)data[blk * 32 + i];
        int rc = orc_quantize_block(vals, (int)have, symmetric, out + blk * Q4_BLOCK_BYTES);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* dequantize_q4_to_f32 / dequantize_row_q4_0: w = nibble * scale + bias in f32
 * (multiply, then add), truncated to original_len.
 * crates/inference/src/weights/q4_weights.rs:558-571, 340-353. */
void orc_dequantize_q4_to_f32(const uint8_t* blocks, size_t n_blocks, size_t original_len, float* out) {
    size_t w = 0;
    for (size_t blk = 0; blk < n_blocks && w < original_len; ++blk) {
        const uint8_t* p = blocks + blk * Q4_BLOCK_BYTES;
        uint16_t sb, bb;
        memcpy(&sb, p, 2);
        memcpy(&bb, p + 2, 2);
        float scale = orc_f16_bits_to_f32(sb), bias = orc_f16_bits_to_f32(bb);
        for (int b = 0; b < 16 && w < original_len; ++b) {
            uint8_t byte = p[4 + b];
            out[w++] = (float)(byte & 0x0f) * scale + bias;
            if (w < original_len) out[w++] = (float)(byte >> 4) * scale + bias;
        }
    }
}

/* Per-block metadata validity used by every loader before bytes reach a device:
 * scale finite and > 0, bias finite.
 * crates/inference/src/weights/ingress.rs:542-560. Returns the index of the
 * first bad block, or -1 when all are valid. */
int64_t orc_q4_first_invalid_block(const uint8_t* blocks, size_t n_blocks) {
    for (size_t blk = 0; blk < n_blocks; ++blk) {
        uint16_t sb, bb;
        memcpy(&sb, blocks + blk * Q4_BLOCK_BYTES, 2);
        memcpy(&bb, blocks + blk * Q4_BLOCK_BYTES + 2, 2);
        float s = orc_f16_bits_to_f32(sb), b = orc_f16_bits_to_f32(bb);
        if (!(isfinite(s) && s > 0.0f) || !isfinite(b)) return (int64_t)blk;
    }
    return -1;
}

/* ------------------------------------------------------------------------
 * `.q4` container.  crates/inference/src/weights/q4_weights.rs:623-645 (save),
 * 709-762 (header), 764-810 (exact payload extent).
 *   "KHQ4" | u32 version=2 | u32 ndim | u64 shape[ndim] | u64 original_len | blocks
 * ---------------------------------------------------------------------- */
int orc_q4_write_file(const char* path, const uint64_t* shape, uint32_t ndim,
                      uint64_t original_len, const uint8_t* blocks, size_t n_blocks) {
    FILE* f = fopen(path, "wb");
    if (!f) return ORC_ERR_IO;
    uint32_t ver = 2;
    int ok = fwrite("KHQ4", 1, 4, f) == 4 && fwrite(&ver, 4, 1, f) == 1 && fwrite(&ndim, 4, 1, f) == 1;
    for (uint32_t i = 0; ok && i < ndim; ++i) ok = fwrite(&shape[i], 8, 1, f) == 1;
    ok = ok && fwrite(&original_len, 8, 1, f) == 1;
    ok = ok && fwrite(blocks, Q4_BLOCK_BYTES, n_blocks, f) == n_blocks;
    fclose(f);
    return ok ? ORC_OK : ORC_ERR_IO;
}

/* Parses a whole in-memory `.q4` image.  On success fills ndim, shape (up to 8
 * dims), original_len and payload_offset and checks the exact file extent. */
int orc_q4_parse(const uint8_t* img, size_t img_len, uint32_t* ndim, uint64_t shape[8],
                 uint64_t* original_len, uint64_t* payload_offset) {
    if (img_len < 12 || memcmp(img, "KHQ4", 4) != 0) return ORC_ERR_FORMAT;
    uint32_t ver;
    memcpy(&ver, img + 4, 4);
    if (ver != 2) return ORC_ERR_FORMAT;      /* v1 (18-byte symmetric blocks) is rejected */
    memcpy(ndim, img + 8, 4);
    if (*ndim > 8 || img_len < 12 + 8ull * (*ndim) + 8) return ORC_ERR_FORMAT;
    uint64_t prod = 1;
    for (uint32_t i = 0; i < *ndim; ++i) {
        memcpy(&shape[i], img + 12 + 8 * i, 8);
        if (shape[i] != 0 && prod > UINT64_MAX / shape[i]) return ORC_ERR_SHAPE;
        prod *= shape[i];
    }
    memcpy(original_len, img + 12 + 8 * (*ndim), 8);
    *payload_offset = 20 + 8ull * (*ndim);
    uint64_t nb = (*original_len + 31) / 32;
    if (img_len != *payload_offset + nb * Q4_BLOCK_BYTES) return ORC_ERR_FORMAT; /* truncated or trailing */
    if (prod != *original_len) return ORC_ERR_SHAPE;
    return ORC_OK;
}

/* ------------------------------------------------------------------------
 * matmul_bt: C[m,n] = A[m,k] * B[n,k]^T, f32, single thread.
 * crates/inference/src/forward/cpu/matmul.rs:58-122 (dispatch rule)
 * crates/inference/src/forward/cpu/matmul.rs:143-204 (scalar kernels)
 * crates/inference/src/forward/cpu/tiled.rs:24-93 (4x8x128 blocking)
 * crates/inference/src/forward/cpu/tiled_avx2.rs:16-279
 * crates/inference/src/forward/cpu/arch_kernels.rs:12-139, 214-228
 * ---------------------------------------------------------------------- */
#define TILE_K 128
#define TILE_I 4
#define TILE_J 8

void orc_matmul_bt_scalar(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    if (m == 1) {
        /* eight interleaved partial sums, combined pairwise */
        size_t u8 = k / 8;
        for (size_t j = 0; j < n; ++j) {
            const float* br = b + j * k;
            float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (size_t p = 0; p < u8; ++p)
                for (int l = 0; l < 8; ++l) s[l] += a[p * 8 + l] * br[p * 8 + l];
            for (size_t p = u8 * 8; p < k; ++p) s[0] += a[p] * br[p];
            c[j] = ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]));
        }
        return;
    }
    size_t u4 = k / 4;
    for (size_t i = 0; i < m; ++i) {
        const float* ar = a + i * k;
        for (size_t j = 0; j < n; ++j) {
            const float* br = b + j * k;
            float s0 = 0, s1 = 0, s2 = 0, s3 = 0;
            for (size_t p = 0; p < u4; ++p) {
                s0 += ar[p * 4] * br[p * 4];
                s1 += ar[p * 4 + 1] * br[p * 4 + 1];
                s2 += ar[p * 4 + 2] * br[p * 4 + 2];
                s3 += ar[p * 4 + 3] * br[p * 4 + 3];
            }
            for (size_t p = u4 * 4; p < k; ++p) s0 += ar[p] * br[p];
            c[i * n + j] = (s0 + s1) + (s2 + s3);
        }
    }
}

static void tile_edge_scalar(const float* a, const float* b, float* c, size_t k, size_t n,
                             size_t i0, size_t i1, size_t j0, size_t j1, size_t k0, size_t k1) {
    for (size_t i = i0; i < i1; ++i)
        for (size_t j = j0; j < j1; ++j) {
            float sum = 0.0f;
            for (size_t p = k0; p < k1; ++p) sum += a[i * k + p] * b[j * k + p];
            c[i * n + j] += sum;
        }
}

void orc_matmul_bt_tiled_scalar(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    memset(c, 0, m * n * sizeof(float));
    for (size_t j0 = 0; j0 < n; j0 += TILE_J) {
        size_t j1 = j0 + TILE_J < n ? j0 + TILE_J : n;
        for (size_t i0 = 0; i0 < m; i0 += TILE_I) {
            size_t i1 = i0 + TILE_I < m ? i0 + TILE_I : m;
            for (size_t k0 = 0; k0 < k; k0 += TILE_K) {
                size_t k1 = k0 + TILE_K < k ? k0 + TILE_K : k;
                tile_edge_scalar(a, b, c, k, n, i0, i1, j0, j1, k0, k1);
            }
        }
    }
}

#if defined(__x86_64__)
/* lanes: (x0+x4)+(x1+x5) then + ((x2+x6)+(x3+x7)) */
__attribute__((target("avx2"))) static inline float hsum256(__m256 v) {
    __m128 hi = _mm256_extractf128_ps(v, 1);
    __m128 lo = _mm256_castps256_ps128(v);
    __m128 s = _mm_add_ps(lo, hi);
    __m128 sh = _mm_movehdup_ps(s);
    __m128 t = _mm_add_ps(s, sh);
    __m128 sh2 = _mm_movehl_ps(t, t);
    return _mm_cvtss_f32(_mm_add_ss(t, sh2));
}

__attribute__((target("avx2,fma")))
void orc_matmul_bt_tiled_avx2(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    memset(c, 0, m * n * sizeof(float));
    for (size_t j0 = 0; j0 < n; j0 += TILE_J) {
        size_t j1 = j0 + TILE_J < n ? j0 + TILE_J : n;
        for (size_t i0 = 0; i0 < m; i0 += TILE_I) {
            size_t i1 = i0 + TILE_I < m ? i0 + TILE_I : m;
            for (size_t k0 = 0; k0 < k; k0 += TILE_K) {
                size_t k1 = k0 + TILE_K < k ? k0 + TILE_K : k;
                size_t kl = k1 - k0;
                if (i1 - i0 == TILE_I && j1 - j0 == TILE_J && kl >= 16) {
                    /* one 8-lane accumulator per (row, col); 8 k-values per fma step */
                    __m256 acc[TILE_I][TILE_J];
                    for (int ii = 0; ii < TILE_I; ++ii)
                        for (int jj = 0; jj < TILE_J; ++jj) acc[ii][jj] = _mm256_setzero_ps();
                    size_t steps = kl / 8;      /* the 2x-unrolled pair loop plus its 8-wide tail */
                    for (size_t s = 0; s < steps; ++s) {
                        size_t ko = k0 + s * 8;
                        __m256 bv[TILE_J];
                        for (int jj = 0; jj < TILE_J; ++jj) bv[jj] = _mm256_loadu_ps(b + (j0 + jj) * k + ko);
                        for (int ii = 0; ii < TILE_I; ++ii) {
                            __m256 av = _mm256_loadu_ps(a + (i0 + ii) * k + ko);
                            for (int jj = 0; jj < TILE_J; ++jj) acc[ii][jj] = _mm256_fmadd_ps(av, bv[jj], acc[ii][jj]);
                        }
                    }
                    for (int jj = 0; jj < TILE_J; ++jj)
                        for (int ii = 0; ii < TILE_I; ++ii) c[(i0 + ii) * n + j0 + jj] += hsum256(acc[ii][jj]);
                    size_t ks = k0 + steps * 8;
                    if (ks < k1) tile_edge_scalar(a, b, c, k, n, i0, i1, j0, j1, ks, k1);
                } else {
                    tile_edge_scalar(a, b, c, k, n, i0, i1, j0, j1, k0, k1);
                }
            }
        }
    }
}

__attribute__((target("avx2,fma"))) static float dot_avx2(const float* a, const float* b, size_t len) {
    __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps()};
    size_t chunks = len / 32;
    for (size_t ch = 0; ch < chunks; ++ch)
        for (int u = 0; u < 4; ++u)
            acc[u] = _mm256_fmadd_ps(_mm256_loadu_ps(a + ch * 32 + u * 8), _mm256_loadu_ps(b + ch * 32 + u * 8), acc[u]);
    float sum = hsum256(_mm256_add_ps(_mm256_add_ps(acc[0], acc[1]), _mm256_add_ps(acc[2], acc[3])));
    size_t r8 = (len / 8) * 8;
    for (size_t off = chunks * 32; off < r8; off += 8)
        sum += hsum256(_mm256_mul_ps(_mm256_loadu_ps(a + off), _mm256_loadu_ps(b + off)));
    for (size_t off = r8; off < len; ++off) sum += a[off] * b[off];
    return sum;
}

__attribute__((target("avx2,fma")))
void orc_matmul_bt_avx2(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) c[i * n + j] = dot_avx2(a + i * k, b + j * k, k);
}

/* The 16-lane horizontal add halves the vector repeatedly (lane i + lane i+8,
 * then +4, +2, +1), which is what both the LLVM and GCC reduce intrinsics do. */
__attribute__((target("avx512f"))) static float dot_avx512(const float* a, const float* b, size_t len) {
    __m512 acc[4] = {_mm512_setzero_ps(), _mm512_setzero_ps(), _mm512_setzero_ps(), _mm512_setzero_ps()};
    size_t chunks = len / 64;
    for (size_t ch = 0; ch < chunks; ++ch)
        for (int u = 0; u < 4; ++u)
            acc[u] = _mm512_fmadd_ps(_mm512_loadu_ps(a + ch * 64 + u * 16), _mm512_loadu_ps(b + ch * 64 + u * 16), acc[u]);
    float sum = _mm512_reduce_add_ps(_mm512_add_ps(_mm512_add_ps(acc[0], acc[1]), _mm512_add_ps(acc[2], acc[3])));
    size_t r16 = (len / 16) * 16;
    for (size_t off = chunks * 64; off < r16; off += 16)
        sum += _mm512_reduce_add_ps(_mm512_mul_ps(_mm512_loadu_ps(a + off), _mm512_loadu_ps(b + off)));
    for (size_t off = r16; off < len; ++off) sum += a[off] * b[off];
    return sum;
}

__attribute__((target("avx512f")))
void orc_matmul_bt_avx512(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) c[i * n + j] = dot_avx512(a + i * k, b + j * k, k);
}
#endif

/* 0 = follow the host CPU like the reference does; 1 = force the scalar kernels
 * (results then do not depend on the machine). */
static int g_force_scalar = 0;
void orc_set_force_scalar(int on) { g_force_scalar = on; }

/* Which kernel orc_matmul_bt would pick: 0 scalar, 1 tiled-scalar, 2 tiled-avx2,
 * 3 avx2 dot, 4 avx512 dot. */
int orc_matmul_bt_kernel_id(size_t m, size_t k, size_t n) {
    int avx2 = 0, fma = 0, avx512 = 0;
#if defined(__x86_64__)
    if (!g_force_scalar) {
        avx2 = __builtin_cpu_supports("avx2");
        fma = __builtin_cpu_supports("fma");
        avx512 = __builtin_cpu_supports("avx512f");
    }
#endif
    unsigned long long work = (unsigned long long)m * n * k;
    if (work >= 1024ull * 1024ull && k >= TILE_K) return (avx2 && fma) ? 2 : 1;
    if (avx512 && fma) return 4;
    if (avx2 && fma) return 3;
    return 0;
}

void orc_matmul_bt(const float* a, const float* b, float* c, size_t m, size_t k, size_t n) {
    switch (orc_matmul_bt_kernel_id(m, k, n)) {
#if defined(__x86_64__)
        case 2: orc_matmul_bt_tiled_avx2(a, b, c, m, k, n); return;
        case 3: orc_matmul_bt_avx2(a, b, c, m, k, n); return;
        case 4: orc_matmul_bt_avx512(a, b, c, m, k, n); return;
#endif
        case 1: orc_matmul_bt_tiled_scalar(a, b, c, m, k, n); return;
        default: orc_matmul_bt_scalar(a, b, c, m, k, n); return;
    }
}

/* Stricter second reference: the same product accumulated in f64. */
void orc_matmul_bt_f64acc(const float* a, const float* b, double* c, size_t m, size_t k, size_t n) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            double s = 0.0;
            for (size_t p = 0; p < k; ++p) s += (double)a[i * k + p] * (double)b[j * k + p];
            c[i * n + j] = s;
        }
}

/* ------------------------------------------------------------------------
 * LoRA.  crates/fann/src/lora.rs:113-120 (effective_scale)
 *        crates/tune/src/lora/apply.rs:48-93 (apply_lora)
 *        crates/inference/src/lora_hook.rs:75-207 (apply_lora_rows: one call per row)
 * A is [rank, d_in] row-major, B is [d_out, rank] row-major.
 * ---------------------------------------------------------------------- */
float orc_effective_scale(size_t rank, float alpha) {
    float scale = rank == 0 ? 0.0f : alpha / (float)rank;
    return (isfinite(alpha) && isfinite(scale)) ? scale : 0.0f;
}

/* Returns 1 when the update was applied, 0 when the shapes disagree (silent
 * no-op, as in the reference). a_len / b_len are element counts. */
int orc_apply_lora(const float* a, size_t a_len, const float* b, size_t b_len, size_t rank,
                   size_t d_in, size_t d_out, float scale, const float* x, size_t x_len,
                   float* out, size_t out_len) {
    if (x_len != d_in || out_len != d_out || rank * d_in != a_len || d_out * rank != b_len) return 0;
    float* t = (float*)malloc((rank ? rank : 1) * sizeof(float));
    for (size_t r = 0; r < rank; ++r) {
        float acc = 0.0f;                                /* sequential f32 sum */
        for (size_t p = 0; p < d_in; ++p) acc += a[r * d_in + p] * x[p];
        t[r] = acc;
    }
    for (size_t o = 0; o < d_out; ++o) {
        float acc = 0.0f;
        for (size_t r = 0; r < rank; ++r) acc += b[o * rank + r] * t[r];
        out[o] += scale * acc;
    }
    free(t);
    return 1;
}

/* ------------------------------------------------------------------------
 * Walsh-Hadamard and the randomized Hadamard rotation R = H * D.
 * crates/inference/src/quant/quarot/hadamard.rs:22-112 (transforms)
 * crates/inference/src/quant/quarot/hadamard.rs:114-160 (splitmix64 signs, block seed)
 * crates/inference/src/quant/quarot/hadamard.rs:176-259 (apply / apply_inverse, f32 and f64)
 * ---------------------------------------------------------------------- */
#define SPLITMIX64_GAMMA 0x9E3779B97F4A7C15ull

uint64_t orc_splitmix64_mix(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

void orc_signs_from_seed(uint64_t seed, size_t n, float* out) {
    uint64_t state = seed + SPLITMIX64_GAMMA;
    for (size_t i = 0; i < n; ++i) {
        state += SPLITMIX64_GAMMA;
        out[i] = (orc_splitmix64_mix(state) & 1ull) == 0 ? 1.0f : -1.0f;
    }
}

uint64_t orc_derive_block_seed(uint64_t seed, uint64_t block_index) {
    return orc_splitmix64_mix(seed + block_index * SPLITMIX64_GAMMA);
}

static int is_pow2(size_t n) { return n != 0 && (n & (n - 1)) == 0; }

int orc_walsh_hadamard_f32(float* d, size_t n) {
    if (!is_pow2(n)) return ORC_ERR_POW2;
    for (size_t h = 1; h < n; h *= 2)
        for (size_t i = 0; i < n; i += 2 * h)
            for (size_t j = i; j < i + h; ++j) {
                float x = d[j], y = d[j + h];
                d[j] = x + y;
                d[j + h] = x - y;
            }
    return ORC_OK;
}

int orc_walsh_hadamard_f64(double* d, size_t n) {
    if (!is_pow2(n)) return ORC_ERR_POW2;
    for (size_t h = 1; h < n; h *= 2)
        for (size_t i = 0; i < n; i += 2 * h)
            for (size_t j = i; j < i + h; ++j) {
                double x = d[j], y = d[j + h];
                d[j] = x + y;
                d[j + h] = x - y;
            }
    return ORC_OK;
}

int orc_walsh_hadamard_orthonormal_f32(float* d, size_t n) {
    int rc = orc_walsh_hadamard_f32(d, n);
    if (rc) return rc;
    float s = 1.0f / sqrtf((float)n);
    for (size_t i = 0; i < n; ++i) d[i] *= s;
    return ORC_OK;
}

int orc_walsh_hadamard_orthonormal_f64(double* d, size_t n) {
    int rc = orc_walsh_hadamard_f64(d, n);
    if (rc) return rc;
    double s = 1.0 / sqrt((double)n);
    for (size_t i = 0; i < n; ++i) d[i] *= s;
    return ORC_OK;
}

/* R x = H (D x): signs first, then the orthonormal transform. */
int orc_rh_apply_f32(const float* signs, size_t n, float* d) {
    if (!is_pow2(n)) return ORC_ERR_POW2;
    for (size_t i = 0; i < n; ++i) d[i] *= signs[i];
    return orc_walsh_hadamard_orthonormal_f32(d, n);
}
int orc_rh_apply_f64(const float* signs, size_t n, double* d) {
    if (!is_pow2(n)) return ORC_ERR_POW2;
    for (size_t i = 0; i < n; ++i) d[i] *= (double)signs[i];
    return orc_walsh_hadamard_orthonormal_f64(d, n);
}
/* R^T x = D (H x). */
int orc_rh_apply_inverse_f32(const float* signs, size_t n, float* d) {
    int rc = orc_walsh_hadamard_orthonormal_f32(d, n);
    if (rc) return rc;
    for (size_t i = 0; i < n; ++i) d[i] *= signs[i];
    return ORC_OK;
}
int orc_rh_apply_inverse_f64(const float* signs, size_t n, double* d) {
    int rc = orc_walsh_hadamard_orthonormal_f64(d, n);
    if (rc) return rc;
    for (size_t i = 0; i < n; ++i) d[i] *= (double)signs[i];
    return ORC_OK;
}

/* BlockHadamard (crates/inference/src/quant/quarot/hadamard.rs:285-484): a block-diagonal rotation
 * of a length-n vector, every block of `block` entries with its own sign diagonal and the
 * orthonormal Walsh-Hadamard of that size.  The constructor's checks (hadamard.rs:358-400): n != 0,
 * n <= 1 << 24, block a power of two that divides n, n / block <= 4096.  Block i's signs are
 * signs_from_seed(derive_block_seed(seed, i), block), stored back to back (hadamard.rs:401-414). */
#define ORC_MAX_BLOCK_HADAMARD_LEN ((size_t)1 << 24)
#define ORC_MAX_BLOCK_HADAMARD_BLOCKS 4096

int orc_block_hadamard_check(size_t n, size_t block) {
    if (n == 0 || n > ORC_MAX_BLOCK_HADAMARD_LEN) return ORC_ERR_SHAPE;
    if (!is_pow2(block)) return ORC_ERR_POW2;
    if (n % block != 0) return ORC_ERR_SHAPE;
    if (n / block > ORC_MAX_BLOCK_HADAMARD_BLOCKS) return ORC_ERR_SHAPE;
    return ORC_OK;
}

int orc_block_hadamard_signs(uint64_t seed, size_t n, size_t block, float* out) {
    int rc = orc_block_hadamard_check(n, block);
    if (rc) return rc;
    for (size_t i = 0; i < n / block; ++i) orc_signs_from_seed(orc_derive_block_seed(seed, i), block, out + i * block);
    return ORC_OK;
}

/* apply (hadamard.rs:444-462): per block D then H; apply_inverse (hadamard.rs:465-482): H then D. */
int orc_block_hadamard_apply_f32(const float* signs, size_t n, size_t block, float* d, int inverse) {
    int rc = orc_block_hadamard_check(n, block);
    if (rc) return rc;
    for (size_t b0 = 0; b0 < n; b0 += block) {
        rc = inverse ? orc_rh_apply_inverse_f32(signs + b0, block, d + b0) : orc_rh_apply_f32(signs + b0, block, d + b0);
        if (rc) return rc;
    }
    return ORC_OK;
}


/* ------------------------------------------------------------------------
 * Rotation absorption.  crates/inference/src/quant/quarot/rotation.rs:82-195.
 * input side:  W <- W R^T  == apply R to every ROW   (rotation dim = cols)
 * output side: W <- R W    == apply R to every COLUMN (rotation dim = rows)
 * ---------------------------------------------------------------------- */
int orc_absorb_input_rotation_f64(double* w, size_t rows, size_t cols, const float* signs, size_t dim) {
    if (dim != cols) return ORC_ERR_SHAPE;
    for (size_t r = 0; r < rows; ++r) {
        int rc = orc_rh_apply_f64(signs, cols, w + r * cols);
        if (rc) return rc;
    }
    return ORC_OK;
}
int orc_absorb_input_rotation_f32(float* w, size_t rows, size_t cols, const float* signs, size_t dim) {
    if (dim != cols) return ORC_ERR_SHAPE;
    for (size_t r = 0; r < rows; ++r) {
        int rc = orc_rh_apply_f32(signs, cols, w + r * cols);
        if (rc) return rc;
    }
    return ORC_OK;
}
int orc_absorb_output_rotation_f64(double* w, size_t rows, size_t cols, const float* signs, size_t dim) {
    if (dim != rows) return ORC_ERR_SHAPE;
    double* col = (double*)malloc(rows * sizeof(double));
    for (size_t c = 0; c < cols; ++c) {
        for (size_t r = 0; r < rows; ++r) col[r] = w[r * cols + c];
        int rc = orc_rh_apply_f64(signs, rows, col);
        if (rc) { free(col); return rc; }
        for (size_t r = 0; r < rows; ++r) w[r * cols + c] = col[r];
    }
    free(col);
    return ORC_OK;
}
int orc_absorb_output_rotation_f32(float* w, size_t rows, size_t cols, const float* signs, size_t dim) {
    if (dim != rows) return ORC_ERR_SHAPE;
    float* col = (float*)malloc(rows * sizeof(float));
    for (size_t c = 0; c < cols; ++c) {
        for (size_t r = 0; r < rows; ++r) col[r] = w[r * cols + c];
        int rc = orc_rh_apply_f32(signs, rows, col);
        if (rc) { free(col); return rc; }
        for (size_t r = 0; r < rows; ++r) w[r * cols + c] = col[r];
    }
    free(col);
    return ORC_OK;
}

/* Adapter rotation for a QuaRot base.
 * crates/inference/src/quant/quarot/lora.rs:32-59: an input-side module's A
 * [rank, d_in] becomes A R^T (R applied to each row of A); an output-side
 * module's B [d_out, rank] becomes R B (R applied to each column of B). */
int orc_counter_rotate_a(float* a, size_t rank, size_t d_in, const float* signs, size_t dim) {
    return orc_absorb_input_rotation_f32(a, rank, d_in, signs, dim);
}
int orc_rotate_b_output_side(float* b, size_t d_out, size_t rank, const float* signs, size_t dim) {
    return orc_absorb_output_rotation_f32(b, d_out, rank, signs, dim);
}

/* ------------------------------------------------------------------------
 * The composed reference linear: what the reference's own tests use as the
 * CPU answer for a Q4 (+LoRA) projection, with the optional online rotation.
 *   [x' = R x per row]  ->  W = dequantize  ->  y = matmul_bt(x', W)
 *   ->  per row: apply_lora(x' row, y row)
 * crates/inference/src/forward/metal_qwen35.rs:22850-22899 (dequant -> f32 matmul),
 * crates/inference/src/model/qwen35/forward.rs:449-492 (matmul_bt then lora.apply).
 * `w_f32` may carry the already dequantized weights (n*k floats) to skip that step;
 * otherwise pass NULL and `payload`.
 * ---------------------------------------------------------------------- */
int orc_q4_linear(const float* x, const uint8_t* payload, const float* w_f32, float* y,
                  size_t m, size_t n, size_t k,
                  const float* lora_a, const float* lora_b, size_t rank, float lora_scale,
                  const float* rot_signs) {
    if (m == 0 || n == 0) return ORC_OK;
    if (k == 0 || k % 32 != 0) return ORC_ERR_SHAPE;
    float* xr = NULL;
    const float* xin = x;
    if (rot_signs) {
        xr = (float*)malloc(m * k * sizeof(float));
        memcpy(xr, x, m * k * sizeof(float));
        for (size_t i = 0; i < m; ++i) {
            int rc = orc_rh_apply_f32(rot_signs, k, xr + i * k);
            if (rc) { free(xr); return rc; }
        }
        xin = xr;
    }
    float* w = NULL;
    if (!w_f32) {
        w = (float*)malloc(n * k * sizeof(float));
        orc_dequantize_q4_to_f32(payload, n * (k / 32), n * k, w);
        w_f32 = w;
    }
    orc_matmul_bt(xin, w_f32, y, m, k, n);
    if (lora_a && lora_b && rank > 0)
        for (size_t i = 0; i < m; ++i)
            orc_apply_lora(lora_a, rank * k, lora_b, n * rank, rank, k, n, lora_scale,
                           xin + i * k, k, y + i * n, n);
    free(w);
    free(xr);
    return ORC_OK;
}

/* Second CPU formulation: the arithmetic of the reference's decode shader,
 * crates/inference/src/forward/shaders/qwen35.metal:799-866, written as plain
 * loops: per 8-weight slice  sum(nibble*x)*d + b*sum(x), slices of a row added
 * in the shader's lane order is NOT reproduced (a sum order the GPU picks);
 * slices are added left to right. */
void orc_gemv_q4_decode_form(const float* x, const uint8_t* payload, float* y, size_t n, size_t k) {
    size_t nb = k / 32;
    for (size_t r = 0; r < n; ++r) {
        float acc = 0.0f;
        for (size_t ib = 0; ib < nb; ++ib) {
            const uint8_t* p = payload + (r * nb + ib) * Q4_BLOCK_BYTES;
            uint16_t sb, bb;
            memcpy(&sb, p, 2);
            memcpy(&bb, p + 2, 2);
            float d = orc_f16_bits_to_f32(sb), b = orc_f16_bits_to_f32(bb);
            for (int il = 0; il < 4; ++il) {
                const float* xs = x + ib * 32 + il * 8;
                float xsum = 0.0f, dot = 0.0f;
                for (int i = 0; i < 8; ++i) xsum += xs[i];
                for (int i = 0; i < 4; ++i) {
                    uint8_t byte = p[4 + il * 4 + i];
                    dot += (float)(byte & 0xf) * xs[2 * i] + (float)(byte >> 4) * xs[2 * i + 1];
                }
                acc += dot * d + b * xsum;
            }
        }
        y[r] = acc;
    }
}

/* QuaRot's online "Hadamard heads" factor H_num_heads (x) I_head_dim on a [num_heads * head_dim] activation
 * (apply_cross_head_rotation, crates/inference/src/quant/quarot/r3_reference.rs:246-264; the R3 descriptor
 * is OnlineRotationSpec::r3_full_attention, quant/quarot/plan.rs): for every within-head channel d the
 * num_heads values data[h * head_dim + d] are gathered, rotated by ONE RandomizedHadamard of dimension
 * num_heads (signs, then the orthonormal transform) and scattered back. */
int orc_cross_head_rotation_f32(const float* signs, size_t num_heads, size_t head_dim, float* data) {
    if (!is_pow2(num_heads)) return ORC_ERR_POW2;
    float* channel = (float*)malloc(num_heads * sizeof(float));
    if (!channel) return ORC_ERR_SHAPE;
    int rc = ORC_OK;
    for (size_t d = 0; d < head_dim && rc == ORC_OK; ++d) {
        for (size_t h = 0; h < num_heads; ++h) channel[h] = data[h * head_dim + d];
        rc = orc_rh_apply_f32(signs, num_heads, channel);
        for (size_t h = 0; h < num_heads; ++h) data[h * head_dim + d] = channel[h];
    }
    free(channel);
    return rc;
}

/* silu_mul_fused (crates/inference/src/forward/shaders/qwen35.metal:712-722) on one token's merged
 * gate || up row: out[i] = gate[i] / (1 + exp(-gate[i])) * up[i], gate = data[0, count), up = data[count, 2 count). */
void orc_silu_mul(const float* gate_up, size_t count, float* out) {
    for (size_t i = 0; i < count; ++i) {
        float gate = gate_up[i], up = gate_up[count + i];
        float s = gate / (1.0f + expf(-gate));
        out[i] = s * up;
    }
}

/* Exact top-k of a logit row in the reference's candidate order:
 * topk_better (crates/inference/src/forward/shaders/qwen35.metal:1697-1703) ranks the higher logit
 * first and breaks ties towards the lower token id; a NaN logit becomes the sentinel
 * (-inf, UINT32_MAX) before it competes (qwen35.metal:1916, :1967), so it never displaces a real
 * token.  Slots past the number of candidates keep the sentinel, as the padded bitonic sort of
 * the merge pass leaves them (qwen35.metal:1746-1768). */
static int orc_topk_better(float al, uint32_t ai, float bl, uint32_t bi) {
    if (al != al) return 0;
    if (bl != bl) return 1;
    if (al != bl) return al > bl;
    return ai < bi;
}

void orc_topk(const float* logits, size_t n, size_t k, float* out_logit, uint32_t* out_id) {
    for (size_t j = 0; j < k; ++j) { out_logit[j] = -INFINITY; out_id[j] = UINT32_MAX; }
    if (k == 0) return;
    for (size_t i = 0; i < n; ++i) {
        float v = logits[i];
        uint32_t id = (uint32_t)i;
        if (v != v) { v = -INFINITY; id = UINT32_MAX; }
        if (!orc_topk_better(v, id, out_logit[k - 1], out_id[k - 1])) continue;
        size_t j = k - 1;
        while (j > 0 && orc_topk_better(v, id, out_logit[j - 1], out_id[j - 1])) {
            out_logit[j] = out_logit[j - 1];
            out_id[j] = out_id[j - 1];
            --j;
        }
        out_logit[j] = v;
        out_id[j] = id;
    }
}

int orc_abi_version(void) { return 1; }
