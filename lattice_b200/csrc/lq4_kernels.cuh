// Host-callable launchers of the kernels; the C ABI in lq4_api.cu validates
// arguments and then calls these.
#pragma once

#include "lq4_common.cuh"
#include "lq4_once.h"

namespace lq4 {

// Opts kernel `fn` in to `bytes` of dynamic shared memory on the CURRENT device, once per device.
inline cudaError_t opt_in_smem(const void* fn, int bytes, DeviceOnce& once) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (!once.needs(dev)) return cudaSuccess;
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) once.mark(dev);
    return e;
}

// ---- lq4_api.cu ---------------------------------------------------------------
// Stores the message lq4_last_error() returns on the calling thread.
void set_last_error(const char* msg);

// ---- lq4_aux.cu ---------------------------------------------------------------
void launch_dequant(const uint8_t* payload, uint64_t n_blocks, float* out, int sm_count, cudaStream_t s);
// `rows` runs of `row_len` values of type `dtype` (LQ4_DTYPE_*), each run cut into 32-value blocks of its own.
void launch_quantize(const void* data, int dtype, uint64_t rows, uint64_t row_len, int symmetric, uint8_t* payload,
                     int32_t* status, int sm_count, cudaStream_t s);
// Rotation absorption into a row-major weight matrix, in place (f32 or f64): R applied to every row of
// length `dim`, or to every column of a matrix with `dim` rows.
cudaError_t launch_absorb_input(void* w, int dtype, uint64_t rows, uint32_t dim, const float* signs, cudaStream_t s);
cudaError_t launch_absorb_output(void* w, int dtype, uint32_t dim, uint64_t cols, const float* signs, int sm_count,
                                 cudaStream_t s);
cudaError_t launch_hadamard_rows(const void* x, int x_dtype, const float* signs, uint32_t dim, uint32_t rows,
                                 float* out, cudaStream_t s, uint32_t sign_rows = 1);
cudaError_t launch_cross_head_rows(const float* x, const float* signs, uint32_t num_heads, uint32_t head_dim,
                                   uint32_t rows, float* out, cudaStream_t s);
cudaError_t launch_silu_mul_rows(const float* gate_up, uint32_t rows, uint32_t inter, float* h, int sm_count,
                                 cudaStream_t s);
void launch_block_rot_signs(uint64_t seed, uint32_t n, uint32_t block, float* signs, cudaStream_t s);
void launch_rot_signs(uint64_t seed, uint32_t dim, float* signs, cudaStream_t s);

// ---- decode kernels: geometry and parameters ------------------------------------------
constexpr int kGemvTileRows = 128;        // output rows per tile: 8 consumer warps x 16
constexpr int kGemvGranuleBlocks = 4;     // stream-K split granularity along k (16-byte aligned pieces)
constexpr int kGemvThreads = 288;         // 8 consumer warps + 1 producer warp
constexpr int kGemvMaxM = 16;             // tokens per decode launch
constexpr int kGemvMaxRank = 512;        // decode kernels (m <= 16); a blend of adapters adds their ranks
constexpr int kGemmMaxRank = 128;        // tensor-core kernel: the adapter rides along as extra k segments
constexpr int kMaxSmem = 232448;          // 227 KB opt-in limit per CTA

// One projection as the decode kernels see it.
struct GemvParams {
    const uint8_t* w;
    float* y;
    uint64_t ldy;
    uint32_t m, n, k;
    uint32_t kb;            // k / 32
    uint32_t kg;            // granules per row = kb / 4
    uint32_t tiles;         // ceil(n / 128)
    uint32_t nstages;
    const void* x;          // activations [m, k]
    const float* x_mul;      // f32 activations, no rotation: the input is silu(x[i]) * x_mul[i] (NULL: x itself)
    uint32_t ldx;            // with x_mul: floats between token rows of x and of x_mul (0: k)
    int32_t x_dtype;
    const float* signs;     // resident kernel only; non-NULL: rotate in the prologue (k a power of two)
    const uint8_t* xs_g;    // dense kernel: activation limb records prepared by launch_dense_prep
    // LoRA: t = A x
    const float* t_g;       // dense kernel: [m][rank], finished by the launch before it
    uint2* tmsg;            // resident kernel: [m][rank][tsplit] {partial dot, tag} messages written by the kernel itself
    uint32_t tsplit;        // resident kernel: pieces each projection dot product is cut into along k
    const float* la;
    const float* lb;
    uint32_t rank;
    float lscale;
    // cross-CTA state
    uint32_t* tsync;        // 64-bit launch counter (8-byte aligned), see launch_tag()
    float* partials;        // [grid][128 rows][tokens] 8-byte {partial sum, tag} messages
    int32_t* status;
    // shared-memory offsets (bytes from the dynamic smem base)
    uint32_t off_stage, off_xs, off_sx, off_xrot, off_t;
    uint32_t use_pdl;
    // fused all-gather (world > 1): results are also written into every peer's buffer
    uint32_t world, grank;
    int64_t peer_off[LQ4_MAX_PEERS];                  // bytes from an element of y to the same element in peer r
    unsigned long long* peer_arrive[LQ4_MAX_PEERS];   // peer r's arrival counter
    unsigned long long* gseq;                         // this rank's count of gathered launches (x 256); gseq[1] counts the CTAs of the running launch
    // x depends on gathered results: wait for the peers' arrivals before reading it (wait_world > 1)
    const unsigned long long* wait_arrive;            // own arrival counter; own sequence counter follows it
    uint32_t wait_world;
    int32_t sm_count;       // SMs of the device (0: assume 148)
    uint32_t whole_tiles;   // resident kernel: every CTA gets entire tiles, no cross-CTA partial sums
};

// ---- lq4_decode.cu ---------------------------------------------------------------
// Resident decode kernel (m <= 4): picks the stage length, fills the shared-memory offsets of
// `p` and returns the dynamic shared memory needed (0 if the activation rows do not fit).
size_t decode_plan_smem(GemvParams& p);
// Work units (tile, stage) of a planned launch; the grid is min(#SM, units).
uint64_t decode_units(const GemvParams& p);
cudaError_t launch_decode(const GemvParams& p, size_t smem, int grid, cudaStream_t s);
// Pieces the resident kernel cuts each LoRA projection dot product into along k (one warp each).
constexpr uint32_t kDecodeMaxTsplit = 8;
inline uint32_t decode_tsplit(uint32_t k) {
    const uint32_t s = (k / 4 + 767) / 768;
    return s < 1 ? 1 : (s > kDecodeMaxTsplit ? kDecodeMaxTsplit : s);
}
// Several independent projections of the same token count in ONE persistent launch: the work
// units of all problems form one stream-K range, so launch, prologue and tail are paid once.
constexpr int kMaxGroup = 8;
// Fills the shared-memory fields of every problem (sized for the longest k) and returns the
// dynamic shared memory needed, or 0 if the group cannot run in one launch.
size_t decode_group_plan_smem(GemvParams* ps, uint32_t count);
uint64_t decode_group_units(const GemvParams* ps, uint32_t count);
cudaError_t launch_decode_group(const GemvParams* ps, uint32_t count, size_t smem, int grid, cudaStream_t s);

// ---- lq4_dense.cu ---------------------------------------------------------------
// Decode kernel for 2..16 tokens (any k): activation limbs are prepared per call into per-block
// records (dense_record_bytes each problem) by launch_dense_prep, which also computes t = A x
// for the problems with an adapter; launch_dense then serves 1..kMaxGroup problems of the same
// token count in one persistent launch.  GemvParams::xs_g points at a problem's records.
size_t dense_record_bytes(uint32_t m, uint32_t k);
size_t dense_plan_smem(GemvParams* ps, uint32_t count);
cudaError_t launch_dense_prep(const GemvParams* ps, uint32_t count, uint8_t* const* rec, float* const* t, int use_pdl,
                              cudaStream_t s);
cudaError_t launch_dense(const GemvParams* ps, uint32_t count, size_t smem, int grid, cudaStream_t s);

// True if `m` (<= 4) activation rows of length k fit the resident decode kernel's shared memory.
bool gemv_resident_fits(uint32_t m, uint32_t k, bool rot);

// Fallbacks for shapes the TMA-based kernels do not take (lq4_gemv.cu).
void launch_lora_t(const void* x, int x_dtype, uint32_t m, uint32_t k, const float* la, uint32_t rank, float* t,
                   cudaStream_t s);
void launch_gemv_generic(const void* x, int x_dtype, const uint8_t* w, float* y, uint64_t ldy, uint32_t m,
                         uint32_t n, uint32_t k, const float* t, const float* lb, uint32_t rank, float lscale,
                         int accumulate_only, cudaStream_t s);

// Exact top-k of a logit row (lq4_topk.cu), one launch.  `lists` holds topk_list_bytes(n, k) bytes; `counters`
// holds topk_counter_bytes(n) bytes that are zero before their first use (every launch leaves them zero).
size_t topk_list_bytes(uint32_t n, uint32_t k);
size_t topk_counter_bytes(uint32_t n);
cudaError_t launch_topk(const float* logits, uint32_t n, uint32_t k, void* lists, uint32_t* counters,
                        lq4_topk_candidate* out, int use_pdl, cudaStream_t s, int* launches);

}  // namespace lq4
