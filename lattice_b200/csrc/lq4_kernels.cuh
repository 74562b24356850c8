// Host-callable launchers of the kernels; the C ABI in lq4_api.cu validates
// arguments and then calls these.
#pragma once

#include "lq4_common.cuh"

namespace lq4 {

// ---- lq4_api.cu ---------------------------------------------------------------
// Stores the message lq4_last_error() returns on the calling thread.
void set_last_error(const char* msg);

// ---- lq4_aux.cu ---------------------------------------------------------------
void launch_dequant(const uint8_t* payload, uint64_t n_blocks, float* out, int sm_count, cudaStream_t s);
void launch_quantize(const float* data, uint64_t len, int symmetric, uint8_t* payload, int32_t* status,
                     int sm_count, cudaStream_t s);
cudaError_t launch_hadamard_rows(const void* x, int x_dtype, const float* signs, uint32_t dim, uint32_t rows,
                                 float* out, cudaStream_t s);
void launch_rot_signs(uint64_t seed, uint32_t dim, float* signs, cudaStream_t s);

// ---- lq4_gemv.cu ----------------------------------------------------------------
// Geometry of the decode kernel.
constexpr int kGemvTileRows = 128;        // output rows per tile: 8 consumer warps x 16
constexpr int kGemvStageBlocks = 16;      // Q4 blocks (of one row) per pipeline stage
constexpr int kGemvGranuleBlocks = 4;     // stream-K split granularity along k (16-byte aligned pieces)
constexpr int kGemvRowStride = kGemvStageBlocks * kBlockBytes + 16;   // 336 B: rows 4 banks apart (x odd)
constexpr int kGemvStageWBytes = kGemvTileRows * kGemvRowStride;      // 43008
constexpr int kGemvThreads = 288;         // 8 consumer warps + 1 producer warp
constexpr int kGemvMaxM = 16;
constexpr int kGemvMaxRank = 128;
constexpr int kMaxSmem = 232448;          // 227 KB opt-in limit per CTA

struct GemvParams {
    const uint8_t* w;
    float* y;
    uint64_t ldy;
    uint32_t m, n, k;
    uint32_t kb;            // k / 32
    uint32_t kg;            // granules per row = kb / 4
    uint32_t tiles;         // ceil(n / 128)
    uint32_t nt;            // n-tiles of 8 columns: ceil(2m / 8)
    uint32_t gmax;          // fragment columns stored per n-tile (2, 4, 6 or 8)
    uint32_t nstages;
    // resident-activation variant: raw activations, converted in the CTA prologue
    const void* x;
    int32_t x_dtype;
    const float* signs;     // non-NULL: rotate in the prologue (k a power of two)
    // staged-activation variant: fragments and block sums prepared by prep_xs
    const uint8_t* xs_g;
    const float* sx_g;
    const float* t_g;       // staged variant: finished t[m][rank]
    // LoRA
    const float* la;
    const float* lb;
    uint32_t rank;
    float lscale;
    float* tpart;           // resident variant: [grid][m*rank] partial projections
    uint32_t* tsync;        // resident variant: {arrived, finished}
    // stream-K fix-up
    float* partials;        // [grid][2][128 * nt * 4]
    uint32_t* tickets;      // [tiles * 8]
    int32_t* status;
    // shared-memory offsets (bytes from the dynamic smem base)
    uint32_t off_t, off_stage, stage_bytes, off_stage_xs, off_stage_sx, off_xs, off_sx, off_xrot;
    uint32_t use_pdl;
    // resident decode kernel (lq4_decode.cu)
    uint32_t stage_blocks;  // Q4 blocks of one row per pipeline stage: 20, 12 or 4
    uint32_t spt;           // stages per tile = ceil(kb / stage_blocks)
    int32_t sm_count;       // SMs of the device (0: assume 148)
    uint32_t whole_tiles;   // 1: every CTA gets entire tiles, no cross-CTA partial sums
};

// ---- lq4_decode.cu ---------------------------------------------------------------
// Resident decode kernel (m <= 4): picks the stage length, fills the shared-memory offsets of
// `p` and returns the dynamic shared memory needed (0 if the activation rows do not fit).
size_t decode_plan_smem(GemvParams& p);
// Work units (tile, stage) of a planned launch; the grid is min(#SM, units).
uint64_t decode_units(const GemvParams& p);
cudaError_t launch_decode(const GemvParams& p, size_t smem, int grid, cudaStream_t s);
// Several independent projections of the same token count in ONE persistent launch: the work
// units of all problems form one stream-K range, so launch, prologue and tail are paid once.
constexpr int kMaxGroup = 8;
// Fills the shared-memory fields of every problem (sized for the longest k) and returns the
// dynamic shared memory needed, or 0 if the group cannot run in one launch.
size_t decode_group_plan_smem(GemvParams* ps, uint32_t count);
uint64_t decode_group_units(const GemvParams* ps, uint32_t count);
cudaError_t launch_decode_group(const GemvParams* ps, uint32_t count, size_t smem, int grid, cudaStream_t s);
// t[i] = A_i x_i for every problem of the group that has an adapter, in one launch (none: no launch).
cudaError_t launch_lora_project_group(const GemvParams* ps, uint32_t count, float* const* t, uint32_t m, int use_pdl,
                                      cudaStream_t s);
// t = A x for the decode kernel's LoRA epilogue; launched right before launch_decode.
cudaError_t launch_lora_project(const void* x, int x_dtype, uint32_t m, uint32_t k, const float* la, uint32_t rank,
                                float* t, int use_pdl, cudaStream_t s);

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

// Fills the smem-dependent fields of `p` and returns the dynamic shared memory the
// launch needs, or 0 if the shape does not fit the requested variant.
size_t gemv_plan_smem(GemvParams& p, bool resident);
bool gemv_resident_fits(uint32_t m, uint32_t k, bool rot);
cudaError_t launch_gemv_mma(const GemvParams& p, bool resident, size_t smem, int grid, cudaStream_t s);

// Activation preparation for the staged variant and for the generic kernel.
void launch_prep_xs(const void* x, int x_dtype, uint32_t m, uint32_t k, uint32_t nt, uint32_t gmax, uint8_t* xs_g,
                    float* sx_g, cudaStream_t s);
void launch_lora_t(const void* x, int x_dtype, uint32_t m, uint32_t k, const float* la, uint32_t rank, float* t,
                   cudaStream_t s);
void launch_gemv_generic(const void* x, int x_dtype, const uint8_t* w, float* y, uint64_t ldy, uint32_t m,
                         uint32_t n, uint32_t k, const float* t, const float* lb, uint32_t rank, float lscale,
                         int accumulate_only, cudaStream_t s);

}  // namespace lq4
