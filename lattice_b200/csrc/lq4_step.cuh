// Decode step kernel: an ordered list of groups of one-token projections in ONE persistent launch
// (lq4_step.cu).  Declarations shared with the C ABI in lq4_api.cu.
#pragma once

#include <cuda.h>

#include "lq4_kernels.cuh"
#include "lq4_step_share.h"

namespace lq4 {

constexpr int kStepMaxProblems = 24;     // at most 32: dec::split_ctas sizes its tables for that
constexpr int kStepMaxGroups = 8;
constexpr int kStepMaxRanges = 8;
constexpr uint32_t kNoSlot = 0xffffffffu;
// Dot products t = A x whose x comes from the mailbox are cut into pieces short enough for ONE lane of the
// projection warp to keep all its loads in flight: at most kStepMailboxStrides float4 per lane.
constexpr int kStepMailboxStrides = 4;
constexpr uint32_t kStepMaxTsplit = 64;

// One projection of a step.  Activations come from plain memory (ready when the launch starts) or from
// the step's mailbox (written by an earlier group of the same launch, on this GPU or on a peer).
struct StepProblem {
    float* y;                  // this rank's output rows, plain f32
    const void* x;             // plain activations; unused when x_slot != kNoSlot
    const float* x_mul;        // plain gating multiplier: the input is silu(x) * x_mul (NULL: none)
    const float* la;           // LoRA A [rank, k]
    const float* lb;           // LoRA B [n, rank]
    uint2* tmsg;               // {partial dot, tag} messages of this problem's projection t = A x
    uint32_t n, k, kb, kg, tiles;
    uint32_t x_slot;           // mailbox index of x[0], or kNoSlot
    uint32_t xmul_slot;        // mailbox index of the gating row, or kNoSlot
    uint32_t y_slot;           // mailbox index of y[0] (published for later groups and for the peers), or kNoSlot
    uint32_t rank, tsplit;
    float lscale;
    int32_t x_dtype;
    uint32_t cta_begin, cta_count;   // CTAs [cta_begin, cta_begin + cta_count) of the grid work on this problem in its group
    uint32_t dot_begin;        // first projection work item of this problem within its group
    uint32_t charge;           // work units a CTA is charged for finishing a tile (see step_share_begin)
    uint32_t pad_[2];
};

struct StepArgs {
    StepProblem p[kStepMaxProblems];
    CUtensorMap maps[kStepMaxProblems][3];       // boxes of 20, 12 and 4 blocks x 128 rows
    uint32_t group_begin[kStepMaxGroups + 1];    // problems [group_begin[g], group_begin[g + 1]) form group g
    uint32_t group_items[kStepMaxGroups];        // projection work items of group g
    uint32_t ngroups;
    uint32_t use_pdl;
    // shared-memory plan (bytes from the dynamic shared memory base)
    uint32_t off_t, t_stride, off_tstage, off_cstage, off_stage, nstages;
    uint32_t off_xbuf, xbuf_stride, xbuf_sx, nxbuf;   // limb buffers: nxbuf (1 or 2) of xbuf_stride bytes, {scale, sum} at xbuf_sx
    // cross-CTA state of this GPU
    uint32_t* tsync;           // 64-bit launch counter: tags of the partial-sum and projection messages
    float* partials;           // [group][grid][128 rows] 8-byte {partial sum, tag} messages
    int32_t* status;
    // mailbox: 8-byte {value, step tag} entries, two halves used by alternate steps
    unsigned long long* mbox;  // this GPU's mailbox (2 * mbox_half entries)
    uint32_t mbox_half;
    uint32_t world, grank;
    uint32_t* step_counter;    // 64-bit counter the step tag comes from (every step launch adds 256); may equal tsync
    int64_t peer_mbox_off[LQ4_MAX_PEERS];        // bytes from this GPU's mailbox to peer r's
    // at the end of the launch every mailbox entry of these ranges is copied to payload[slot] as plain f32:
    // when the launch completes, this GPU holds every rank's results
    float* payload;
    uint32_t range_begin[kStepMaxRanges], range_count[kStepMaxRanges];
    uint32_t n_ranges;
};

// Fills the shared-memory plan for limb buffers of `cap_blocks` Q4 blocks (the longest k range any CTA converts in
// any group), the widest adapter and the largest rank x pieces product of one problem; returns the dynamic shared
// memory needed, or 0 if it does not fit.
size_t step_plan_smem(StepArgs& a, uint32_t cap_blocks, uint32_t max_rank, uint32_t max_items);
cudaError_t launch_decode_step(const StepArgs& a, size_t smem, int grid, cudaStream_t s);

}  // namespace lq4
