/*
 * lattice_q4.h - C ABI of the B200 (sm_100a) backend for Lattice's Q4 weight-only
 * linear layer with the LoRA delta fused in and the optional QuaRot activation
 * rotation in the prologue.
 *
 * The reference (ohdearquant/lattice, Rust) has no FFI for this path: its Q4
 * matmul seam is a set of inherent methods on the Metal engine state.  Each
 * entry point below names the reference call site it stands in for (paths are
 * relative to the reference project root); a Rust `extern "C"` block binds
 * these one to one.
 *
 * Conventions
 *   - every function returns an lq4_status (0 = ok) and never aborts;
 *   - pointers are DEVICE pointers unless the parameter name starts with `h_`;
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it
 *     unless stated otherwise;
 *   - a context belongs to one device and one owning host thread (the reference
 *     keeps its GPU state on a single worker thread:
 *     crates/inference/src/serve/metal_worker.rs:1-34).  Calls that share a
 *     context must be ordered on one stream: its workspace is reused per call.
 *   - weights use the reference's on-disk block layout unchanged: row-major
 *     [n][k/32] blocks of 20 bytes {f16 scale, f16 bias, 16 bytes of nibbles,
 *     low nibble first}, w = nibble * scale + bias
 *     (crates/inference/src/weights/q4_weights.rs:3-45, 65-92).
 */
#ifndef LATTICE_Q4_H
#define LATTICE_Q4_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t lq4_status;

enum {
    LQ4_OK = 0,
    LQ4_ERR_NULL = 1,          /* a required pointer is NULL */
    LQ4_ERR_K = 2,             /* k == 0 or k % 32 != 0 (the reference panics here) */
    LQ4_ERR_OVERFLOW = 3,      /* m*k, n*k or m*n does not fit */
    LQ4_ERR_ALIGN = 4,         /* pointer alignment below the documented minimum */
    LQ4_ERR_DTYPE = 5,
    LQ4_ERR_LORA = 6,          /* rank == 0, non-finite scale, or NULL factor */
    LQ4_ERR_ROT = 7,           /* rotation dim != k or not a power of two */
    LQ4_ERR_BAD_BLOCK = 8,     /* a block's scale is not finite-positive or its bias not finite */
    LQ4_ERR_CUDA = 9,          /* a CUDA runtime call failed; see lq4_last_error() */
    LQ4_ERR_UNSUPPORTED = 10,  /* shape outside what this build handles */
    LQ4_ERR_DEVICE = 11,       /* a kernel reported a failed bounded wait */
    LQ4_ERR_FORMAT = 12,       /* malformed .q4 image */
    LQ4_ERR_IO = 13,
    LQ4_ERR_SHAPE = 14,        /* shape / length mismatch */
    LQ4_ERR_NOSPACE = 15       /* request exceeds a fixed capacity */
};

enum { LQ4_DTYPE_F32 = 0, LQ4_DTYPE_BF16 = 1, LQ4_DTYPE_F64 = 2 };   /* F64: converter-side calls only */
enum { LQ4_QUANT_ASYMMETRIC = 0, LQ4_QUANT_SYMMETRIC = 1 };

/* Which kernel family lq4_linear picks.  AUTO is the product path. */
enum {
    LQ4_PATH_AUTO = 0,
    LQ4_PATH_GEMV_MMA = 1,       /* m <= 16: TMA-staged stream-K decode kernel */
    LQ4_PATH_GEMV_GENERIC = 2,   /* any alignment, any k % 32 == 0; slow */
    LQ4_PATH_GEMM_TC = 3         /* m > 16: tcgen05 / TMEM tensor-core kernel */
};

typedef struct lq4_ctx lq4_ctx;
typedef struct lq4_weights lq4_weights;
typedef struct lq4_lora lq4_lora;

/* One LoRA projection: y += scale * B (A x).  A is [rank, k] row-major, B is
 * [n, rank] row-major, both f32 on the device
 * (crates/tune/src/lora/mod.rs:124-137, crates/tune/src/lora/apply.rs:48-93). */
typedef struct {
    const float* a;
    const float* b;
    uint32_t rank;
    float scale;
} lq4_lora_desc;

/* Online randomized Hadamard rotation x' = H (D x) applied to every activation
 * row before the matmul; `signs` holds k entries of +1/-1 (f32, device)
 * (crates/inference/src/quant/quarot/hadamard.rs:176-209).
 * dim == k: one rotation over the whole row (k a power of two).  dim < k: the block-diagonal
 * rotation BlockHadamard (hadamard.rs:285-484) with block size `dim` (a power of two that divides k,
 * k / dim <= 4096), the R4 rotation in front of down_proj on axes that are not powers of two
 * (3584 = 28 x 128, 17408 = 68 x 256); block i uses signs[i * dim, (i + 1) * dim). */
#define LQ4_MAX_ROT_LEN (1u << 24)   /* MAX_BLOCK_HADAMARD_LEN, hadamard.rs:318 */
#define LQ4_MAX_ROT_BLOCKS 4096u     /* MAX_BLOCK_HADAMARD_BLOCKS, hadamard.rs:345 */
typedef struct {
    const float* signs;
    uint32_t dim;
} lq4_rot_desc;

/* Column-parallel all-gather fused into the decode kernels' epilogue: every GPU of the group
 * computes its own rows of W (an N-shard) and writes the results straight into the output
 * buffer of EVERY GPU over NVLink, then signals each peer's arrival counter.  `bases[r]` is
 * rank r's peer buffer (lq4_peer_buf_*) as mapped in this process, bases[rank] this GPU's own;
 * all buffers have the same layout and `y` of the call must point into the own buffer's payload
 * (lq4_peer_buf_payload): the same byte offset is written in every peer.  No counterpart in the
 * reference (single GPU); the NCCL all-gather it replaces is the plain way to do the same. */
#define LQ4_MAX_PEERS 8
typedef struct {
    uint32_t world, rank;
    void* bases[LQ4_MAX_PEERS];
} lq4_gather_desc;

typedef struct {
    const void* x;        /* [m, k] row-major activations, f32 or bf16 */
    int32_t x_dtype;      /* LQ4_DTYPE_* */
    uint32_t m, n, k;
    const uint8_t* w;     /* Q4 payload for rows [0, n): the header is already skipped;
                             an N-shard or a row slice of a fused matrix is addressed by
                             adding n0 * (k/32) * 20 bytes.  4-byte aligned at least;
                             16-byte aligned with k % 128 == 0 for the fast kernels. */
    float* y;             /* [m, n] f32, OVERWRITTEN */
    uint64_t ldy;         /* elements between consecutive rows of y; 0 means n */
    const lq4_lora_desc* lora;   /* NULL = no adapter for this projection */
    const lq4_rot_desc* rot;     /* NULL = no online rotation */
    int32_t path;         /* LQ4_PATH_* */
    const lq4_gather_desc* gather;   /* NULL = results stay on this GPU; else the epilogue also stores every result
                                        into each peer's buffer: decode shapes (m <= 16) and the tensor-core kernel
                                        (m > 16, adapter rank <= 128); fast layout only */
    const lq4_gather_desc* wait_gather;   /* non-NULL: x holds gathered results (it lives in the own peer buffer):
                                             before x is read, wait (bounded) until every peer's results of all
                                             gathered launches this rank has issued so far have arrived; the
                                             same wait as lq4_gather_wait, without a launch of its own */
} lq4_linear_args;

/* ---- context ----------------------------------------------------------- */

/* Creates the per-device state (workspace, status word) on `device`.  Allocates. */
lq4_status lq4_ctx_create(int32_t device, lq4_ctx** out);
void lq4_ctx_destroy(lq4_ctx* ctx);
/* Grows the workspace so that a later lq4_linear of this shape allocates nothing. */
lq4_status lq4_ctx_reserve(lq4_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t rank);
/* Synchronises `stream` and returns LQ4_ERR_DEVICE if any kernel launched through
 * this context gave up on a bounded wait since the last call; clears the flag. */
lq4_status lq4_ctx_check(lq4_ctx* ctx, void* stream);
/* Per-context switches.  LQ4_OPT_MLP_ONE_LAUNCH (default 1): lq4_mlp_block runs a one-token block whose
 * gate||up row lives in the library's workspace as ONE lq4_decode_step launch instead of two launches (measured
 * on B200, hidden 5120 / inter 17408: 42.5 us against 47.0 us).  LQ4_OPT_PDL (default
 * 1): programmatic dependent launch between consecutive kernels.  LQ4_OPT_ALLOW_GROW (default 1): 0 makes a call
 * whose workspace is too small return LQ4_ERR_NOSPACE instead of reallocating (after lq4_ctx_reserve, for
 * callers that must not hit cudaMalloc in the decode loop). */
enum { LQ4_OPT_MLP_ONE_LAUNCH = 1, LQ4_OPT_PDL = 2, LQ4_OPT_ALLOW_GROW = 3 };
lq4_status lq4_ctx_set_option(lq4_ctx* ctx, int32_t option, int32_t value);
/* Number of kernels this library has launched through `ctx` so far. */
uint64_t lq4_ctx_launch_count(const lq4_ctx* ctx);
const char* lq4_last_error(void);
const char* lq4_status_string(lq4_status s);
int32_t lq4_abi_version(void);

/* ---- the hot path ------------------------------------------------------- */

/* y = x Wq4^T (+ LoRA) with the optional rotation of x first.
 * Replaces dispatch_gemm_q4 / dispatch_gemm_q4_at / dispatch_matmul_q4
 * (crates/inference/src/forward/metal_qwen35/inner/dispatch.rs:148-229, 1037-1097)
 * with dispatch_lora_if_active (.../inner/layers/mod.rs:15-51) folded into the same
 * launch.  m == 0 or n == 0 is a no-op; k == 0 or k % 32 != 0 returns LQ4_ERR_K. */
lq4_status lq4_linear(lq4_ctx* ctx, const lq4_linear_args* args, void* stream);

/* Several independent decode projections in ONE persistent launch.  `args[0..count)` are
 * complete lq4_linear problems; none may read what another one writes.  When every problem has
 * the same m <= 16, no rotation, k % 128 == 0, 16-byte aligned w and x, LoRA rank <= 512, and
 * count <= 8, the work of all problems is split evenly over the SMs as one range (launch,
 * activation prologue and tail are paid once, not once per projection).  Any other group is served
 * problem by problem through lq4_linear, with identical results - except 9 to 24 one-token projections that
 * qualify for lq4_decode_step (below), which run as one group of that kernel, again ONE launch (sixteen
 * large-layer projections: 93 us against 116 us as four groups of four).  Replaces the reference's habit of encoding a decode
 * step's projections back to back into one Metal command buffer
 * (crates/inference/src/forward/metal_qwen35.rs:4458-4462, one encoder for all layers) and its
 * merged-row GEMVs with per-range adapters (inner/layers/gdn.rs:69-105,293-300: one GEMV over
 * qkv||z rows, then LoRA into sub-ranges): q/k/v, or gate/up, share x and go in one group.
 * The adapters are projected inside the same launch by its producer warps (no launch of their own); the
 * one-launch form takes m <= 16.  count == 1 is allowed: the single projection then runs on the grouped
 * kernel (a group of one).  A decode step that interleaves grouped launches with single projections
 * (o_proj, down_proj) should issue those this way: two different kernels in turn start every launch with
 * a cold instruction cache (about 2.5 us per switch on B200), one kernel for both does not. */
lq4_status lq4_linear_group(lq4_ctx* ctx, const lq4_linear_args* args, uint32_t count, void* stream);

typedef struct lq4_peer_buf lq4_peer_buf;

/* ---- a whole decode step in one launch -------------------------------------------------------- */

/* A step buffer holds the activations that travel between the groups of a step (and between the GPUs of
 * an N-sharded step): `payload_floats` f32 values followed by the library's mailbox for them.  It is a peer
 * buffer (lq4_peer_buf_export / _open / _close / _base / _payload / _free apply): with several GPUs every
 * rank creates one of the same size and maps the others'.  Allocates (cudaMalloc), zero-filled. */
lq4_status lq4_step_buf_create(uint64_t payload_floats, lq4_peer_buf** out);

typedef struct {
    const lq4_linear_args* args;   /* independent one-token projections, as for lq4_linear_group */
    uint32_t count;
} lq4_step_group;

typedef struct {
    const float* start;            /* inside this rank's step-buffer payload */
    uint64_t count;                /* floats */
} lq4_step_range;

typedef struct {
    const lq4_gather_desc* bufs;   /* the ranks' step buffers: bases[rank] this GPU's own (world 1: just that one) */
    const lq4_step_range* gathered;   /* ranges of the payload that are complete, as plain f32, on THIS GPU when
                                         the launch completes: the full rows (all ranks' columns) of the outputs
                                         the caller reads afterwards.  With world > 1 every output must be covered. */
    uint32_t n_gathered;
} lq4_step_desc;

/* Runs groups[0], groups[1], ... in ONE persistent launch.  The projections of a group are independent;
 * a projection of a later group may take its activations from what earlier groups of the same call wrote:
 * its x then points into the step buffer's payload at the place where those outputs' y pointed (for an
 * N-sharded step: at the full row that the ranks' column slices form together).  Such an input is read
 * through the mailbox as the values arrive - from this GPU's CTAs or, over NVLink, from the peers' - so
 * the weight stream of the next group never stops for a launch boundary, a fence or a collective.  When
 * the launch completes on a rank, every `gathered` range is complete there as plain f32.  Replaces the
 * reference's one command buffer per decode step (crates/inference/src/forward/metal_qwen35.rs:4458-4462:
 * all of a step's dispatches are encoded back to back and committed once), whose dispatches are ordered
 * by the encoder; here the order is carried by the data.
 * Every problem: m == 1, no rotation, k % 128 == 0, 16-byte aligned w and x, LoRA rank <= 512, the row
 * fits in shared memory (k <= about 50k), fused-gather fields NULL; at most 24 problems in 8 groups;
 * inputs taken from the step buffer are f32.  Outputs outside the step buffer are written as usual but
 * cannot feed later groups.  `step` may be NULL when no group depends on another and there is one GPU.
 * All ranks of an N-sharded step must issue the same sequence of lq4_decode_step calls on their buffers.
 * Every wait is bounded (about two seconds, then LQ4_ERR_DEVICE through lq4_ctx_check). */
lq4_status lq4_decode_step(lq4_ctx* ctx, const lq4_step_group* groups, uint32_t ngroups, const lq4_step_desc* step,
                           void* stream);

/* lq4_decode_step with HOST activations and outputs, the step-level counterpart of lq4_linear_host.  Every
 * input that does not lie in the step buffer's payload is first copied into the library's workspace by a
 * small stage-in kernel chained in front of the step kernel (programmatic launch: the step kernel's weight
 * stream starts while the copy runs), so it may live in page-locked host memory that the device can address
 * (cudaHostAlloc / cudaHostRegister under unified addressing; a device pointer works too).  Outputs are
 * stored where y points by the step kernel itself, so they may live in such host memory as well: the
 * results of an early group cross PCIe while the later groups compute, and no copy engine is involved in
 * either direction (measured on B200: a copy node in front of and behind the kernel costs 14 us and 10 us of
 * a 136 us step).  The host must not touch the inputs before the launch has completed, and reads the
 * outputs after it has.  With world > 1 the outputs must lie in the step buffer as for lq4_decode_step.
 * Pointers the device cannot address (pageable host memory) are refused with LQ4_ERR_UNSUPPORTED.
 * The staging area grows on first use (which synchronises the stream and allocates): make one plain call
 * before capturing this call into a CUDA graph.
 * No counterpart in the reference, whose buffers are zero-copy unified memory
 * (crates/inference/src/forward/metal.rs:4, StorageModeShared). */
lq4_status lq4_decode_step_host(lq4_ctx* ctx, const lq4_step_group* groups, uint32_t ngroups, const lq4_step_desc* step,
                                void* stream);

/* ---- peer buffers for the fused all-gather ------------------------------------ */
#define LQ4_PEER_HANDLE_BYTES 64
/* Allocates (cudaMalloc, zero-filled) a buffer other processes on the same node can map:
 * 256 control bytes (arrival counter, launch sequence, CTA counter) followed by `payload_bytes` of output. */
lq4_status lq4_peer_buf_create(uint64_t payload_bytes, lq4_peer_buf** out);
void lq4_peer_buf_free(lq4_peer_buf* b);
/* The buffer's base (what goes into lq4_gather_desc::bases for the owner) and its payload. */
void* lq4_peer_buf_base(const lq4_peer_buf* b);
void* lq4_peer_buf_payload(const lq4_peer_buf* b);
/* 64 opaque bytes to hand to the other ranks (any transport), and the call that maps a peer's
 * buffer from them; the returned base goes into lq4_gather_desc::bases[peer]. */
lq4_status lq4_peer_buf_export(const lq4_peer_buf* b, uint8_t* handle_out);
lq4_status lq4_peer_buf_open(const uint8_t* handle, void** base_out);
lq4_status lq4_peer_buf_close(void* base);
/* Stream-ordered wait (bounded: about two seconds, then LQ4_ERR_DEVICE through lq4_ctx_check) until
 * every peer's results of all gathered launches issued so far on this rank have arrived here.
 * Ranks must issue the same sequence of gathered launches.  A buffer may be overwritten by the
 * peers' NEXT gathered launch as soon as they get there: alternate two buffers, or synchronise the
 * ranks, before reading results late. */
lq4_status lq4_gather_wait(lq4_ctx* ctx, const lq4_gather_desc* gather, void* stream);

/* Decode projection (m <= 4) for callers that cannot allocate device memory: an engine that
 * handed every byte to its own pool at start-up, or a decode loop that cannot afford the
 * device-wide synchronisation inside cudaMalloc/cudaFree.  No counterpart in the reference:
 * this entry point exists only in this library.  It takes no context; the kernel's scratch
 * (stream-K partial-sum messages, the launch counter, the LoRA projection messages) lives in a fixed 1 MB
 * array inside the loaded module, held by every GPU that loads the library until exit.
 * Limits, rejected with LQ4_ERR_NOSPACE: m <= 4, n <= 32768, LoRA rank <= 64, and m * k small
 * enough for the activation rows to sit in shared memory (m * k <= 56000); k % 128 == 0
 * and 16-byte aligned w and x are required (LQ4_ERR_ALIGN).  It calls no cudaMalloc, cudaFree
 * or other allocating routine.  The first call on a device resolves the array's address; make
 * that call before any stream capture.  All calls on a device share the array, which keeps the
 * last call's contents (messages in it carry a per-launch tag, so nothing stale is reused): calls that
 * overlap on the GPU race, so order them on one stream.  `args->path` is ignored. */
lq4_status lq4_linear_decode_noalloc(const lq4_linear_args* args, void* stream);
/* The status word of lq4_linear_decode_noalloc lives in the same built-in array (that entry point has no
 * context to ask).  Drains `stream`, reads the word of the current device with a 4-byte copy (no
 * allocation), clears it, and returns LQ4_ERR_DEVICE if a kernel launched through the entry point gave up
 * on a bounded wait since the last check.  No counterpart in the reference. */
lq4_status lq4_noalloc_check(void* stream);

/* Same call with HOST activations and HOST output: copies x to the device,
 * runs lq4_linear, copies y back and waits for it.  Weights and LoRA factors
 * stay device resident, as the reference keeps them in GPU-visible buffers for
 * the model's lifetime (crates/inference/src/forward/metal_qwen35.rs:599-702). */
lq4_status lq4_linear_host(lq4_ctx* ctx, const lq4_linear_args* args_with_host_x_y, void* stream);

/* ---- dense MLP block: gate||up -> silu(gate) * up -> down -------------------------------- */

/* The FFN half of encode_mlp_block for dense layers
 * (crates/inference/src/forward/metal_qwen35/inner/layers/mod.rs:93-148): one matmul over the merged
 * gate_up_proj rows (N = 2 * inter) with the gate_proj / up_proj adapters on the two halves of its output,
 * silu_mul_fused (shaders/qwen35.metal:712-722), then down_proj with its adapter. */
typedef struct {
    const void* x;                 /* [m, hidden] activations (the normed hidden state) */
    int32_t x_dtype;
    uint32_t m, hidden, inter;
    const uint8_t* w_gate_up;      /* Q4 rows [2 * inter, hidden]: gate rows, then up rows (the merged file of
                                      q4_weights.rs:1362-1639) */
    const uint8_t* w_down;         /* Q4 rows [hidden, inter] */
    const lq4_lora_desc* lora_gate;   /* each may be NULL */
    const lq4_lora_desc* lora_up;
    const lq4_lora_desc* lora_down;
    float* gate_up;                /* [m, 2 * inter] f32 scratch (activations.gate), OVERWRITTEN, contents
                                      unspecified afterwards; NULL = the context's workspace */
    float* y;                      /* [m, hidden] f32, OVERWRITTEN (activations.ffn_out) */
    const lq4_rot_desc* rot_down;  /* NULL, or the online rotation of silu(gate) * up in front of down_proj
                                      (R4: block-diagonal, dim = block size; OnlineRotationSpec::r4_dense_mlp,
                                      quant/quarot/plan.rs); the gated vector is then formed by a pass of its
                                      own and rotated before the projection reads it */
} lq4_mlp_args;

/* Two launches for one token: gate and up rows as one grouped launch, then down_proj, whose kernel applies
 * silu(gate) * up to its own input while it stages the activations (no separate gating pass, no round
 * trip of the gated vector through memory); likewise up to 16 tokens (the record builder of the dense decode
 * kernel gates).  More tokens: the same three steps with a gating pass.
 * hidden and inter divisible by 32 (LQ4_ERR_K otherwise). */
lq4_status lq4_mlp_block(lq4_ctx* ctx, const lq4_mlp_args* args, void* stream);

/* ---- lm_head: vocabulary projection + exact top-k ----------------------------------------- */

#define LQ4_MAX_TOP_K 256u       /* MAX_TOP_K of the reference's selection kernels (shaders/qwen35.metal:1686) */

/* One selected token: TopKCandidate (crates/inference/src/forward/shaders/qwen35.metal:1688-1695).
 * Unused tail entries (top_k > number of non-NaN logits) hold the sentinel (-inf, UINT32_MAX). */
typedef struct {
    float logit;
    uint32_t token_id;
} lq4_topk_candidate;

/* out[0 .. top_k) = the top_k entries of logits[0 .. n) in the order of topk_better
 * (shaders/qwen35.metal:1697-1703): higher logit first, ties to the lower token id; NaN logits never rank.
 * Replaces logits_topk first pass + logits_topk_merge_pass (shaders/qwen35.metal:1730-1770); exact for any
 * distribution.  logits and out are device pointers.  top_k outside 1..LQ4_MAX_TOP_K: LQ4_ERR_SHAPE. */
lq4_status lq4_logits_topk(lq4_ctx* ctx, const float* logits, uint32_t n, uint32_t top_k,
                           lq4_topk_candidate* out, void* stream);

/* The reference's two-stage lm_head path, lm_head_block_topk_q4 + merge (shaders/qwen35.metal:1931-1979,
 * dispatched from forward/metal_qwen35/inner/dispatch.rs:1346-1436): logits = lq4_linear(args) for one
 * token (args->m must be 1, else LQ4_ERR_SHAPE), then lq4_logits_topk over the n = vocabulary rows.
 * args->y may be NULL: the logit row then lives only in the context's workspace (the sampler never sees
 * it, as in the reference); non-NULL y receives the full row as well.  The fused all-gather fields must
 * be NULL (LQ4_ERR_UNSUPPORTED). */
lq4_status lq4_lm_head_topk(lq4_ctx* ctx, const lq4_linear_args* args, uint32_t top_k,
                            lq4_topk_candidate* out, void* stream);

/* Standalone y[m, d_out] += scale * B (A x): the two-dispatch form of
 * dispatch_lora_if_active, for fused outputs where two adapters write two
 * column ranges of one y (gate||up, qkv||z). */
lq4_status lq4_lora_apply(lq4_ctx* ctx, const void* x, int32_t x_dtype, uint32_t m, uint32_t k,
                          float* y, uint32_t n, uint64_t ldy, const lq4_lora_desc* lora, void* stream);

/* Dequantizes n_blocks blocks to 32 * n_blocks floats, bit-identical to
 * dequantize_q4_to_f32 (crates/inference/src/weights/q4_weights.rs:558-571). */
lq4_status lq4_dequant_f32(const uint8_t* payload, uint64_t n_blocks, float* out, void* stream);

/* Quantizes `len` f32 values in flat 32-element chunks (last one zero padded),
 * bit-identical to quantize_f32_to_q4 (asymmetric) and to quantize_f64_to_q4 on
 * f32-representable input (symmetric)
 * (crates/inference/src/weights/q4_weights.rs:239-295, 470-487, 514-553).
 * `status_out` (device int32, may be NULL) receives LQ4_ERR_BAD_BLOCK if a block
 * had a non-finite input or unrepresentable metadata. */
lq4_status lq4_quantize_f32(const float* data, uint64_t len, int32_t mode, uint8_t* payload,
                            int32_t* status_out, void* stream);

/* The other quantizer entry points of the reference, on the device.  `data` holds rows * cols values
 * of `dtype`:
 *   F32,  per_row = 0  quantize_f32_to_q4 (flat 32-value chunks across row ends; q4_weights.rs:470-487)
 *   F32,  per_row = 1  quantize_tensor_q4_0 / quantize_row_q4_0 (every row ends in its own zero-padded
 *                      block when cols % 32 != 0; q4_weights.rs:312-328, 364-388)
 *   BF16, per_row = 0  quantize_bf16_to_q4 / stream_quantize_shard (widened exactly; :428-447, 580-606)
 *   F64,  per_row = 0  quantize_f64_to_q4_mode: every value is narrowed to f32 first, as `v as f32`
 *                      does (:514-553); mode SYMMETRIC is quantize_f64_to_q4, the QuaRot quantizer
 * `payload` receives rows * ceil(cols / 32) blocks (per_row) or ceil(rows * cols / 32) blocks (flat);
 * bit-identical to the reference.  Non-finite input (also an f64 beyond the f32 range) or metadata
 * that f16 cannot hold sets *status_out to LQ4_ERR_BAD_BLOCK, like the reference's InvalidInput. */
lq4_status lq4_quantize_tensor(const void* data, int32_t dtype, uint64_t rows, uint64_t cols, int32_t per_row,
                               int32_t mode, uint8_t* payload, int32_t* status_out, void* stream);

/* Rotation absorption of the offline QuaRot conversion, in place on a row-major [rows, cols] matrix of
 * f32 or f64 (`dtype`) on the device, bit-identical to the reference's loops:
 *   lq4_absorb_input_rotation   W <- W R^T, R applied to every row; rot->dim must equal cols
 *     (absorb_input_rotation / absorb_input_rotation_f64,
 *      crates/inference/src/quant/quarot/rotation.rs:86-107, 146-166)
 *   lq4_absorb_output_rotation  W <- R W, R applied to every column; rot->dim must equal rows
 *     (absorb_output_rotation / absorb_output_rotation_f64, rotation.rs:115-142, 169-195)
 * These are what absorb_rotations (quant/quarot/pipeline.rs:202-235) calls per planned tensor with the
 * f64 forms.  A dimension mismatch or a dim that is not a power of two returns LQ4_ERR_ROT (the
 * reference's Err).  Row rotation: dim <= 16384 (f64) / 32768 (f32), the row is staged in shared memory. */
lq4_status lq4_absorb_input_rotation(void* w, int32_t dtype, uint64_t rows, uint64_t cols,
                                     const lq4_rot_desc* rot, void* stream);
lq4_status lq4_absorb_output_rotation(void* w, int32_t dtype, uint64_t rows, uint64_t cols,
                                      const lq4_rot_desc* rot, void* stream);

/* Writes a `.q4` file exactly as save_q4_file does (crates/inference/src/weights/q4_weights.rs:623-645):
 * "KHQ4", u32 version 2, u32 ndim, u64 shape[ndim], u64 original_len, then ceil(original_len / 32)
 * blocks read from the DEVICE pointer `payload` (copied to the host on `stream`, which is drained).
 * The product of `h_shape` must equal original_len (what the reference's constructors guarantee);
 * ndim 1..8.  A file written here loads through lq4_weights_load_q4_file when it is 2-D. */
lq4_status lq4_q4_file_write(const char* h_path, const uint64_t* h_shape, uint32_t ndim, uint64_t original_len,
                             const uint8_t* payload, void* stream);

/* Applies x' = H (D x) to `rows` rows of length `dim` (a power of two <= 16384),
 * f32 in and out, bit-identical to RandomizedHadamard::apply
 * (crates/inference/src/quant/quarot/hadamard.rs:197-209). */
lq4_status lq4_hadamard_rows(const float* x, float* out, uint32_t rows, const lq4_rot_desc* rot, void* stream);

/* BlockHadamard::apply (hadamard.rs:444-462) on `rows` vectors of length n: block size rot->dim, signs
 * of n entries; bit-identical to the reference.  The constructor's refusals (n == 0, n > 1 << 24, block
 * not a power of two or not dividing n, more than 4096 blocks) return LQ4_ERR_ROT. */
lq4_status lq4_block_hadamard_rows(const float* x, float* out, uint32_t rows, uint32_t n,
                                   const lq4_rot_desc* rot, void* stream);

/* QuaRot's online "Hadamard heads" rotation H_num_heads (x) I_head_dim on `rows` activations of
 * num_heads * head_dim entries each: for every within-head channel the num_heads values across the heads
 * are rotated by one RandomizedHadamard of dimension num_heads (`signs`: num_heads entries, device), the
 * R3 rotation of the gated attention output in front of o_proj
 * (apply_cross_head_rotation, crates/inference/src/quant/quarot/r3_reference.rs:246-264;
 * OnlineRotationSpec::r3_full_attention, quant/quarot/plan.rs).  Bit-identical to that loop.  num_heads a
 * power of two <= 128, else LQ4_ERR_ROT.  x and out must not overlap. */
lq4_status lq4_cross_head_hadamard_rows(const float* x, float* out, uint32_t rows, uint32_t num_heads,
                                        uint32_t head_dim, const float* signs, void* stream);

/* Fills `signs` (n entries) as BlockHadamard::new(seed, n, block) does: block i draws
 * signs_from_seed(derive_block_seed(seed, i), block) (hadamard.rs:153-155, 401-414). */
lq4_status lq4_block_rot_signs_from_seed(uint64_t seed, uint32_t n, uint32_t block, float* signs, void* stream);

/* Fills `signs` with the +1/-1 diagonal of RandomizedHadamard::new(seed, dim)
 * (crates/inference/src/quant/quarot/hadamard.rs:114-139). */
lq4_status lq4_rot_signs_from_seed(uint64_t seed, uint32_t dim, float* signs, void* stream);

/* ---- resident objects ---------------------------------------------------- */

/* Validates every block (scale finite and > 0, bias finite) on the host and only
 * then copies the payload into a 256-byte aligned device allocation: the
 * counterpart of mmap_q4_weight (crates/inference/src/forward/metal_qwen35.rs:660-702;
 * rule: crates/inference/src/weights/ingress.rs:542-560).  Synchronous. */
lq4_status lq4_weights_upload(const uint8_t* h_payload, uint64_t n, uint64_t k, lq4_weights** out);
/* Loads a `.q4` file ("KHQ4", version 2): header, exact extent, optional
 * expected shape (pass ndim 0 to skip), block validity
 * (crates/inference/src/weights/q4_weights.rs:709-868). */
lq4_status lq4_weights_load_q4_file(const char* h_path, const uint64_t* h_expected_shape,
                                    uint32_t expected_ndim, lq4_weights** out);
const uint8_t* lq4_weights_payload(const lq4_weights* w);
uint64_t lq4_weights_rows(const lq4_weights* w);
uint64_t lq4_weights_cols(const lq4_weights* w);
void lq4_weights_free(lq4_weights* w);

/* Copies host LoRA factors to the device after the checks load_lora_adapter makes
 * per projection: rank > 0, d_in > 0, d_out > 0, finite scale, A and B element
 * counts equal rank*d_in and d_out*rank, sizes fit u32
 * (crates/inference/src/forward/metal_qwen35.rs:3806-3986).  Synchronous. */
lq4_status lq4_lora_upload(const float* h_a, uint64_t a_len, const float* h_b, uint64_t b_len,
                           uint64_t rank, uint64_t d_in, uint64_t d_out, float scale, lq4_lora** out);
/* Fills `desc` with the device pointers of rows [n0, n1) of B (all of A). */
lq4_status lq4_lora_desc_for_rows(const lq4_lora* l, uint64_t n0, uint64_t n1, lq4_lora_desc* desc);
void lq4_lora_free(lq4_lora* l);

/* ---- N-sharding ----------------------------------------------------------- */

/* Column-parallel split of the n output rows over `world` ranks: rank r owns rows
 * [n0, n1) = [r*n/world, (r+1)*n/world) and its payload starts `byte_offset` bytes
 * into the full payload - the qw_extra_offset addressing of dispatch_gemm_q4_at. */
lq4_status lq4_shard_plan(uint64_t n, uint64_t k, uint32_t world, uint32_t rank,
                          uint64_t* n0, uint64_t* n1, uint64_t* byte_offset);

/* ---- N-sharded linear with the slices gathered over NCCL ------------------------------------ */

/* The communicator is the caller's: a Rust host passes the ncclComm_t of its own NCCL binding.  The three
 * calls below wrap ncclGetUniqueId / ncclCommInitRank / ncclCommDestroy for hosts without one: rank 0
 * draws an id, hands its 128 bytes to the other ranks by any transport, and every rank (its GPU current)
 * creates the communicator.  The library binds NCCL at run time (the libnccl.so.2 already loaded in the
 * process, else the system's); without one these calls return LQ4_ERR_UNSUPPORTED.  No counterpart in
 * the reference (single GPU). */
#define LQ4_NCCL_ID_BYTES 128
lq4_status lq4_nccl_unique_id(uint8_t* h_id_out);
lq4_status lq4_nccl_comm_create(const uint8_t* h_id, uint32_t world, uint32_t rank, void** comm_out);
void lq4_nccl_comm_destroy(void* comm);

typedef struct {
    void* nccl_comm;      /* ncclComm_t, one rank per GPU */
    uint32_t world, rank;
    uint64_t n_total;     /* rows of the whole weight = columns of the gathered output */
    float* y_full;        /* [m, ldy_full] f32 on this GPU, OVERWRITTEN with every rank's columns */
    uint64_t ldy_full;    /* elements between rows of y_full; 0 means n_total */
} lq4_shard_desc;

/* Column-parallel linear: `local` describes THIS rank's rows of the weight exactly as a plain lq4_linear
 * call would (w = payload + lq4_shard_plan's byte offset, n = n1 - n0, the same rows of LoRA B; its y and
 * the fused-gather fields are ignored), the library computes the slice and all-gathers the [m, n / world]
 * slices of all ranks into y_full[:, n0_r : n1_r] with ncclAllGather (equal slices) or grouped
 * ncclBroadcast (unequal), on a second stream, tile-row block by block so that the exchange of one block
 * overlaps the product of the next; a placement pass moves each block from NCCL's rank-major order into
 * the row-major y_full.  On return the work is ordered on `stream`.  Every rank must make the same call.
 * Not capturable in a CUDA graph (NCCL collectives on an internal stream).  The addressing is the
 * qw_extra_offset row-slice addressing of dispatch_gemm_q4_at
 * (crates/inference/src/forward/metal_qwen35/inner/dispatch.rs:1037-1097); the reference itself runs on
 * one GPU. */
lq4_status lq4_linear_sharded(lq4_ctx* ctx, const lq4_linear_args* local, const lq4_shard_desc* shard, void* stream);

/* The placement pass of lq4_linear_sharded on its own, for hosts that run the collective themselves:
 * `gathered` holds what an all-gather of the [rows, n_r] slices delivers, rank after rank
 * ([world][rows][n_r], n_r = the rows of lq4_shard_plan(n_total, world, r)); they are moved to the
 * row-major y_full[rows, ldy_full] (0 = n_total), slice r to columns [n0_r, n1_r).  No counterpart in the
 * reference. */
lq4_status lq4_place_slices(const float* gathered, float* y_full, uint64_t ldy_full, uint32_t rows, uint64_t n_total,
                            uint32_t world, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LATTICE_Q4_H */
