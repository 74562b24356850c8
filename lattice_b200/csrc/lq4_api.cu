// C ABI: argument validation, workspace management and kernel selection.
// Validation happens before any launch and mirrors the reference's call-site
// contract: m == 0 or n == 0 is a no-op, k must be a non-zero multiple of 32
// (crates/inference/src/forward/metal_qwen35/inner/dispatch.rs:181-188), element
// counts are overflow-checked first (crates/inference/src/forward/cpu/gemm_validate.rs:1-60).
#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include <map>

#include "lq4_gemm.cuh"
#include "lq4_kernels.cuh"
#include "lq4_step.cuh"
#include "lq4_decode_common.cuh"

using namespace lq4;

namespace {

thread_local std::string g_last_error;

lq4_status fail(lq4_status s, const std::string& msg) {
    g_last_error = msg;
    return s;
}
lq4_status cuda_fail(cudaError_t e, const char* what) {
    return fail(LQ4_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
#define LQ4_CUDA(call)                                        \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
    } while (0)

struct Buf {
    void* p = nullptr;
    size_t cap = 0;
};

}  // namespace

namespace lq4 {
void set_last_error(const char* msg) { g_last_error = msg ? msg : ""; }
}  // namespace lq4

struct lq4_ctx {
    int device = 0;
    int sm_count = 0;
    uint64_t launches = 0;
    int32_t* status = nullptr;    // device status word
    uint32_t* tsync = nullptr;    // 64-bit launch counter of the decode kernels
    Buf xrot, xs, t, tmsg, partials, hx, hy, gemm, logits, topk, topk_ctr, mlp, mlp_h;   // xs: activation limb records of the dense decode kernel
    lq4_peer_buf* mlp_step = nullptr;   // step buffer of lq4_mlp_block's one-launch form (gate||up row + mailbox)
    Buf shard_send, shard_recv;   // staging of lq4_linear_sharded: local slices, NCCL's rank-major blocks
    cudaStream_t comm_stream = nullptr;      // second stream of lq4_linear_sharded (created on first use)
    cudaEvent_t ev_block[4] = {nullptr, nullptr, nullptr, nullptr}, ev_comm = nullptr;
    bool allow_grow = true;
    int pdl = 1;
    int mlp_one_launch = 1;       // LQ4_OPT_MLP_ONE_LAUNCH
    uint64_t alloc_gen = 0;       // bumped whenever a workspace buffer is reallocated (plans hold workspace pointers)
    struct StepPlan* step_plan = nullptr;      // the last lq4_decode_step call's argument block, reused when the call repeats
};

struct lq4_weights {
    uint8_t* payload = nullptr;
    uint64_t rows = 0, cols = 0;
    int device = 0;
};

struct lq4_lora {
    float* a = nullptr;
    float* b = nullptr;
    uint64_t rank = 0, d_in = 0, d_out = 0;
    float scale = 0.0f;
};

namespace {

// Grows `b` to at least `bytes`.  Growing frees the old allocation, so the stream
// that may still use it is drained first.
lq4_status ensure(lq4_ctx* ctx, Buf& b, size_t bytes, bool zero, cudaStream_t s) {
    if (bytes <= b.cap) return LQ4_OK;
    if (!ctx->allow_grow) return fail(LQ4_ERR_NOSPACE, "workspace too small and growth is disabled");
    LQ4_CUDA(cudaStreamSynchronize(s));
    if (b.p) LQ4_CUDA(cudaFree(b.p));
    b.p = nullptr;
    b.cap = 0;
    size_t cap = (bytes + 255) / 256 * 256;
    LQ4_CUDA(cudaMalloc(&b.p, cap));
    if (zero) LQ4_CUDA(cudaMemsetAsync(b.p, 0, cap, s));      // on the caller's stream: ordered before the first launch that reads it
    b.cap = cap;
    ++ctx->alloc_gen;
    return LQ4_OK;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline bool is_pow2(uint64_t v) { return v && !(v & (v - 1)); }

bool mul_overflows(uint64_t a, uint64_t b, uint64_t limit) { return a != 0 && b > limit / a; }

lq4_status validate_linear(const lq4_linear_args* a) {
    if (!a) return fail(LQ4_ERR_NULL, "args is NULL");
    if (a->m == 0 || a->n == 0) return LQ4_OK;
    if (a->k == 0 || a->k % 32 != 0)
        return fail(LQ4_ERR_K, "k must be non-zero and divisible by 32, got " + std::to_string(a->k));
    const uint64_t lim = (uint64_t)1 << 40;
    if (mul_overflows(a->m, a->k, lim) || mul_overflows(a->n, a->k, lim) || mul_overflows(a->m, a->n, lim))
        return fail(LQ4_ERR_OVERFLOW, "m*k, n*k or m*n exceeds the supported element count");
    if (!a->x || !a->w || !a->y) return fail(LQ4_ERR_NULL, "x, w and y must be non-NULL");
    if (a->x_dtype != LQ4_DTYPE_F32 && a->x_dtype != LQ4_DTYPE_BF16) return fail(LQ4_ERR_DTYPE, "unknown x_dtype");
    if (!aligned(a->w, 4) || !aligned(a->y, 4) || !aligned(a->x, a->x_dtype == LQ4_DTYPE_F32 ? 4 : 2))
        return fail(LQ4_ERR_ALIGN, "w and y need 4-byte alignment, x its element alignment");
    if (a->ldy != 0 && a->ldy < a->n) return fail(LQ4_ERR_SHAPE, "ldy is smaller than n");
    if (a->lora) {
        const lq4_lora_desc* l = a->lora;
        if (!l->a || !l->b) return fail(LQ4_ERR_LORA, "LoRA factor pointer is NULL");
        if (l->rank == 0) return fail(LQ4_ERR_LORA, "LoRA rank is 0");
        if (!std::isfinite(l->scale)) return fail(LQ4_ERR_LORA, "LoRA scale must be finite");
        if (!aligned(l->a, 4) || !aligned(l->b, 4)) return fail(LQ4_ERR_ALIGN, "LoRA factors need 4-byte alignment");
    }
    if (a->rot) {
        if (!a->rot->signs) return fail(LQ4_ERR_ROT, "rotation signs pointer is NULL");
        // dim == k: one randomized Hadamard over the row; dim < k: block-diagonal (one per `dim` entries)
        const uint32_t dim = a->rot->dim;
        if (!is_pow2(dim) || dim > 16384) return fail(LQ4_ERR_ROT, "rotation needs a power-of-two dim <= 16384");
        if (dim > a->k || a->k % dim != 0) return fail(LQ4_ERR_ROT, "rotation dim must equal k or divide it");
        if (a->k / dim > LQ4_MAX_ROT_BLOCKS) return fail(LQ4_ERR_ROT, "more than 4096 rotation blocks");
    }
    if (a->path < LQ4_PATH_AUTO || a->path > LQ4_PATH_GEMM_TC) return fail(LQ4_ERR_UNSUPPORTED, "unknown path");
    if (a->wait_gather) {
        const lq4_gather_desc* g = a->wait_gather;
        if (g->world < 1 || g->world > LQ4_MAX_PEERS || g->rank >= g->world || !g->bases[g->rank])
            return fail(LQ4_ERR_SHAPE, "wait_gather: world must be 1..8, rank < world, own base non-NULL");
    }
    if (a->gather) {
        const lq4_gather_desc* g = a->gather;
        if (g->world < 1 || g->world > LQ4_MAX_PEERS || g->rank >= g->world)
            return fail(LQ4_ERR_SHAPE, "gather: world must be 1..8 and rank < world");
        for (uint32_t r = 0; r < g->world; ++r)
            if (!g->bases[r] || !aligned(g->bases[r], 256)) return fail(LQ4_ERR_NULL, "gather: a peer buffer base is NULL or misaligned");
        if (reinterpret_cast<const char*>(a->y) < static_cast<const char*>(g->bases[g->rank]) + 256)
            return fail(LQ4_ERR_SHAPE, "gather: y must point into the payload of this rank's own peer buffer");
    }
    return LQ4_OK;
}

void fill_params(lq4_ctx* ctx, const lq4_linear_args* a, const void* x, int x_dtype, uint32_t m, float* y,
                 uint64_t ldy, GemvParams& p) {
    p = GemvParams{};
    p.w = a->w; p.y = y; p.ldy = ldy;
    p.m = m; p.n = a->n; p.k = a->k;
    p.kb = a->k / 32; p.kg = p.kb / kGemvGranuleBlocks;
    p.tiles = (a->n + kGemvTileRows - 1) / kGemvTileRows;
    p.status = ctx->status;
    p.tsync = ctx->tsync;          // 64-bit launch counter the message tags come from
    p.use_pdl = ctx->pdl;
    p.sm_count = ctx->sm_count;
    p.x = x; p.x_dtype = x_dtype;
    if (a->gather && a->gather->world > 1) {
        const lq4_gather_desc* g = a->gather;
        p.world = g->world;
        p.grank = g->rank;
        for (uint32_t r = 0; r < g->world; ++r) {
            p.peer_off[r] = static_cast<const char*>(g->bases[r]) - static_cast<const char*>(g->bases[g->rank]);
            p.peer_arrive[r] = static_cast<unsigned long long*>(g->bases[r]);
        }
        p.gseq = static_cast<unsigned long long*>(g->bases[g->rank]) + 1;
    }
    if (a->wait_gather && a->wait_gather->world > 1) {
        p.wait_arrive = static_cast<const unsigned long long*>(a->wait_gather->bases[a->wait_gather->rank]);
        p.wait_world = a->wait_gather->world;
    }
    p.tsplit = 1;
    if (a->lora) {
        p.la = a->lora->a; p.lb = a->lora->b; p.rank = a->lora->rank; p.lscale = a->lora->scale;
        p.tsplit = decode_tsplit(a->k);
    }
}

// The dense decode kernel over 1..kMaxGroup problems of the same token count (<= 16): one
// preparation launch (activation limbs, adapter projections), one persistent launch.
lq4_status run_dense(lq4_ctx* ctx, GemvParams* ps, uint32_t count, cudaStream_t s) {
    const uint32_t m = ps[0].m;
    lq4_status st;
    size_t rec_total = 0, t_floats = 0;
    for (uint32_t i = 0; i < count; ++i) {
        rec_total += (dense_record_bytes(m, ps[i].k) + 255) / 256 * 256;
        t_floats += ((size_t)m * ps[i].rank + 63) / 64 * 64;
    }
    if ((st = ensure(ctx, ctx->xs, rec_total, false, s))) return st;
    if ((st = ensure(ctx, ctx->t, t_floats * sizeof(float) + 256, false, s))) return st;
    uint8_t* rec[kMaxGroup];
    float* tptr[kMaxGroup];
    size_t roff = 0, toff = 0;
    uint64_t units = 0;
    for (uint32_t i = 0; i < count; ++i) {
        rec[i] = (uint8_t*)ctx->xs.p + roff;
        tptr[i] = (float*)ctx->t.p + toff;
        roff += (dense_record_bytes(m, ps[i].k) + 255) / 256 * 256;
        toff += ((size_t)m * ps[i].rank + 63) / 64 * 64;
        ps[i].xs_g = rec[i];
        ps[i].t_g = ps[i].rank ? tptr[i] : nullptr;
        units += (uint64_t)ps[i].tiles * ps[i].kg;
    }
    const size_t smem = dense_plan_smem(ps, count);
    if (!smem) return fail(LQ4_ERR_UNSUPPORTED, "dense decode plan does not fit");
    const int grid = (int)(units < (uint64_t)ctx->sm_count ? units : (uint64_t)ctx->sm_count);
    const size_t ng = (m + 3) / 4;
    if ((st = ensure(ctx, ctx->partials, (size_t)grid * kGemvTileRows * ng * 4 * 8, true, s))) return st;
    for (uint32_t i = 0; i < count; ++i) ps[i].partials = (float*)ctx->partials.p;
    LQ4_CUDA(launch_dense_prep(ps, count, rec, tptr, ctx->pdl, s));
    LQ4_CUDA(launch_dense(ps, count, smem, grid, s));
    ctx->launches += 2;
    return LQ4_OK;
}

// One projection of at most 16 tokens through the decode kernels: a single token whose row fits
// in shared memory takes the resident kernel, everything else the dense one.
lq4_status run_gemv_mma(lq4_ctx* ctx, const lq4_linear_args* a, const void* x, int x_dtype, const float* signs,
                        uint32_t m, float* y, uint64_t ldy, cudaStream_t s, const float* x_mul = nullptr,
                        bool as_group = false, uint32_t ldx = 0) {
    GemvParams p;
    fill_params(ctx, a, x, x_dtype, m, y, ldy, p);
    lq4_status st;
    if (x_mul && (signs || x_dtype != LQ4_DTYPE_F32))
        return fail(LQ4_ERR_UNSUPPORTED, "a gated input is f32 and takes no rotation");
    p.x_mul = x_mul;
    p.ldx = ldx;
    if (m == 1 && gemv_resident_fits(1, a->k, signs != nullptr)) {
        p.signs = signs;
        const uint64_t total = (uint64_t)p.tiles * p.kg;
        const int grid = (int)(total < (uint64_t)ctx->sm_count ? total : (uint64_t)ctx->sm_count);
        if ((st = ensure(ctx, ctx->partials, (size_t)grid * kGemvTileRows * 4 * 8, true, s))) return st;
        p.partials = (float*)ctx->partials.p;
        if (p.rank) {
            // the kernel's producer warps compute t = A x themselves and pass it on as tagged messages
            if ((st = ensure(ctx, ctx->tmsg, (size_t)m * p.rank * p.tsplit * sizeof(uint2), true, s))) return st;
            p.tmsg = (uint2*)ctx->tmsg.p;
        }
        const size_t smem = decode_plan_smem(p);
        if (!smem) return fail(LQ4_ERR_UNSUPPORTED, "resident plan does not fit");
        // Decode steps alternate grouped launches (q/k/v, gate/up) with single ones (o_proj, down_proj), and two
        // different kernels in turn start each launch with a cold instruction cache: about 2.5 us per switch
        // here.  A caller that knows a grouped launch comes before (lq4_mlp_block; lq4_linear_group with one
        // problem) asks for the grouped kernel's instantiation, as a group of one.  On its own the single
        // kernel's plan (more stages, whole-tile mode) is about 1.5 us quicker per launch.
        if (as_group && !signs) {
            GemvParams g = p;
            const size_t gsmem = decode_group_plan_smem(&g, 1);
            if (gsmem) {
                const uint64_t gunits = decode_group_units(&g, 1);
                const int ggrid = (int)(gunits < (uint64_t)ctx->sm_count ? gunits : (uint64_t)ctx->sm_count);
                LQ4_CUDA(launch_decode_group(&g, 1, gsmem, ggrid, s));
                ctx->launches += 1;
                return LQ4_OK;
            }
        }
        const uint64_t units = decode_units(p);
        const int dgrid = (int)(units < (uint64_t)ctx->sm_count ? units : (uint64_t)ctx->sm_count);
        LQ4_CUDA(launch_decode(p, smem, dgrid, s));
        ctx->launches += 1;
        return LQ4_OK;
    }
    if (signs) return fail(LQ4_ERR_UNSUPPORTED, "rotation must be applied before the dense decode kernel");
    return run_dense(ctx, &p, 1, s);
}

// Completion signal of a gathered tensor-core product (see lq4_linear): a system-scope fence, one remote
// reduction of 256 on every peer's arrival counter, 256 on this rank's own sequence counter.
struct GatherSignal {
    unsigned long long* arrive[LQ4_MAX_PEERS];    // every rank's buffer base: arrival counter at [0], sequence at [1]
    uint32_t world, rank;
};
__global__ void gather_signal_kernel(const GatherSignal g) {
    __threadfence_system();
    for (uint32_t r = 0; r < g.world; ++r)
        if (r != g.rank)
            asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(g.arrive[r]), "l"(256ull) : "memory");
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(g.arrive[g.rank] + 1), "l"(256ull) : "memory");
}

}  // namespace

extern "C" {

int32_t lq4_abi_version(void) { return 3; }

const char* lq4_last_error(void) { return g_last_error.c_str(); }

const char* lq4_status_string(lq4_status s) {
    switch (s) {
        case LQ4_OK: return "ok";
        case LQ4_ERR_NULL: return "null pointer";
        case LQ4_ERR_K: return "k must be a non-zero multiple of 32";
        case LQ4_ERR_OVERFLOW: return "element count overflow";
        case LQ4_ERR_ALIGN: return "misaligned pointer";
        case LQ4_ERR_DTYPE: return "unknown dtype";
        case LQ4_ERR_LORA: return "invalid LoRA descriptor";
        case LQ4_ERR_ROT: return "invalid rotation descriptor";
        case LQ4_ERR_BAD_BLOCK: return "invalid Q4 block metadata";
        case LQ4_ERR_CUDA: return "CUDA error";
        case LQ4_ERR_UNSUPPORTED: return "unsupported shape or path";
        case LQ4_ERR_DEVICE: return "device-side bounded wait failed";
        case LQ4_ERR_FORMAT: return "malformed .q4 file";
        case LQ4_ERR_IO: return "I/O error";
        case LQ4_ERR_SHAPE: return "shape mismatch";
        case LQ4_ERR_NOSPACE: return "capacity exceeded";
        default: return "unknown status";
    }
}

lq4_status lq4_ctx_create(int32_t device, lq4_ctx** out) {
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    *out = nullptr;
    int count = 0;
    LQ4_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return fail(LQ4_ERR_UNSUPPORTED, "no such CUDA device");
    LQ4_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop{};
    LQ4_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(LQ4_ERR_UNSUPPORTED, "this library contains sm_100a code only; device is sm_" +
                                             std::to_string(prop.major) + std::to_string(prop.minor));
    lq4_ctx* ctx = new lq4_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    LQ4_CUDA(cudaMalloc(&ctx->status, 256));
    LQ4_CUDA(cudaMemset(ctx->status, 0, 256));
    ctx->tsync = reinterpret_cast<uint32_t*>(ctx->status) + 16;
    const char* env = getenv("LQ4_DISABLE_PDL");
    if (env && env[0] == '1') ctx->pdl = 0;
    env = getenv("LQ4_MLP_ONE_LAUNCH");
    if (env && (env[0] == '0' || env[0] == '1')) ctx->mlp_one_launch = env[0] == '1';
    *out = ctx;
    return lq4_ctx_reserve(ctx, 16, 32768, 32768, 128);
}

static void free_step_plan(struct StepPlan* p);      // (defined with the struct, beside lq4_decode_step)

void lq4_ctx_destroy(lq4_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    free_step_plan(ctx->step_plan);
    for (Buf* b : {&ctx->xrot, &ctx->xs, &ctx->t, &ctx->tmsg, &ctx->partials, &ctx->hx, &ctx->hy, &ctx->gemm, &ctx->logits, &ctx->topk, &ctx->topk_ctr, &ctx->mlp, &ctx->mlp_h, &ctx->shard_send, &ctx->shard_recv})
        if (b->p) cudaFree(b->p);
    if (ctx->mlp_step) lq4_peer_buf_free(ctx->mlp_step);
    for (cudaEvent_t e : ctx->ev_block)
        if (e) cudaEventDestroy(e);
    if (ctx->ev_comm) cudaEventDestroy(ctx->ev_comm);
    if (ctx->comm_stream) cudaStreamDestroy(ctx->comm_stream);
    if (ctx->status) cudaFree(ctx->status);
    delete ctx;
}

lq4_status lq4_ctx_reserve(lq4_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, uint32_t rank) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    LQ4_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t s = 0;
    const uint32_t mm = m < 16 ? m : 16;
    const size_t G = ctx->sm_count;
    lq4_status st;
    // a group of eight problems of this shape still fits without growing
    if ((st = ensure(ctx, ctx->xrot, (size_t)m * k * 4, false, s))) return st;
    if ((st = ensure(ctx, ctx->xs, (size_t)kMaxGroup * (dense_record_bytes(mm, k) + 256), false, s))) return st;
    if ((st = ensure(ctx, ctx->t, (size_t)kMaxGroup * ((size_t)mm * rank + 64) * 4 + 256, false, s))) return st;
    if ((st = ensure(ctx, ctx->tmsg, (size_t)kMaxGroup * (rank ? rank : 1) * 8 * sizeof(uint2), true, s))) return st;
    if ((st = ensure(ctx, ctx->partials, G * kGemvTileRows * ((mm + 3) / 4) * 4 * 8, true, s))) return st;
    if ((st = ensure(ctx, ctx->hx, (size_t)m * k * 4, false, s))) return st;
    if ((st = ensure(ctx, ctx->hy, (size_t)m * n * 4, false, s))) return st;
    if (m > 16) {
        const size_t need = gemm_workspace_bytes(m, n, k, rank);
        if ((st = ensure(ctx, ctx->gemm, need, false, s))) return st;
    }
    // the clears above ran on the legacy default stream, which does not order a later launch on a
    // non-blocking stream behind them: finish them here (set-up time, not the hot path)
    LQ4_CUDA(cudaStreamSynchronize(s));
    return LQ4_OK;
}

lq4_status lq4_ctx_check(lq4_ctx* ctx, void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    cudaStream_t s = (cudaStream_t)stream;
    int32_t h = 0;
    LQ4_CUDA(cudaMemcpyAsync(&h, ctx->status, 4, cudaMemcpyDeviceToHost, s));
    LQ4_CUDA(cudaStreamSynchronize(s));
    if (h != 0) {
        cudaMemsetAsync(ctx->status, 0, 4, s);
        cudaStreamSynchronize(s);
        return fail(LQ4_ERR_DEVICE, "kernel reported a failed bounded wait, status bits " + std::to_string(h));
    }
    return LQ4_OK;
}

uint64_t lq4_ctx_launch_count(const lq4_ctx* ctx) { return ctx ? ctx->launches : 0; }

lq4_status lq4_ctx_set_option(lq4_ctx* ctx, int32_t option, int32_t value) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    switch (option) {
        case LQ4_OPT_MLP_ONE_LAUNCH: ctx->mlp_one_launch = value != 0; return LQ4_OK;
        case LQ4_OPT_PDL: ctx->pdl = value != 0; return LQ4_OK;
        case LQ4_OPT_ALLOW_GROW: ctx->allow_grow = value != 0; return LQ4_OK;
        default: return fail(LQ4_ERR_UNSUPPORTED, "unknown option");
    }
}

lq4_status lq4_linear(lq4_ctx* ctx, const lq4_linear_args* a, void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    lq4_status st = validate_linear(a);
    if (st) return st;
    if (a->m == 0 || a->n == 0) return LQ4_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const uint64_t ldy = a->ldy ? a->ldy : a->n;
    const uint32_t rank = a->lora ? a->lora->rank : 0;

    const bool fast_layout = (a->k % 128 == 0) && aligned(a->w, 16) && aligned(a->x, 16) && rank <= kGemvMaxRank;
    int path = a->path;
    if (path == LQ4_PATH_AUTO) {
        if (!fast_layout) path = LQ4_PATH_GEMV_GENERIC;
        else if (a->m <= (uint32_t)kGemvMaxM) path = LQ4_PATH_GEMV_MMA;                          // decode kernels
        else if (a->m <= 32 || (a->m <= 64 && a->n <= 8192)) {
            // A few dozen tokens leave the tensor-core kernel with too few 256-row tiles to fill the GPU and a
            // serial walk over k in each (measured, 5120 -> 17408: 98 us at 32 tokens; 17408 -> 5120: 250 us);
            // the decode kernel in chunks of 16 tokens streams the weights once per chunk and is quicker here
            // (31 to 35 us per chunk on those shapes).  Not with a fused all-gather: that path is per launch.
            path = (a->gather && a->gather->world > 1) ? LQ4_PATH_GEMM_TC : LQ4_PATH_GEMV_MMA;
            if (path == LQ4_PATH_GEMM_TC && !gemm_supported(a->m, a->n, a->k, rank > (uint32_t)kGemmMaxRank ? 0u : rank)) path = LQ4_PATH_GEMV_MMA;
        }
        else path = gemm_supported(a->m, a->n, a->k, rank > (uint32_t)kGemmMaxRank ? 0u : rank) ? LQ4_PATH_GEMM_TC : LQ4_PATH_GEMV_MMA;
    }
    if (path != LQ4_PATH_GEMV_GENERIC && !fast_layout)
        return fail(LQ4_ERR_ALIGN, "fast paths need k % 128 == 0, 16-byte aligned w and x, rank <= 512");
    if (a->gather && a->gather->world > 1) {
        const bool decode = path == LQ4_PATH_GEMV_MMA && a->m <= (uint32_t)kGemvMaxM;
        const bool prefill = path == LQ4_PATH_GEMM_TC && rank <= (uint32_t)kGemmMaxRank;
        if (!decode && !prefill)
            return fail(LQ4_ERR_UNSUPPORTED, "the fused all-gather is built into the decode kernels (m <= 16) and the tensor-core "
                                             "kernel (adapter rank <= 128), fast layout");
    }

    const void* x = a->x;
    int x_dtype = a->x_dtype;
    const float* signs = a->rot ? a->rot->signs : nullptr;
    // the decode kernels wait for gathered inputs themselves; every other first reader of x
    // (rotation kernel, tensor-core path, generic kernel) gets the stand-alone wait in front
    bool wait_in_kernel = path == LQ4_PATH_GEMV_MMA && a->m <= (uint32_t)kGemvMaxM;

    // The decode kernel rotates in its own prologue when the row fits; otherwise the
    // rotation runs as a kernel of its own into the workspace.
    const bool in_kernel_rot = signs && a->rot->dim == a->k && path == LQ4_PATH_GEMV_MMA && a->m == 1 && rank == 0 &&
                               gemv_resident_fits(1, a->k, true);
    if (signs && !in_kernel_rot) wait_in_kernel = false;
    if (a->wait_gather && a->wait_gather->world > 1 && !wait_in_kernel)
        if ((st = lq4_gather_wait(ctx, a->wait_gather, stream))) return st;
    if (signs && !in_kernel_rot) {
        if ((st = ensure(ctx, ctx->xrot, (size_t)a->m * a->k * 4, false, s))) return st;
        const uint32_t blocks = a->k / a->rot->dim;          // 1: full rotation; more: block-diagonal
        LQ4_CUDA(launch_hadamard_rows(x, x_dtype, signs, a->rot->dim, a->m * blocks, (float*)ctx->xrot.p, s, blocks));
        ctx->launches += 1;
        x = ctx->xrot.p;
        x_dtype = LQ4_DTYPE_F32;
        signs = nullptr;
    }

    if (path == LQ4_PATH_GEMV_MMA) {
        for (uint32_t m0 = 0; m0 < a->m; m0 += kGemvMaxM) {
            const uint32_t mc = a->m - m0 < (uint32_t)kGemvMaxM ? a->m - m0 : (uint32_t)kGemvMaxM;
            const size_t esz = x_dtype == LQ4_DTYPE_F32 ? 4 : 2;
            const void* xc = static_cast<const uint8_t*>(x) + (size_t)m0 * a->k * esz;
            if ((st = run_gemv_mma(ctx, a, xc, x_dtype, signs, mc, a->y + (size_t)m0 * ldy, ldy, s))) return st;
        }
        return LQ4_OK;
    }
    if (path == LQ4_PATH_GEMM_TC) {
        // An adapter wider than the tensor-core kernel carries along (a blend of several adapters adds their
        // ranks) is applied as the reference applies every adapter: the projection first, then
        // y += scale * B (A x) in a pass of its own.
        const bool wide = rank > (uint32_t)kGemmMaxRank;
        const uint32_t grank = wide ? 0u : rank;
        if (!gemm_supported(a->m, a->n, a->k, grank)) return fail(LQ4_ERR_UNSUPPORTED, "shape not handled by the tensor-core kernel");
        const size_t need = gemm_workspace_bytes(a->m, a->n, a->k, grank);
        if ((st = ensure(ctx, ctx->gemm, need, false, s))) return st;
        int launches = 0;
        std::string err;
        int64_t peer_off[LQ4_MAX_PEERS];
        uint32_t n_peers = 0;
        const lq4_gather_desc* gd = (a->gather && a->gather->world > 1) ? a->gather : nullptr;
        if (gd)
            for (uint32_t r = 0; r < gd->world; ++r)
                if (r != gd->rank) peer_off[n_peers++] = static_cast<const char*>(gd->bases[r]) - static_cast<const char*>(gd->bases[gd->rank]);
        cudaError_t e = launch_gemm_tc(x, x_dtype, a->w, a->y, ldy, a->m, a->n, a->k,
                                       grank ? a->lora->a : nullptr, grank ? a->lora->b : nullptr, grank,
                                       grank ? a->lora->scale : 0.0f, ctx->gemm.p, ctx->gemm.cap, ctx->status,
                                       ctx->sm_count, s, &launches, &err, peer_off, n_peers);
        ctx->launches += launches;
        if (e != cudaSuccess) return fail(LQ4_ERR_CUDA, "tensor-core GEMM: " + err + ": " + cudaGetErrorString(e));
        if (gd) {
            // the product's stores into the peers' buffers are complete when its kernel is; the kernel behind it
            // tells every peer (one remote reduction each) and advances this rank's sequence, exactly what the
            // last CTA of a gathered decode launch does, so lq4_gather_wait serves both
            GatherSignal sig{};
            sig.world = gd->world; sig.rank = gd->rank;
            for (uint32_t r = 0; r < gd->world; ++r) sig.arrive[r] = static_cast<unsigned long long*>(gd->bases[r]);
            gather_signal_kernel<<<1, 1, 0, s>>>(sig);
            LQ4_CUDA(cudaGetLastError());
            ctx->launches += 1;
        }
        if (wide) return lq4_lora_apply(ctx, x, x_dtype, a->m, a->k, a->y, a->n, ldy, a->lora, stream);
        return LQ4_OK;
    }
    // generic
    const float* t = nullptr;
    if (rank) {
        if ((st = ensure(ctx, ctx->t, (size_t)a->m * rank * 4, false, s))) return st;
        launch_lora_t(x, x_dtype, a->m, a->k, a->lora->a, rank, (float*)ctx->t.p, s);
        ctx->launches += 1;
        t = (const float*)ctx->t.p;
    }
    launch_gemv_generic(x, x_dtype, a->w, a->y, ldy, a->m, a->n, a->k, t, a->lora ? a->lora->b : nullptr, rank,
                        a->lora ? a->lora->scale : 0.0f, 0, s);
    ctx->launches += 1;
    LQ4_CUDA(cudaGetLastError());
    return LQ4_OK;
}

namespace {
struct StepSpec {
    lq4_linear_args a;
    const float* x_mul;      // gating row for this problem's input (silu(x) * x_mul), or NULL
};
lq4_status step_core(lq4_ctx* ctx, const StepSpec* specs, const uint32_t* gsize, uint32_t ngroups, const lq4_step_desc* step,
                     cudaStream_t s);
}  // namespace

lq4_status lq4_linear_group(lq4_ctx* ctx, const lq4_linear_args* args, uint32_t count, void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (count == 0) return LQ4_OK;
    if (!args) return fail(LQ4_ERR_NULL, "args is NULL");
    lq4_status st;
    for (uint32_t i = 0; i < count; ++i)
        if ((st = validate_linear(&args[i]))) return st;
    cudaStream_t s = (cudaStream_t)stream;

    // One launch serves the whole group when every problem is a decode-kernel case of the same
    // token count; anything else runs problem by problem with the same results.
    if (count == 1) {
        // a group of one: the same result as lq4_linear, on the grouped kernel's instantiation where the
        // shape allows it (for callers that interleave single projections with grouped launches)
        const lq4_linear_args& a = args[0];
        const uint32_t rank = a.lora ? a.lora->rank : 0;
        const bool fits = a.m == 1 && a.n > 0 && !a.rot && (a.k % 128 == 0) && aligned(a.w, 16) && aligned(a.x, 16) &&
                          rank <= (uint32_t)kGemvMaxRank && (a.path == LQ4_PATH_AUTO || a.path == LQ4_PATH_GEMV_MMA) &&
                          !(a.wait_gather && a.wait_gather->world > 1) && gemv_resident_fits(1, a.k, false);
        if (!fits) return lq4_linear(ctx, &a, stream);
        return run_gemv_mma(ctx, &a, a.x, a.x_dtype, nullptr, 1, a.y, a.ldy ? a.ldy : a.n, s, nullptr, true);
    }
    if (count > (uint32_t)kMaxGroup && count <= (uint32_t)kStepMaxProblems) {
        // 9 to 24 one-token projections: one group of the step kernel (one persistent launch) when every
        // problem qualifies for it; else problem by problem below
        bool step_ok = true;
        for (uint32_t i = 0; i < count && step_ok; ++i) {
            const lq4_linear_args& a = args[i];
            const uint32_t rank = a.lora ? a.lora->rank : 0;
            step_ok = a.m == 1 && a.n > 0 && !a.rot && !a.gather && !a.wait_gather && (a.k % 128 == 0) && aligned(a.w, 16) &&
                      aligned(a.x, 16) && rank <= (uint32_t)kGemvMaxRank && (!a.lora || aligned(a.lora->a, 16)) &&
                      (a.path == LQ4_PATH_AUTO || a.path == LQ4_PATH_GEMV_MMA) && (a.ldy == 0 || a.ldy == a.n) &&
                      gemv_resident_fits(1, a.k, false);
            // no output may be another problem's input (a step orders its groups; a group's problems are independent)
            for (uint32_t j = 0; j < count && step_ok; ++j) {
                const char* y0 = reinterpret_cast<const char*>(args[j].y);
                const char* x0 = static_cast<const char*>(a.x);
                const size_t xb = (size_t)a.k * (a.x_dtype == LQ4_DTYPE_BF16 ? 2 : 4);
                step_ok = !(x0 < y0 + (size_t)args[j].n * 4 && y0 < x0 + xb);
            }
        }
        if (step_ok) {
            StepSpec specs[kStepMaxProblems];
            for (uint32_t i = 0; i < count; ++i) { specs[i].a = args[i]; specs[i].x_mul = nullptr; }
            const uint32_t gsize[1] = {count};
            st = step_core(ctx, specs, gsize, 1, nullptr, s);
            if (st != LQ4_ERR_UNSUPPORTED) return st;      // (refused before anything was launched: e.g. a row too long for two limb buffers)
        }
    }
    bool one_launch = count >= 2 && count <= (uint32_t)kMaxGroup;
    GemvParams ps[kMaxGroup];
    const uint32_t m = args[0].m;
    for (uint32_t i = 0; i < count && one_launch; ++i) {
        const lq4_linear_args& a = args[i];
        const uint32_t rank = a.lora ? a.lora->rank : 0;
        one_launch = a.m >= 1 && a.m <= (uint32_t)kGemvMaxM && a.m == m && a.n > 0 && !a.rot && (a.k % 128 == 0) &&
                     aligned(a.w, 16) && aligned(a.x, 16) && rank <= (uint32_t)kGemvMaxRank &&
                     (a.path == LQ4_PATH_AUTO || a.path == LQ4_PATH_GEMV_MMA);
        one_launch = one_launch && a.gather == args[0].gather &&      // one arrival signal, one wait per launch
                     a.wait_gather == args[0].wait_gather;
        if (one_launch) fill_params(ctx, &a, a.x, a.x_dtype, a.m, a.y, a.ldy ? a.ldy : a.n, ps[i]);
    }
    size_t smem = 0;
    if (one_launch && m == 1) {
        smem = decode_group_plan_smem(ps, count);      // 0: some row does not fit in shared memory
    }
    if (!one_launch) {
        for (uint32_t i = 0; i < count; ++i)
            if ((st = lq4_linear(ctx, &args[i], stream))) return st;
        return LQ4_OK;
    }
    if (m > 1 || !smem) return run_dense(ctx, ps, count, s);

    size_t items = 0;
    for (uint32_t i = 0; i < count; ++i) items += (size_t)m * ps[i].rank * ps[i].tsplit;
    if ((st = ensure(ctx, ctx->tmsg, items * sizeof(uint2), true, s))) return st;
    items = 0;
    for (uint32_t i = 0; i < count; ++i) {
        ps[i].tmsg = (uint2*)ctx->tmsg.p + items;
        items += (size_t)m * ps[i].rank * ps[i].tsplit;
    }
    const uint64_t units = decode_group_units(ps, count);
    const int grid = (int)(units < (uint64_t)ctx->sm_count ? units : (uint64_t)ctx->sm_count);
    if ((st = ensure(ctx, ctx->partials, (size_t)grid * kGemvTileRows * 4 * 8, true, s))) return st;
    for (uint32_t i = 0; i < count; ++i) ps[i].partials = (float*)ctx->partials.p;
    LQ4_CUDA(launch_decode_group(ps, count, smem, grid, s));
    ctx->launches += 1;
    return LQ4_OK;
}

// ---- peer buffers and the wait of the fused all-gather ------------------------------------
struct lq4_peer_buf {
    void* base = nullptr;
    uint64_t payload_bytes = 0;
    uint64_t mailbox_off = 0;      // step buffers: bytes from base to the mailbox (0: none)
    uint64_t mailbox_half = 0;     // entries per half
};

namespace {
// Layout of the buffers created in this process, by base address: the C ABI passes bases, and the
// peers' buffers have the layout of the own one.
std::mutex g_peer_mu;
std::map<void*, lq4_peer_buf> g_peer_bufs;

bool peer_buf_info(void* base, lq4_peer_buf* out) {
    std::lock_guard<std::mutex> lk(g_peer_mu);
    auto it = g_peer_bufs.find(base);
    if (it == g_peer_bufs.end()) return false;
    *out = it->second;
    return true;
}

lq4_status peer_buf_alloc(uint64_t payload_bytes, bool mailbox, lq4_peer_buf** out) {
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    *out = nullptr;
    if (payload_bytes == 0) return fail(LQ4_ERR_SHAPE, "payload size is 0");
    if (payload_bytes > ((uint64_t)1 << 40)) return fail(LQ4_ERR_OVERFLOW, "payload too large");
    lq4_peer_buf* b = new lq4_peer_buf();
    const uint64_t pay = (payload_bytes + 255) / 256 * 256;
    uint64_t bytes = 256 + pay;
    if (mailbox) {
        b->mailbox_off = bytes;
        b->mailbox_half = pay / 4;                 // one 8-byte entry per payload float, twice
        bytes += 2 * b->mailbox_half * 8;
    }
    cudaError_t e = cudaMalloc(&b->base, bytes);
    if (e == cudaSuccess) e = cudaMemset(b->base, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (b->base) cudaFree(b->base);
        delete b;
        return cuda_fail(e, "peer buffer allocation");
    }
    b->payload_bytes = payload_bytes;
    {
        std::lock_guard<std::mutex> lk(g_peer_mu);
        g_peer_bufs[b->base] = *b;
    }
    *out = b;
    return LQ4_OK;
}
}  // namespace

namespace {
// One thread.  With programmatic dependent launch it first lets the launch after it start (a decode
// kernel begins streaming weights at once and waits for this grid before it reads activations),
// then waits for the gathered launch before it, whose sequence count it needs.
__global__ void gather_wait_kernel(const unsigned long long* arrive, const unsigned long long* gseq, uint32_t world,
                                   int32_t* status, int use_pdl) {
    if (use_pdl) {
        pdl_launch_dependents();
        pdl_wait_prior_grids();
    }
    unsigned long long seq;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(seq) : "l"(gseq) : "memory");
    const unsigned long long need = (seq >> 8) * 256ull * (world - 1);
    const long long t0 = wait_clock();
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(arrive) : "memory");
        if (v >= need) break;
        if (wait_expired(t0)) { atomicOr(status, kDevErrGridWaitTimeout); break; }
    }
}
}  // namespace

lq4_status lq4_peer_buf_create(uint64_t payload_bytes, lq4_peer_buf** out) {
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    *out = nullptr;
    if (payload_bytes == 0) return fail(LQ4_ERR_SHAPE, "payload_bytes is 0");
    return peer_buf_alloc(payload_bytes, false, out);
}

lq4_status lq4_step_buf_create(uint64_t payload_floats, lq4_peer_buf** out) {
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    *out = nullptr;
    if (payload_floats == 0) return fail(LQ4_ERR_SHAPE, "payload_floats is 0");
    if (payload_floats > 0x7fffffffull) return fail(LQ4_ERR_OVERFLOW, "a step buffer holds fewer than 2^31 floats");
    return peer_buf_alloc(payload_floats * 4, true, out);
}

void lq4_peer_buf_free(lq4_peer_buf* b) {
    if (!b) return;
    {
        std::lock_guard<std::mutex> lk(g_peer_mu);
        g_peer_bufs.erase(b->base);
    }
    if (b->base) cudaFree(b->base);
    delete b;
}

void* lq4_peer_buf_base(const lq4_peer_buf* b) { return b ? b->base : nullptr; }
void* lq4_peer_buf_payload(const lq4_peer_buf* b) { return b ? static_cast<char*>(b->base) + 256 : nullptr; }

lq4_status lq4_peer_buf_export(const lq4_peer_buf* b, uint8_t* handle_out) {
    if (!b || !handle_out) return fail(LQ4_ERR_NULL, "buffer or handle_out is NULL");
    static_assert(sizeof(cudaIpcMemHandle_t) == LQ4_PEER_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    LQ4_CUDA(cudaIpcGetMemHandle(&h, b->base));
    memcpy(handle_out, &h, sizeof(h));
    return LQ4_OK;
}

lq4_status lq4_peer_buf_open(const uint8_t* handle, void** base_out) {
    if (!handle || !base_out) return fail(LQ4_ERR_NULL, "handle or base_out is NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    LQ4_CUDA(cudaIpcOpenMemHandle(base_out, h, cudaIpcMemLazyEnablePeerAccess));
    return LQ4_OK;
}

lq4_status lq4_peer_buf_close(void* base) {
    if (!base) return LQ4_OK;
    LQ4_CUDA(cudaIpcCloseMemHandle(base));
    return LQ4_OK;
}

lq4_status lq4_gather_wait(lq4_ctx* ctx, const lq4_gather_desc* g, void* stream) {
    if (!ctx || !g) return fail(LQ4_ERR_NULL, "ctx or gather is NULL");
    if (g->world < 1 || g->world > LQ4_MAX_PEERS || g->rank >= g->world || !g->bases[g->rank])
        return fail(LQ4_ERR_SHAPE, "gather: world must be 1..8, rank < world, own base non-NULL");
    if (g->world == 1) return LQ4_OK;
    const unsigned long long* own = static_cast<const unsigned long long*>(g->bases[g->rank]);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (ctx->pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    LQ4_CUDA(cudaLaunchKernelEx(&cfg, gather_wait_kernel, own, own + 1, g->world, ctx->status, ctx->pdl));
    ctx->launches += 1;
    return LQ4_OK;
}

namespace {

}  // namespace

// A decode loop issues the same step again and again (same buffers, same weights): planning it (validation,
// CTA shares, tensor maps, shared-memory plan: about 15 us of host time for sixteen projections) is done once and
// the argument block is kept.  The key is every byte the plan depends on: the problems' argument structs and
// adapter descriptors, the group sizes, the step descriptor with its buffer layout, the context's switches and
// the generation of its workspace.
struct StepPlan {
    std::vector<uint8_t> key;
    StepArgs args;
    size_t smem = 0;
    int grid = 0;
};
static void free_step_plan(StepPlan* p) { delete p; }

namespace {

// Core of lq4_decode_step: `specs` are the problems in group order, `gsize[g]` the size of group g.
lq4_status step_core(lq4_ctx* ctx, const StepSpec* specs, const uint32_t* gsize, uint32_t ngroups, const lq4_step_desc* step,
                     cudaStream_t s) {
    uint32_t np = 0;
    for (uint32_t g = 0; g < ngroups; ++g) np += gsize[g];
    if (ngroups == 0 || np == 0) return LQ4_OK;
    if (ngroups > (uint32_t)kStepMaxGroups) return fail(LQ4_ERR_NOSPACE, "a step holds at most 8 groups");
    if (np > (uint32_t)kStepMaxProblems) return fail(LQ4_ERR_NOSPACE, "a step holds at most 24 projections");
    lq4_status st;

    // the step buffer, if any
    lq4_peer_buf info{};
    const lq4_gather_desc* gd = step ? step->bufs : nullptr;
    uint32_t world = 1, grank = 0;
    char* base = nullptr;
    if (gd) {
        if (gd->world < 1 || gd->world > LQ4_MAX_PEERS || gd->rank >= gd->world) return fail(LQ4_ERR_SHAPE, "step: world must be 1..8 and rank < world");
        world = gd->world; grank = gd->rank;
        for (uint32_t r = 0; r < world; ++r)
            if (!gd->bases[r] || !aligned(gd->bases[r], 256)) return fail(LQ4_ERR_NULL, "step: a buffer base is NULL or misaligned");
        base = static_cast<char*>(gd->bases[grank]);
        if (!peer_buf_info(base, &info) || info.mailbox_off == 0)
            return fail(LQ4_ERR_SHAPE, "step: bases[rank] is not a step buffer created by lq4_step_buf_create in this process");
    } else if (step) {
        return fail(LQ4_ERR_NULL, "step->bufs is NULL");
    }
    thread_local std::vector<uint8_t> key;
    key.clear();
    auto put = [&](const void* p, size_t n) {
        const uint8_t* b = static_cast<const uint8_t*>(p);
        key.insert(key.end(), b, b + n);
    };
    put(&ngroups, sizeof(ngroups));
    put(gsize, sizeof(uint32_t) * ngroups);
    put(&ctx->pdl, sizeof(ctx->pdl));
    put(&ctx->alloc_gen, sizeof(ctx->alloc_gen));
    for (uint32_t i = 0; i < np; ++i) {
        put(&specs[i].a, sizeof(lq4_linear_args));
        put(&specs[i].x_mul, sizeof(specs[i].x_mul));
        if (specs[i].a.lora) put(specs[i].a.lora, sizeof(lq4_lora_desc));
    }
    if (step) {
        put(&step->n_gathered, sizeof(step->n_gathered));
        if (step->gathered && step->n_gathered <= (uint32_t)kStepMaxRanges) put(step->gathered, sizeof(lq4_step_range) * step->n_gathered);
        if (gd) put(gd, sizeof(lq4_gather_desc));
        put(&info.payload_bytes, sizeof(info.payload_bytes));
        put(&info.mailbox_off, sizeof(info.mailbox_off));
        put(&info.mailbox_half, sizeof(info.mailbox_half));
    }
    if (ctx->step_plan && ctx->step_plan->key == key) {
        LQ4_CUDA(launch_decode_step(ctx->step_plan->args, ctx->step_plan->smem, ctx->step_plan->grid, s));
        ctx->launches += 1;
        return LQ4_OK;
    }
    float* payload = base ? reinterpret_cast<float*>(base + 256) : nullptr;
    const uint64_t pfloats = base ? info.payload_bytes / 4 : 0;
    auto in_payload = [&](const void* p, uint64_t count) {
        if (!payload) return false;
        const char* c = static_cast<const char*>(p);
        return c >= reinterpret_cast<const char*>(payload) && c + count * 4 <= reinterpret_cast<const char*>(payload + pfloats);
    };

    thread_local StepArgs sa;
    sa = StepArgs{};
    sa.ngroups = ngroups;
    sa.use_pdl = ctx->pdl;
    sa.tsync = ctx->tsync;
    sa.status = ctx->status;
    sa.world = world;
    sa.grank = grank;
    uint32_t max_kb = 0, max_rank = 0;
    size_t items_total = 0;
    uint32_t pi = 0;
    uint64_t max_units = 0;
    for (uint32_t g = 0; g < ngroups; ++g) {
        sa.group_begin[g] = pi;
        uint64_t units = 0;
        for (uint32_t i = 0; i < gsize[g]; ++i, ++pi) {
            const lq4_linear_args& a = specs[pi].a;
            if ((st = validate_linear(&a))) return st;
            const uint32_t rank = a.lora ? a.lora->rank : 0;
            if (a.m != 1 || a.n == 0) return fail(LQ4_ERR_SHAPE, "a step takes one-token projections (m == 1, n > 0)");
            if (a.rot) return fail(LQ4_ERR_UNSUPPORTED, "a step takes no online rotation");
            if (a.gather || a.wait_gather) return fail(LQ4_ERR_UNSUPPORTED, "a step's exchange is described by lq4_step_desc, not per projection");
            if (a.k % 128 != 0 || !aligned(a.w, 16) || !aligned(a.x, 16) || rank > (uint32_t)kGemvMaxRank)
                return fail(LQ4_ERR_ALIGN, "a step needs k % 128 == 0, 16-byte aligned w and x, rank <= 512");
            if (a.lora && !aligned(a.lora->a, 16)) return fail(LQ4_ERR_ALIGN, "a step needs 16-byte aligned LoRA A");
            if (a.path != LQ4_PATH_AUTO && a.path != LQ4_PATH_GEMV_MMA) return fail(LQ4_ERR_UNSUPPORTED, "a step runs on the decode kernel");
            StepProblem& q = sa.p[pi];
            q.y = a.y;
            q.x = a.x;
            q.x_mul = specs[pi].x_mul;
            q.x_dtype = a.x_dtype;
            q.n = a.n; q.k = a.k; q.kb = a.k / 32; q.kg = q.kb / kGemvGranuleBlocks;
            q.tiles = (a.n + kGemvTileRows - 1) / kGemvTileRows;
            q.x_slot = q.xmul_slot = q.y_slot = kNoSlot;
            q.rank = rank;
            q.tsplit = 1;
            if (rank) { q.la = a.lora->a; q.lb = a.lora->b; q.lscale = a.lora->scale; q.tsplit = decode_tsplit(a.k); }
            q.dot_begin = 0;
            if (in_payload(a.y, a.n)) q.y_slot = (uint32_t)(a.y - payload);
            else if (world > 1) return fail(LQ4_ERR_SHAPE, "N-sharded step: every output must lie in the step buffer's payload");
            max_kb = q.kb > max_kb ? q.kb : max_kb;
            max_rank = rank > max_rank ? rank : max_rank;
            items_total += (size_t)rank * q.tsplit;
            units += (uint64_t)q.tiles * q.kg;
        }
        max_units = units > max_units ? units : max_units;
    }
    sa.group_begin[ngroups] = pi;

    // which inputs come from earlier groups of this launch
    auto overlaps = [](const char* a0, const char* a1, const char* b0, const char* b1) { return a0 < b1 && b0 < a1; };
    for (uint32_t g = 0; g < ngroups; ++g) {
        for (uint32_t i = sa.group_begin[g]; i < sa.group_begin[g + 1]; ++i) {
            StepProblem& q = sa.p[i];
            const lq4_linear_args& a = specs[i].a;
            const size_t esz = a.x_dtype == LQ4_DTYPE_BF16 ? 2 : 4;
            const char* x0 = static_cast<const char*>(a.x);
            const char* x1 = x0 + (size_t)a.k * esz;
            const char* u0 = reinterpret_cast<const char*>(specs[i].x_mul);
            const char* u1 = u0 ? u0 + (size_t)a.k * 4 : nullptr;
            bool x_internal = false, u_internal = false;
            for (uint32_t j = 0; j < np; ++j) {
                const char* y0 = reinterpret_cast<const char*>(sa.p[j].y);
                const char* y1 = y0 + (size_t)sa.p[j].n * 4;
                const bool earlier = j < sa.group_begin[g];
                const bool hx = overlaps(x0, x1, y0, y1), hu = u0 && overlaps(u0, u1, y0, y1);
                if ((hx || hu) && !earlier)
                    return fail(LQ4_ERR_SHAPE, "a projection reads what a projection of the same or a later group writes");
                x_internal = x_internal || hx;
                u_internal = u_internal || hu;
            }
            if (x_internal || u_internal) {
                if (a.x_dtype != LQ4_DTYPE_F32) return fail(LQ4_ERR_DTYPE, "inputs taken from earlier groups are f32");
                if (!in_payload(a.x, a.k) || (u0 && !in_payload(u0, a.k)))
                    return fail(LQ4_ERR_SHAPE, "inputs taken from earlier groups must lie in the step buffer's payload");
                if (u0 && x_internal != u_internal) return fail(LQ4_ERR_UNSUPPORTED, "a gated input and its multiplier must both come from earlier groups");
                q.x_slot = (uint32_t)(static_cast<const float*>(a.x) - payload);
                if (u0) q.xmul_slot = (uint32_t)(specs[i].x_mul - payload);
                if (q.rank) {
                    // short pieces: one lane of the projection warp keeps a whole piece's loads in flight
                    const uint32_t per_piece = 32u * (uint32_t)kStepMailboxStrides;       // float4 per piece
                    uint32_t ts = (a.k / 4 + per_piece - 1) / per_piece;
                    q.tsplit = ts < 1 ? 1 : (ts > kStepMaxTsplit ? kStepMaxTsplit : ts);
                }
                if ((q.x_slot & 3u) || (u0 && (q.xmul_slot & 3u))) return fail(LQ4_ERR_ALIGN, "inputs taken from earlier groups need 16-byte alignment");
            }
            if (u0 && !aligned(u0, 16)) return fail(LQ4_ERR_ALIGN, "the gating row needs 16-byte alignment");
        }
    }

    items_total = 0;
    uint32_t max_items = 0;
    for (uint32_t i = 0; i < np; ++i) {
        items_total += (size_t)sa.p[i].rank * sa.p[i].tsplit;
        max_items = sa.p[i].rank * sa.p[i].tsplit > max_items ? sa.p[i].rank * sa.p[i].tsplit : max_items;
    }
    const int grid = (int)(max_units < (uint64_t)ctx->sm_count ? max_units : (uint64_t)ctx->sm_count);

    // CTA shares and projection items per group
    if ((st = ensure(ctx, ctx->tmsg, (items_total + 1) * sizeof(uint2), true, s))) return st;
    if ((st = ensure(ctx, ctx->partials, (size_t)ngroups * grid * kGemvTileRows * 8, true, s))) return st;
    sa.partials = (float*)ctx->partials.p;
    size_t item_off = 0;
    // Work units charged per finished tile: between the problems of a group (how many CTAs each gets) and
    // inside a problem (where its CTAs' shares are cut).  Measured on the large-layer step (a finished tile
    // costs its CTA 1 to 1.5 us, a work unit streams in about 0.24 us): 5 and 8 are quickest, 3.4 % ahead of an
    // even cut inside the problems.  LQ4_TILE_CHARGE / LQ4_STEP_SHARE_CHARGE override them for tuning.
    constexpr uint32_t kStepTileCharge = 5, kStepShareCharge = 8;
    static const uint32_t share_charge = [] {
        const char* e = getenv("LQ4_STEP_SHARE_CHARGE");
        return e ? (uint32_t)atoi(e) : kStepShareCharge;
    }();
    for (uint32_t g = 0; g < ngroups; ++g) {
        const uint32_t b = sa.group_begin[g], cnt = sa.group_begin[g + 1] - b;
        GemvParams tmp[kStepMaxProblems];
        uint32_t cta_begin[kStepMaxProblems + 1];
        for (uint32_t i = 0; i < cnt; ++i) { tmp[i] = GemvParams{}; tmp[i].tiles = sa.p[b + i].tiles; tmp[i].kg = sa.p[b + i].kg; }
        if ((uint32_t)grid < cnt) return fail(LQ4_ERR_UNSUPPORTED, "a group has more projections than the launch has CTAs");
        dec::split_ctas(tmp, cnt, (uint32_t)grid, cta_begin, kStepTileCharge);
        uint32_t dots = 0;
        for (uint32_t i = 0; i < cnt; ++i) {
            StepProblem& q = sa.p[b + i];
            q.cta_begin = cta_begin[i];
            q.cta_count = cta_begin[i + 1] - cta_begin[i];
            {
                // the same charge inside a problem; small shares (a few units per CTA) are cut evenly instead
                const uint64_t per_cta = (uint64_t)q.tiles * q.kg / q.cta_count;
                q.charge = per_cta / 4 < share_charge ? (uint32_t)(per_cta / 4) : share_charge;
                // the kernel does this arithmetic in 32 bits (enough for any payload that fits the device's memory)
                if (!step_share_fits32(q.tiles, q.kg, q.charge, q.cta_count)) return fail(LQ4_ERR_UNSUPPORTED, "a projection of this step has too many work units");
            }
            q.dot_begin = dots;
            q.tmsg = (uint2*)ctx->tmsg.p + item_off + dots;
            dots += q.rank * q.tsplit;
            const dec::MapEntry* e = dec::maps_for(specs[b + i].a.w, q.n, q.kb);
            if (!e) return fail(LQ4_ERR_CUDA, "tensor map encoding failed");
            for (int j = 0; j < 3; ++j) sa.maps[b + i][j] = e->m[j];
        }
        sa.group_items[g] = dots;
        item_off += dots;
    }
    // limb buffers: the longest k range a CTA converts in any group (the whole row when its share spans a tile)
    uint32_t cap_blocks = 0;
    for (uint32_t i = 0; i < np; ++i) {
        const StepProblem& q = sa.p[i];
        // no share is longer than the even cut of the stretched range (a share without a tile start is exactly that long)
        const uint64_t totalv = (uint64_t)q.tiles * ((uint64_t)q.kg + q.charge);
        const uint64_t share = (totalv + q.cta_count - 1) / q.cta_count;
        const uint32_t blocks = share >= q.kg ? q.kb : (uint32_t)share * kGemvGranuleBlocks;
        cap_blocks = blocks > cap_blocks ? blocks : cap_blocks;
    }
    const size_t smem = step_plan_smem(sa, cap_blocks, max_rank, max_items);
    if (!smem) return fail(LQ4_ERR_UNSUPPORTED, "a row of this step does not fit in shared memory");

    // mailbox and the ranges to hand back as plain f32
    sa.step_counter = ctx->tsync;
    if (base) {
        sa.mbox = reinterpret_cast<unsigned long long*>(base + info.mailbox_off);
        sa.mbox_half = (uint32_t)info.mailbox_half;
        sa.step_counter = reinterpret_cast<uint32_t*>(base + 32);
        sa.payload = payload;
        for (uint32_t r = 0; r < world; ++r)
            sa.peer_mbox_off[r] = static_cast<const char*>(gd->bases[r]) - base;
        if (step->n_gathered > (uint32_t)kStepMaxRanges) return fail(LQ4_ERR_NOSPACE, "a step hands back at most 8 ranges");
        if (step->n_gathered && !step->gathered) return fail(LQ4_ERR_NULL, "step->gathered is NULL");
        for (uint32_t u = 0; u < step->n_gathered; ++u) {
            const lq4_step_range& rg = step->gathered[u];
            if (!in_payload(rg.start, rg.count)) return fail(LQ4_ERR_SHAPE, "a gathered range lies outside the step buffer's payload");
            sa.range_begin[u] = (uint32_t)(rg.start - payload);
            sa.range_count[u] = (uint32_t)rg.count;
        }
        sa.n_ranges = step->n_gathered;
        if (world > 1) {
            // every output must come back: what a peer wrote is only in the mailbox until the gather moves it
            for (uint32_t i = 0; i < np; ++i) {
                bool covered = false;
                for (uint32_t u = 0; u < sa.n_ranges; ++u)
                    covered = covered || (sa.p[i].y_slot >= sa.range_begin[u] && sa.p[i].y_slot + sa.p[i].n <= sa.range_begin[u] + sa.range_count[u]);
                if (!covered) return fail(LQ4_ERR_SHAPE, "N-sharded step: every output must lie inside a gathered range");
            }
        }
    }
    LQ4_CUDA(launch_decode_step(sa, smem, grid, s));
    ctx->launches += 1;
    // keep the plan for the next call (the workspace may have grown while it was made: take the generation as it is now)
    if (!ctx->step_plan) ctx->step_plan = new StepPlan();
    const size_t gen_at = sizeof(ngroups) + sizeof(uint32_t) * ngroups + sizeof(ctx->pdl);
    memcpy(key.data() + gen_at, &ctx->alloc_gen, sizeof(ctx->alloc_gen));
    ctx->step_plan->key = key;
    ctx->step_plan->args = sa;
    ctx->step_plan->smem = smem;
    ctx->step_plan->grid = grid;
    return LQ4_OK;
}

}  // namespace

namespace {

// Copies up to kStepMaxProblems segments (whole 16-byte words) with plain loads and stores: the sources may be
// page-locked host memory.  The dependent launch (the step kernel) is released at once; it waits for this grid
// to complete before it reads an activation.
struct StageArgs {
    const uint4* src[kStepMaxProblems];
    uint4* dst[kStepMaxProblems];
    uint32_t words[kStepMaxProblems];
    uint32_t count;
};
__global__ void __launch_bounds__(256) stage_in_kernel(const __grid_constant__ StageArgs a) {
    pdl_launch_dependents();
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x, nt = gridDim.x * blockDim.x;
    for (uint32_t sgi = 0; sgi < a.count; ++sgi) {
        const uint4* src = a.src[sgi];
        uint4* dst = a.dst[sgi];
        for (uint32_t i = tid; i < a.words[sgi]; i += nt) {
            uint4 v;
            // host memory can change between launches: a load that no cache of this GPU keeps
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i) : "memory");
            dst[i] = v;
        }
    }
}

lq4_status collect_step(const lq4_step_group* groups, uint32_t ngroups, StepSpec* specs, uint32_t* gsize) {
    if (ngroups > (uint32_t)kStepMaxGroups) return fail(LQ4_ERR_NOSPACE, "a step holds at most 8 groups");
    uint32_t np = 0;
    for (uint32_t g = 0; g < ngroups; ++g) {
        if (groups[g].count && !groups[g].args) return fail(LQ4_ERR_NULL, "a group's args is NULL");
        if (groups[g].count == 0) return fail(LQ4_ERR_SHAPE, "a group is empty");
        if (np + groups[g].count > (uint32_t)kStepMaxProblems) return fail(LQ4_ERR_NOSPACE, "a step holds at most 24 projections");
        for (uint32_t i = 0; i < groups[g].count; ++i) { specs[np].a = groups[g].args[i]; specs[np].x_mul = nullptr; ++np; }
        gsize[g] = groups[g].count;
    }
    return LQ4_OK;
}

}  // namespace

lq4_status lq4_decode_step(lq4_ctx* ctx, const lq4_step_group* groups, uint32_t ngroups, const lq4_step_desc* step,
                           void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (ngroups == 0) return LQ4_OK;
    if (!groups) return fail(LQ4_ERR_NULL, "groups is NULL");
    StepSpec specs[kStepMaxProblems];
    uint32_t gsize[kStepMaxGroups];
    lq4_status st;
    if ((st = collect_step(groups, ngroups, specs, gsize))) return st;
    return step_core(ctx, specs, gsize, ngroups, step, (cudaStream_t)stream);
}

lq4_status lq4_decode_step_host(lq4_ctx* ctx, const lq4_step_group* groups, uint32_t ngroups, const lq4_step_desc* step,
                                void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (ngroups == 0) return LQ4_OK;
    if (!groups) return fail(LQ4_ERR_NULL, "groups is NULL");
    StepSpec specs[kStepMaxProblems];
    uint32_t gsize[kStepMaxGroups];
    lq4_status st;
    if ((st = collect_step(groups, ngroups, specs, gsize))) return st;
    uint32_t np = 0;
    for (uint32_t g = 0; g < ngroups; ++g) np += gsize[g];
    cudaStream_t s = (cudaStream_t)stream;

    // the inputs outside the step buffer, each distinct (pointer, bytes) once
    const char* pay0 = nullptr;
    const char* pay1 = nullptr;
    if (step && step->bufs && step->bufs->rank < LQ4_MAX_PEERS && step->bufs->bases[step->bufs->rank]) {
        lq4_peer_buf info{};
        char* base = static_cast<char*>(step->bufs->bases[step->bufs->rank]);
        if (peer_buf_info(base, &info)) { pay0 = base + 256; pay1 = pay0 + info.payload_bytes; }
    }
    // Pageable host memory is not addressable by the device: refuse it here instead of faulting in a kernel.
    auto device_can_address = [](const void* p) {
        cudaPointerAttributes at{};
        if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
        return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeHost || at.type == cudaMemoryTypeManaged;
    };
    StageArgs sg{};
    size_t off[kStepMaxProblems], total = 0;
    int seg_of[kStepMaxProblems];
    for (uint32_t i = 0; i < np; ++i) {
        const lq4_linear_args& a = specs[i].a;
        seg_of[i] = -1;
        if (a.m == 0 || a.n == 0) continue;
        if (!a.x || !a.y) return fail(LQ4_ERR_NULL, "x and y must be non-NULL");
        if (!device_can_address(a.y) || !device_can_address(a.y + (a.n - 1)))
            return fail(LQ4_ERR_UNSUPPORTED, "y must be device memory or page-locked host memory (cudaHostAlloc / cudaHostRegister)");
        if (!aligned(a.x, 16) || a.k % 32 != 0) return fail(LQ4_ERR_ALIGN, "a step needs 16-byte aligned x and k % 32 == 0");
        const size_t bytes = (size_t)a.k * (a.x_dtype == LQ4_DTYPE_BF16 ? 2 : 4);
        const char* x0 = static_cast<const char*>(a.x);
        if (pay0 && x0 >= pay0 && x0 + bytes <= pay1) continue;      // written by an earlier group: read through the mailbox
        for (uint32_t j = 0; j < sg.count; ++j)
            if (sg.src[j] == reinterpret_cast<const uint4*>(a.x) && sg.words[j] == bytes / 16) seg_of[i] = (int)j;
        if (seg_of[i] < 0) {
            if (!device_can_address(x0) || !device_can_address(x0 + bytes - 1))
                return fail(LQ4_ERR_UNSUPPORTED, "x must be device memory or page-locked host memory (cudaHostAlloc / cudaHostRegister)");
            seg_of[i] = (int)sg.count;
            sg.src[sg.count] = reinterpret_cast<const uint4*>(a.x);
            sg.words[sg.count] = (uint32_t)(bytes / 16);
            off[sg.count] = total;
            total += (bytes + 255) / 256 * 256;
            ++sg.count;
        }
    }
    if (sg.count) {
        if ((st = ensure(ctx, ctx->hx, total, false, s))) return st;
        uint64_t words = 0;
        for (uint32_t j = 0; j < sg.count; ++j) {
            sg.dst[j] = reinterpret_cast<uint4*>(static_cast<char*>(ctx->hx.p) + off[j]);
            words += sg.words[j];
        }
        for (uint32_t i = 0; i < np; ++i)
            if (seg_of[i] >= 0) specs[i].a.x = sg.dst[seg_of[i]];
        const uint64_t blocks = (words + 255) / 256;
        stage_in_kernel<<<(unsigned)(blocks < 64 ? blocks : 64), 256, 0, s>>>(sg);
        LQ4_CUDA(cudaGetLastError());
        ctx->launches += 1;
    }
    return step_core(ctx, specs, gsize, ngroups, step, s);
}

lq4_status lq4_linear_host(lq4_ctx* ctx, const lq4_linear_args* a, void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (!a) return fail(LQ4_ERR_NULL, "args is NULL");
    if (a->gather || a->wait_gather) return fail(LQ4_ERR_UNSUPPORTED, "lq4_linear_host takes host buffers: no fused all-gather");
    if (a->m == 0 || a->n == 0) return LQ4_OK;
    if (!a->x || !a->y) return fail(LQ4_ERR_NULL, "x and y must be non-NULL");
    if (a->k == 0 || a->k % 32 != 0) return fail(LQ4_ERR_K, "k must be non-zero and divisible by 32");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t esz = a->x_dtype == LQ4_DTYPE_BF16 ? 2 : 4;
    const size_t xbytes = (size_t)a->m * a->k * esz, ybytes = (size_t)a->m * a->n * 4;
    lq4_status st;
    if ((st = ensure(ctx, ctx->hx, xbytes, false, s))) return st;
    if ((st = ensure(ctx, ctx->hy, ybytes, false, s))) return st;
    LQ4_CUDA(cudaMemcpyAsync(ctx->hx.p, a->x, xbytes, cudaMemcpyHostToDevice, s));
    lq4_linear_args d = *a;
    d.x = ctx->hx.p;
    d.y = (float*)ctx->hy.p;
    d.ldy = a->n;
    if ((st = lq4_linear(ctx, &d, stream))) return st;
    const uint64_t ldy = a->ldy ? a->ldy : a->n;
    if (ldy == a->n) {
        LQ4_CUDA(cudaMemcpyAsync(a->y, ctx->hy.p, ybytes, cudaMemcpyDeviceToHost, s));
    } else {
        LQ4_CUDA(cudaMemcpy2DAsync(a->y, ldy * 4, ctx->hy.p, (size_t)a->n * 4, (size_t)a->n * 4, a->m,
                                   cudaMemcpyDeviceToHost, s));
    }
    LQ4_CUDA(cudaStreamSynchronize(s));
    return LQ4_OK;
}

lq4_status lq4_mlp_block(lq4_ctx* ctx, const lq4_mlp_args* a, void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (!a) return fail(LQ4_ERR_NULL, "args is NULL");
    if (a->m == 0) return LQ4_OK;
    if (a->hidden == 0 || a->inter == 0) return fail(LQ4_ERR_SHAPE, "hidden and inter must be non-zero");
    if (a->hidden % 32 != 0 || a->inter % 32 != 0) return fail(LQ4_ERR_K, "hidden and inter must be divisible by 32");
    if (!a->x || !a->w_gate_up || !a->w_down || !a->y) return fail(LQ4_ERR_NULL, "x, w_gate_up, w_down and y must be non-NULL");
    if ((uint64_t)a->m * 2 * a->inter > 0xffffffffull) return fail(LQ4_ERR_OVERFLOW, "m * 2 * inter does not fit");
    cudaStream_t s = (cudaStream_t)stream;
    lq4_status st;
    float* gate_up = a->gate_up;
    if (!gate_up) {
        if ((st = ensure(ctx, ctx->mlp, (size_t)a->m * 2 * a->inter * 4, false, s))) return st;
        gate_up = (float*)ctx->mlp.p;
    }
    // 1. gate rows and up rows of the merged matrix, each with its own adapter, into the two halves of
    //    gate_up: two problems that share x, one launch where the shapes allow it
    lq4_linear_args g[2] = {};
    for (int i = 0; i < 2; ++i) {
        g[i].x = a->x; g[i].x_dtype = a->x_dtype;
        g[i].m = a->m; g[i].n = a->inter; g[i].k = a->hidden;
        g[i].w = a->w_gate_up + (size_t)i * a->inter * (a->hidden / 32) * 20;
        g[i].y = gate_up + (size_t)i * a->inter;
        g[i].ldy = 2ull * a->inter;
        g[i].lora = i == 0 ? a->lora_gate : a->lora_up;
        g[i].path = LQ4_PATH_AUTO;
    }
    // 2. down_proj on silu(gate) * up.  One token: the decode kernel gates its own input while it builds
    //    the activation limbs (and in the adapter's projection); otherwise a gating pass of its own.
    lq4_linear_args d = {};
    d.x = gate_up; d.x_dtype = LQ4_DTYPE_F32;
    d.m = a->m; d.n = a->hidden; d.k = a->inter;
    d.w = a->w_down; d.y = a->y; d.ldy = 0;
    d.lora = a->lora_down;
    d.rot = a->rot_down;
    d.path = LQ4_PATH_AUTO;
    if ((st = validate_linear(&d))) return st;          // all three projections are checked before the first launch
    for (int i = 0; i < 2; ++i)
        if ((st = validate_linear(&g[i]))) return st;
    // One token with the gate||up row in the library's own buffer: the whole block is ONE launch.  The row
    // lives in a step buffer, gate and up rows form the first group, down_proj the second; its CTAs read
    // silu(gate) * up through the mailbox as the values arrive (lq4_step.cu).
    if (a->m == 1 && !a->gate_up && !a->rot_down && ctx->mlp_one_launch && a->hidden % 128 == 0 && a->inter % 128 == 0 &&
        aligned(a->x, 16) && aligned(a->w_gate_up, 16) && aligned(a->w_down, 16) &&
        gemv_resident_fits(1, a->hidden > a->inter ? a->hidden : a->inter, false)) {
        bool lora_ok = true;
        for (const lq4_lora_desc* l : {a->lora_gate, a->lora_up, a->lora_down})
            lora_ok = lora_ok && (!l || (l->rank <= (uint32_t)kGemvMaxRank && aligned(l->a, 16)));
        const uint64_t need = 2ull * a->inter;
        // without room for the row and with growth disabled the block runs as two launches (below)
        if (lora_ok && !ctx->allow_grow && (!ctx->mlp_step || ctx->mlp_step->payload_bytes < need * 4)) lora_ok = false;
        if (lora_ok) {
            if (!ctx->mlp_step || ctx->mlp_step->payload_bytes < need * 4) {
                LQ4_CUDA(cudaStreamSynchronize(s));
                if (ctx->mlp_step) { lq4_peer_buf_free(ctx->mlp_step); ctx->mlp_step = nullptr; }
                if ((st = lq4_step_buf_create(need, &ctx->mlp_step))) return st;
            }
            float* row = static_cast<float*>(lq4_peer_buf_payload(ctx->mlp_step));
            StepSpec specs[3];
            for (int i = 0; i < 2; ++i) {
                specs[i].a = g[i];
                specs[i].a.y = row + (size_t)i * a->inter;
                specs[i].a.ldy = 0;
                specs[i].x_mul = nullptr;
            }
            specs[2].a = d;
            specs[2].a.x = row;
            specs[2].x_mul = row + a->inter;
            const uint32_t gsize[2] = {2, 1};
            lq4_gather_desc gd{};
            gd.world = 1; gd.rank = 0; gd.bases[0] = lq4_peer_buf_base(ctx->mlp_step);
            lq4_step_desc sd{};
            sd.bufs = &gd;
            return step_core(ctx, specs, gsize, 2, &sd, s);
        }
    }
    if ((st = lq4_linear_group(ctx, g, 2, stream))) return st;
    const uint32_t rank = d.lora ? d.lora->rank : 0;
    // up to 16 tokens: the decode kernels gate their own input (the resident kernel in its prologue, the dense
    // kernel's record builder for 2..16 tokens), so the gated vector is never written
    const bool fused = a->m <= (uint32_t)kGemvMaxM && !d.rot && d.k % 128 == 0 && aligned(d.w, 16) && aligned(gate_up, 16) &&
                       (!d.lora || aligned(d.lora->a, 16)) && rank <= (uint32_t)kGemvMaxRank &&
                       (a->m > 1 || gemv_resident_fits(1, d.k, false));
    if (fused)
        return run_gemv_mma(ctx, &d, gate_up, LQ4_DTYPE_F32, nullptr, a->m, d.y, d.n, s, gate_up + a->inter, true,
                            2 * a->inter);
    if ((st = ensure(ctx, ctx->mlp_h, (size_t)a->m * a->inter * 4, false, s))) return st;
    LQ4_CUDA(launch_silu_mul_rows(gate_up, a->m, a->inter, (float*)ctx->mlp_h.p, ctx->sm_count, s));
    ctx->launches += 1;
    d.x = ctx->mlp_h.p;
    return lq4_linear(ctx, &d, stream);
}

lq4_status lq4_logits_topk(lq4_ctx* ctx, const float* logits, uint32_t n, uint32_t top_k, lq4_topk_candidate* out,
                           void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (top_k == 0 || top_k > LQ4_MAX_TOP_K) return fail(LQ4_ERR_SHAPE, "top_k must be in 1..256");
    if (!logits || !out) return fail(LQ4_ERR_NULL, "logits and out must be non-NULL");
    if (n == 0) return fail(LQ4_ERR_SHAPE, "n must be non-zero");
    if (n > 0x7fffffffu) return fail(LQ4_ERR_OVERFLOW, "n does not fit");
    cudaStream_t s = (cudaStream_t)stream;
    lq4_status st;
    if ((st = ensure(ctx, ctx->topk, topk_list_bytes(n, top_k), false, s))) return st;
    if ((st = ensure(ctx, ctx->topk_ctr, topk_counter_bytes(n), true, s))) return st;      // zero once; launches keep it zero
    int nl = 0;
    LQ4_CUDA(launch_topk(logits, n, top_k, ctx->topk.p, (uint32_t*)ctx->topk_ctr.p, out, ctx->pdl, s, &nl));
    ctx->launches += nl;
    return LQ4_OK;
}

lq4_status lq4_lm_head_topk(lq4_ctx* ctx, const lq4_linear_args* a, uint32_t top_k, lq4_topk_candidate* out,
                            void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (!a) return fail(LQ4_ERR_NULL, "args is NULL");
    if (top_k == 0 || top_k > LQ4_MAX_TOP_K) return fail(LQ4_ERR_SHAPE, "top_k must be in 1..256");
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    if (a->m != 1) return fail(LQ4_ERR_SHAPE, "lq4_lm_head_topk takes one token (m == 1)");
    if (a->n == 0) return fail(LQ4_ERR_SHAPE, "n must be non-zero");
    if (a->gather || a->wait_gather) return fail(LQ4_ERR_UNSUPPORTED, "lq4_lm_head_topk has no fused all-gather");
    cudaStream_t s = (cudaStream_t)stream;
    lq4_linear_args b = *a;
    lq4_status st;
    if (!b.y) {
        if ((st = ensure(ctx, ctx->logits, (size_t)a->n * 4, false, s))) return st;
        b.y = (float*)ctx->logits.p;
        b.ldy = 0;
    }
    if ((st = lq4_linear(ctx, &b, stream))) return st;
    return lq4_logits_topk(ctx, b.y, a->n, top_k, out, stream);
}

lq4_status lq4_lora_apply(lq4_ctx* ctx, const void* x, int32_t x_dtype, uint32_t m, uint32_t k, float* y, uint32_t n,
                          uint64_t ldy, const lq4_lora_desc* lora, void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (!lora) return LQ4_OK;   // no adapter for this projection: no-op, as in the reference
    if (m == 0 || n == 0) return LQ4_OK;
    if (!x || !y || !lora->a || !lora->b) return fail(LQ4_ERR_NULL, "x, y and the LoRA factors must be non-NULL");
    if (lora->rank == 0 || !std::isfinite(lora->scale)) return fail(LQ4_ERR_LORA, "rank 0 or non-finite scale");
    if (k == 0) return fail(LQ4_ERR_K, "k must be non-zero");
    if (x_dtype != LQ4_DTYPE_F32 && x_dtype != LQ4_DTYPE_BF16) return fail(LQ4_ERR_DTYPE, "unknown x_dtype");
    cudaStream_t s = (cudaStream_t)stream;
    if (ldy == 0) ldy = n;
    lq4_status st;
    if ((st = ensure(ctx, ctx->t, (size_t)m * lora->rank * 4, false, s))) return st;
    launch_lora_t(x, x_dtype, m, k, lora->a, lora->rank, (float*)ctx->t.p, s);
    launch_gemv_generic(x, x_dtype, nullptr, y, ldy, m, n, k, (const float*)ctx->t.p, lora->b, lora->rank,
                        lora->scale, 1, s);
    ctx->launches += 2;
    LQ4_CUDA(cudaGetLastError());
    return LQ4_OK;
}

lq4_status lq4_dequant_f32(const uint8_t* payload, uint64_t n_blocks, float* out, void* stream) {
    if (n_blocks == 0) return LQ4_OK;
    if (!payload || !out) return fail(LQ4_ERR_NULL, "payload and out must be non-NULL");
    if (!aligned(payload, 4) || !aligned(out, 16)) return fail(LQ4_ERR_ALIGN, "payload needs 4-byte, out 16-byte alignment");
    int dev = 0, sms = 0;
    LQ4_CUDA(cudaGetDevice(&dev));
    LQ4_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    launch_dequant(payload, n_blocks, out, sms, (cudaStream_t)stream);
    LQ4_CUDA(cudaGetLastError());
    return LQ4_OK;
}

lq4_status lq4_quantize_f32(const float* data, uint64_t len, int32_t mode, uint8_t* payload, int32_t* status_out,
                            void* stream) {
    if (len == 0) return LQ4_OK;
    if (!data || !payload) return fail(LQ4_ERR_NULL, "data and payload must be non-NULL");
    if (mode != LQ4_QUANT_ASYMMETRIC && mode != LQ4_QUANT_SYMMETRIC) return fail(LQ4_ERR_UNSUPPORTED, "unknown mode");
    if (!aligned(payload, 4) || !aligned(data, 4)) return fail(LQ4_ERR_ALIGN, "data and payload need 4-byte alignment");
    int dev = 0, sms = 0;
    LQ4_CUDA(cudaGetDevice(&dev));
    LQ4_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    launch_quantize(data, LQ4_DTYPE_F32, 1, len, mode == LQ4_QUANT_SYMMETRIC, payload, status_out, sms, (cudaStream_t)stream);
    LQ4_CUDA(cudaGetLastError());
    return LQ4_OK;
}

lq4_status lq4_quantize_tensor(const void* data, int32_t dtype, uint64_t rows, uint64_t cols, int32_t per_row,
                               int32_t mode, uint8_t* payload, int32_t* status_out, void* stream) {
    if (mul_overflows(rows, cols, (uint64_t)1 << 48))
        return fail(LQ4_ERR_OVERFLOW, "Q4 tensor shape overflows the supported element count");   // checked first, as the reference does
    if (rows == 0 || cols == 0) return LQ4_OK;
    if (!data || !payload) return fail(LQ4_ERR_NULL, "data and payload must be non-NULL");
    if (mode != LQ4_QUANT_ASYMMETRIC && mode != LQ4_QUANT_SYMMETRIC) return fail(LQ4_ERR_UNSUPPORTED, "unknown mode");
    size_t esz;
    switch (dtype) {
        case LQ4_DTYPE_F32: esz = 4; break;
        case LQ4_DTYPE_BF16: esz = 2; break;
        case LQ4_DTYPE_F64: esz = 8; break;
        default: return fail(LQ4_ERR_DTYPE, "unknown dtype");
    }
    if (!aligned(payload, 4) || !aligned(data, esz)) return fail(LQ4_ERR_ALIGN, "payload needs 4-byte alignment, data its element alignment");
    int dev = 0, sms = 0;
    LQ4_CUDA(cudaGetDevice(&dev));
    LQ4_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (per_row) launch_quantize(data, dtype, rows, cols, mode == LQ4_QUANT_SYMMETRIC, payload, status_out, sms, (cudaStream_t)stream);
    else launch_quantize(data, dtype, 1, rows * cols, mode == LQ4_QUANT_SYMMETRIC, payload, status_out, sms, (cudaStream_t)stream);
    LQ4_CUDA(cudaGetLastError());
    return LQ4_OK;
}

static lq4_status check_absorb(const void* w, int32_t dtype, uint64_t rows, uint64_t cols, const lq4_rot_desc* rot,
                               uint64_t must_match, const char* which) {
    if (mul_overflows(rows, cols, (uint64_t)1 << 48)) return fail(LQ4_ERR_OVERFLOW, "rows*cols overflow");   // rotation.rs:64-68
    if (!rot || !rot->signs) return fail(LQ4_ERR_NULL, "rot and rot->signs must be non-NULL");
    if (dtype != LQ4_DTYPE_F32 && dtype != LQ4_DTYPE_F64) return fail(LQ4_ERR_DTYPE, "absorption takes f32 or f64 weights");
    if (!is_pow2(rot->dim)) return fail(LQ4_ERR_ROT, "rotation needs a power-of-two dim");
    if ((uint64_t)rot->dim != must_match)
        return fail(LQ4_ERR_ROT, std::string("rotation.dim()=") + std::to_string(rot->dim) + " but weight." + which + "=" + std::to_string(must_match));
    if (rows && cols && !w) return fail(LQ4_ERR_NULL, "w is NULL");
    if (!aligned(w, dtype == LQ4_DTYPE_F64 ? 8 : 4)) return fail(LQ4_ERR_ALIGN, "w needs its element alignment");
    return LQ4_OK;
}

lq4_status lq4_absorb_input_rotation(void* w, int32_t dtype, uint64_t rows, uint64_t cols, const lq4_rot_desc* rot,
                                     void* stream) {
    lq4_status st = check_absorb(w, dtype, rows, cols, rot, cols, "cols");
    if (st) return st;
    if ((uint64_t)rot->dim * (dtype == LQ4_DTYPE_F64 ? 8 : 4) > 128 * 1024)
        return fail(LQ4_ERR_UNSUPPORTED, "row rotation stages the row in shared memory: dim <= 16384 (f64) or 32768 (f32)");
    LQ4_CUDA(launch_absorb_input(w, dtype, rows, rot->dim, rot->signs, (cudaStream_t)stream));
    return LQ4_OK;
}

lq4_status lq4_absorb_output_rotation(void* w, int32_t dtype, uint64_t rows, uint64_t cols, const lq4_rot_desc* rot,
                                      void* stream) {
    lq4_status st = check_absorb(w, dtype, rows, cols, rot, rows, "rows");
    if (st) return st;
    int dev = 0, sms = 0;
    LQ4_CUDA(cudaGetDevice(&dev));
    LQ4_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    LQ4_CUDA(launch_absorb_output(w, dtype, rot->dim, cols, rot->signs, sms, (cudaStream_t)stream));
    return LQ4_OK;
}

lq4_status lq4_q4_file_write(const char* h_path, const uint64_t* h_shape, uint32_t ndim, uint64_t original_len,
                             const uint8_t* payload, void* stream) {
    if (!h_path || !h_shape) return fail(LQ4_ERR_NULL, "path and shape must be non-NULL");
    if (ndim == 0 || ndim > 8) return fail(LQ4_ERR_SHAPE, "ndim must be 1..8");
    uint64_t prod = 1;
    for (uint32_t i = 0; i < ndim; ++i) {
        if (mul_overflows(prod, h_shape[i], (uint64_t)1 << 48)) return fail(LQ4_ERR_OVERFLOW, "shape product overflows");
        prod *= h_shape[i];
    }
    if (prod != original_len) return fail(LQ4_ERR_SHAPE, "shape product does not equal original_len");
    const uint64_t nb = (original_len + 31) / 32;
    if (nb && !payload) return fail(LQ4_ERR_NULL, "payload is NULL");
    std::vector<uint8_t> host((size_t)nb * 20);
    cudaStream_t s = (cudaStream_t)stream;
    if (nb) {
        LQ4_CUDA(cudaMemcpyAsync(host.data(), payload, host.size(), cudaMemcpyDeviceToHost, s));
        LQ4_CUDA(cudaStreamSynchronize(s));
    }
    FILE* f = fopen(h_path, "wb");
    if (!f) return fail(LQ4_ERR_IO, std::string("cannot create ") + h_path);
    const uint32_t ver = 2;
    bool ok = fwrite("KHQ4", 1, 4, f) == 4 && fwrite(&ver, 4, 1, f) == 1 && fwrite(&ndim, 4, 1, f) == 1;
    for (uint32_t i = 0; ok && i < ndim; ++i) ok = fwrite(&h_shape[i], 8, 1, f) == 1;
    ok = ok && fwrite(&original_len, 8, 1, f) == 1;
    ok = ok && (host.empty() || fwrite(host.data(), 1, host.size(), f) == host.size());
    ok = (fclose(f) == 0) && ok;
    if (!ok) return fail(LQ4_ERR_IO, std::string("short write to ") + h_path);
    return LQ4_OK;
}

lq4_status lq4_hadamard_rows(const float* x, float* out, uint32_t rows, const lq4_rot_desc* rot, void* stream) {
    if (rows == 0) return LQ4_OK;
    if (!x || !out || !rot || !rot->signs) return fail(LQ4_ERR_NULL, "x, out and rot->signs must be non-NULL");
    if (!is_pow2(rot->dim) || rot->dim > 16384) return fail(LQ4_ERR_ROT, "rotation needs a power-of-two dim <= 16384");
    LQ4_CUDA(launch_hadamard_rows(x, LQ4_DTYPE_F32, rot->signs, rot->dim, rows, out, (cudaStream_t)stream));
    return LQ4_OK;
}

static lq4_status check_block_rotation(uint32_t n, uint32_t block) {
    // BlockHadamard::new, crates/inference/src/quant/quarot/hadamard.rs:358-400
    if (n == 0 || n > LQ4_MAX_ROT_LEN) return fail(LQ4_ERR_ROT, "block rotation needs 0 < n <= 1 << 24");
    if (!is_pow2(block)) return fail(LQ4_ERR_ROT, "block rotation needs a power-of-two block size");
    if (n % block != 0) return fail(LQ4_ERR_ROT, "block size does not divide n");
    if (n / block > LQ4_MAX_ROT_BLOCKS) return fail(LQ4_ERR_ROT, "more than 4096 rotation blocks");
    return LQ4_OK;
}

lq4_status lq4_block_hadamard_rows(const float* x, float* out, uint32_t rows, uint32_t n, const lq4_rot_desc* rot,
                                   void* stream) {
    if (!x || !out || !rot || !rot->signs) return fail(LQ4_ERR_NULL, "x, out and rot->signs must be non-NULL");
    lq4_status st;
    if ((st = check_block_rotation(n, rot->dim))) return st;
    if (rot->dim > 16384) return fail(LQ4_ERR_ROT, "block size above 16384");
    if (rows == 0) return LQ4_OK;
    const uint64_t launch_rows = (uint64_t)rows * (n / rot->dim);
    if (launch_rows > 0x7fffffffull) return fail(LQ4_ERR_OVERFLOW, "rows * blocks does not fit");
    LQ4_CUDA(launch_hadamard_rows(x, LQ4_DTYPE_F32, rot->signs, rot->dim, (uint32_t)launch_rows, out, (cudaStream_t)stream,
                                  n / rot->dim));
    return LQ4_OK;
}

lq4_status lq4_cross_head_hadamard_rows(const float* x, float* out, uint32_t rows, uint32_t num_heads,
                                        uint32_t head_dim, const float* signs, void* stream) {
    if (!x || !out || !signs) return fail(LQ4_ERR_NULL, "x, out and signs must be non-NULL");
    if (!is_pow2(num_heads) || num_heads > 128) return fail(LQ4_ERR_ROT, "num_heads must be a power of two <= 128");
    if (head_dim == 0) return fail(LQ4_ERR_ROT, "head_dim must be non-zero");
    if ((uint64_t)num_heads * head_dim > LQ4_MAX_ROT_LEN) return fail(LQ4_ERR_ROT, "num_heads * head_dim above 1 << 24");
    if ((uint64_t)rows * head_dim > 0x7fffffffull * 128) return fail(LQ4_ERR_OVERFLOW, "rows * head_dim does not fit");
    LQ4_CUDA(launch_cross_head_rows(x, signs, num_heads, head_dim, rows, out, (cudaStream_t)stream));
    return LQ4_OK;
}

lq4_status lq4_block_rot_signs_from_seed(uint64_t seed, uint32_t n, uint32_t block, float* signs, void* stream) {
    lq4_status st;
    if ((st = check_block_rotation(n, block))) return st;
    if (!signs) return fail(LQ4_ERR_NULL, "signs is NULL");
    launch_block_rot_signs(seed, n, block, signs, (cudaStream_t)stream);
    LQ4_CUDA(cudaGetLastError());
    return LQ4_OK;
}

lq4_status lq4_rot_signs_from_seed(uint64_t seed, uint32_t dim, float* signs, void* stream) {
    if (dim == 0) return LQ4_OK;
    if (!signs) return fail(LQ4_ERR_NULL, "signs is NULL");
    launch_rot_signs(seed, dim, signs, (cudaStream_t)stream);
    LQ4_CUDA(cudaGetLastError());
    return LQ4_OK;
}

// ---- resident objects ---------------------------------------------------------

static float f16_bits_to_f32_host(uint16_t h) {
    const uint32_t sign = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1f, f = h & 0x3ff;
    uint32_t bits;
    if (e == 0) {
        if (f == 0) bits = sign;
        else {
            int ue = -14;
            uint32_t m = f;
            while (!(m & 0x400)) { m <<= 1; --ue; }
            bits = sign | ((uint32_t)(ue + 127) << 23) | ((m & 0x3ff) << 13);
        }
    } else if (e == 0x1f) bits = sign | 0x7f800000u | (f << 13);
    else bits = sign | ((e + 112) << 23) | (f << 13);
    float v;
    memcpy(&v, &bits, 4);
    return v;
}

static lq4_status check_blocks(const uint8_t* payload, uint64_t n_blocks) {
    for (uint64_t b = 0; b < n_blocks; ++b) {
        uint16_t sb, bb;
        memcpy(&sb, payload + b * 20, 2);
        memcpy(&bb, payload + b * 20 + 2, 2);
        const float sc = f16_bits_to_f32_host(sb), bi = f16_bits_to_f32_host(bb);
        if (!(std::isfinite(sc) && sc > 0.0f) || !std::isfinite(bi))
            return fail(LQ4_ERR_BAD_BLOCK, "block " + std::to_string(b) + " has a non-finite or non-positive scale, or a non-finite bias");
    }
    return LQ4_OK;
}

lq4_status lq4_weights_upload(const uint8_t* h_payload, uint64_t n, uint64_t k, lq4_weights** out) {
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    *out = nullptr;
    if (!h_payload) return fail(LQ4_ERR_NULL, "payload is NULL");
    if (k == 0 || k % 32 != 0) return fail(LQ4_ERR_K, "k must be non-zero and divisible by 32");
    if (n == 0) return fail(LQ4_ERR_SHAPE, "n must be non-zero");
    if (mul_overflows(n, k / 32, ((uint64_t)1 << 40) / 20)) return fail(LQ4_ERR_OVERFLOW, "payload too large");
    const uint64_t nb = n * (k / 32);
    lq4_status st = check_blocks(h_payload, nb);   // before the bytes are published to the GPU
    if (st) return st;
    lq4_weights* w = new lq4_weights();
    w->rows = n; w->cols = k;
    cudaGetDevice(&w->device);
    cudaError_t e = cudaMalloc(&w->payload, nb * 20 + 256);
    if (e == cudaSuccess) e = cudaMemcpy(w->payload, h_payload, nb * 20, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        if (w->payload) cudaFree(w->payload);
        delete w;
        return cuda_fail(e, "weights upload");
    }
    *out = w;
    return LQ4_OK;
}

lq4_status lq4_weights_load_q4_file(const char* h_path, const uint64_t* h_expected_shape, uint32_t expected_ndim,
                                    lq4_weights** out) {
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    *out = nullptr;
    if (!h_path) return fail(LQ4_ERR_NULL, "path is NULL");
    FILE* f = fopen(h_path, "rb");
    if (!f) return fail(LQ4_ERR_IO, std::string("cannot open ") + h_path);
    std::vector<uint8_t> img;
    fseek(f, 0, SEEK_END);
    const long len = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (len < 0) { fclose(f); return fail(LQ4_ERR_IO, "cannot size file"); }
    img.resize((size_t)len);
    const size_t got = len ? fread(img.data(), 1, (size_t)len, f) : 0;
    fclose(f);
    if (got != (size_t)len) return fail(LQ4_ERR_IO, "short read");
    if (img.size() < 12 || memcmp(img.data(), "KHQ4", 4) != 0) return fail(LQ4_ERR_FORMAT, "invalid magic: not a .q4 file");
    uint32_t ver, ndim;
    memcpy(&ver, img.data() + 4, 4);
    memcpy(&ndim, img.data() + 8, 4);
    if (ver == 1) return fail(LQ4_ERR_FORMAT, "legacy .q4 file (v1 symmetric 18-byte blocks): re-quantize");
    if (ver != 2) return fail(LQ4_ERR_FORMAT, "unsupported .q4 version " + std::to_string(ver));
    if (ndim == 0 || ndim > 8 || img.size() < 20 + 8ull * ndim) return fail(LQ4_ERR_FORMAT, "bad ndim or truncated header");
    std::vector<uint64_t> shape(ndim);
    uint64_t prod = 1;
    for (uint32_t i = 0; i < ndim; ++i) {
        memcpy(&shape[i], img.data() + 12 + 8 * i, 8);
        if (mul_overflows(prod, shape[i], (uint64_t)1 << 48)) return fail(LQ4_ERR_OVERFLOW, "shape product overflows");
        prod *= shape[i];
    }
    uint64_t original_len;
    memcpy(&original_len, img.data() + 12 + 8 * ndim, 8);
    const uint64_t off = 20 + 8ull * ndim, nb = (original_len + 31) / 32;
    if (prod != original_len) return fail(LQ4_ERR_SHAPE, "shape product does not equal original_len");
    if (img.size() < off + nb * 20) return fail(LQ4_ERR_FORMAT, "file truncated below the Q4 block payload");
    if (img.size() > off + nb * 20) return fail(LQ4_ERR_FORMAT, "file has trailing bytes after the Q4 block payload");
    if (expected_ndim) {
        if (expected_ndim != ndim) return fail(LQ4_ERR_SHAPE, "rank differs from the expected shape");
        for (uint32_t i = 0; i < ndim; ++i)
            if (h_expected_shape[i] != shape[i]) return fail(LQ4_ERR_SHAPE, "shape differs from the expected shape");
    }
    if (ndim != 2) return fail(LQ4_ERR_UNSUPPORTED, "a linear layer needs a 2-D tensor");
    if (shape[1] == 0 || shape[1] % 32 != 0) return fail(LQ4_ERR_K, "row length must be a non-zero multiple of 32");
    return lq4_weights_upload(img.data() + off, shape[0], shape[1], out);
}

const uint8_t* lq4_weights_payload(const lq4_weights* w) { return w ? w->payload : nullptr; }
uint64_t lq4_weights_rows(const lq4_weights* w) { return w ? w->rows : 0; }
uint64_t lq4_weights_cols(const lq4_weights* w) { return w ? w->cols : 0; }
void lq4_weights_free(lq4_weights* w) {
    if (!w) return;
    if (w->payload) cudaFree(w->payload);
    delete w;
}

lq4_status lq4_lora_upload(const float* h_a, uint64_t a_len, const float* h_b, uint64_t b_len, uint64_t rank,
                           uint64_t d_in, uint64_t d_out, float scale, lq4_lora** out) {
    if (!out) return fail(LQ4_ERR_NULL, "out is NULL");
    *out = nullptr;
    if (!h_a || !h_b) return fail(LQ4_ERR_NULL, "A and B must be non-NULL");
    if (!std::isfinite(scale)) return fail(LQ4_ERR_LORA, "scale must be finite");
    if (rank == 0) return fail(LQ4_ERR_LORA, "rank=0");
    if (d_in == 0 || d_out == 0) return fail(LQ4_ERR_LORA, "zero dimension");
    if (rank > UINT32_MAX || d_in > UINT32_MAX || d_out > UINT32_MAX) return fail(LQ4_ERR_OVERFLOW, "rank, d_in or d_out exceeds u32");
    if (mul_overflows(rank, d_in, UINT64_MAX / 4) || mul_overflows(d_out, rank, UINT64_MAX / 4))
        return fail(LQ4_ERR_OVERFLOW, "rank*d_in or d_out*rank overflows");
    if (a_len != rank * d_in) return fail(LQ4_ERR_LORA, "A length != rank*d_in");
    if (b_len != d_out * rank) return fail(LQ4_ERR_LORA, "B length != d_out*rank");
    lq4_lora* l = new lq4_lora();
    l->rank = rank; l->d_in = d_in; l->d_out = d_out; l->scale = scale;
    cudaError_t e = cudaMalloc(&l->a, a_len * 4);
    if (e == cudaSuccess) e = cudaMalloc(&l->b, b_len * 4);
    if (e == cudaSuccess) e = cudaMemcpy(l->a, h_a, a_len * 4, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(l->b, h_b, b_len * 4, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        lq4_lora_free(l);
        return cuda_fail(e, "lora upload");
    }
    *out = l;
    return LQ4_OK;
}

lq4_status lq4_lora_desc_for_rows(const lq4_lora* l, uint64_t n0, uint64_t n1, lq4_lora_desc* desc) {
    if (!l || !desc) return fail(LQ4_ERR_NULL, "lora and desc must be non-NULL");
    if (n0 > n1 || n1 > l->d_out) return fail(LQ4_ERR_SHAPE, "row range outside [0, d_out]");
    desc->a = l->a;
    desc->b = l->b + n0 * l->rank;
    desc->rank = (uint32_t)l->rank;
    desc->scale = l->scale;
    return LQ4_OK;
}

void lq4_lora_free(lq4_lora* l) {
    if (!l) return;
    if (l->a) cudaFree(l->a);
    if (l->b) cudaFree(l->b);
    delete l;
}

lq4_status lq4_shard_plan(uint64_t n, uint64_t k, uint32_t world, uint32_t rank, uint64_t* n0, uint64_t* n1,
                          uint64_t* byte_offset) {
    if (!n0 || !n1 || !byte_offset) return fail(LQ4_ERR_NULL, "output pointers must be non-NULL");
    if (world == 0 || rank >= world) return fail(LQ4_ERR_SHAPE, "rank must be below world");
    if (k == 0 || k % 32 != 0) return fail(LQ4_ERR_K, "k must be non-zero and divisible by 32");
    *n0 = n * rank / world;
    *n1 = n * (rank + 1) / world;
    *byte_offset = *n0 * (k / 32) * 20;
    return LQ4_OK;
}

// ---- N-sharded linear over NCCL ------------------------------------------------------------------
}  // extern "C"

namespace {

// The handful of NCCL entry points this path needs, bound at run time so that the library loads (and
// every other entry point works) on a machine without NCCL.  Types follow NCCL's public C API.
struct NcclId { char internal[LQ4_NCCL_ID_BYTES]; };
typedef void* NcclComm;
constexpr int kNcclFloat = 7;       // ncclFloat32
struct NcclApi {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};

const NcclApi& nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // the copy the process already holds (a framework's bundled NCCL) first, then the system's
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        auto sym = [&](const char* name) { return dlsym(h, name); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.Broadcast &&
                 api.GroupStart && api.GroupEnd && api.GetErrorString;
    });
    return api;
}

lq4_status nccl_fail(int rc, const char* what) {
    return fail(LQ4_ERR_CUDA, std::string(what) + ": NCCL: " + nccl_api().GetErrorString(rc));
}
#define LQ4_NCCL(call)                                   \
    do {                                                 \
        int rc__ = (call);                               \
        if (rc__ != 0) return nccl_fail(rc__, #call);    \
    } while (0)

// NCCL delivers block b as [rank][rows][n_r] (rank-major); y_full wants [rows][n_total] (row-major).
// One thread per four output floats of a row; every global access is a coalesced 16-byte one when the
// slice widths and the row pitch are multiples of four floats, a 4-byte one otherwise.
__global__ void __launch_bounds__(256) place_slices_kernel(const float* __restrict__ recv, float* __restrict__ y,
                                                           uint64_t ldy, uint32_t rows, uint64_t n_total, uint32_t world,
                                                           int vec4) {
    // slice r covers columns [n_total * r / world, n_total * (r + 1) / world)
    const uint64_t per_row = vec4 ? n_total / 4 : n_total;
    const uint64_t total = per_row * rows;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / per_row, c = (i - row * per_row) * (vec4 ? 4 : 1);
        uint32_t r = (uint32_t)(((c + 1) * world - 1) / n_total);          // owner of column c
        while (n_total * r / world > c) --r;
        while (n_total * (r + 1) / world <= c) ++r;
        const uint64_t n0 = n_total * r / world, n1 = n_total * (r + 1) / world;
        const float* src = recv + n0 * rows + row * (n1 - n0) + (c - n0);     // blocks of earlier ranks hold n0 * rows floats
        float* dst = y + row * ldy + c;
        if (vec4) *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
        else *dst = *src;
    }
}

cudaError_t place_slices(const float* gathered, float* y, uint64_t ldy, uint32_t rows, uint64_t n_total, uint32_t world,
                         int sm_count, cudaStream_t s) {
    const int vec4 = (n_total % ((uint64_t)4 * world) == 0 && ldy % 4 == 0 && aligned(y, 16) && aligned(gathered, 16)) ? 1 : 0;
    const uint64_t work = (vec4 ? n_total / 4 : n_total) * rows;
    const uint64_t want = (work + 255) / 256, cap_blocks = (uint64_t)sm_count * 8;
    place_slices_kernel<<<(unsigned)(want < cap_blocks ? want : cap_blocks), 256, 0, s>>>(gathered, y, ldy, rows, n_total, world, vec4);
    return cudaGetLastError();
}

}  // namespace

extern "C" {

lq4_status lq4_nccl_unique_id(uint8_t* h_id_out) {
    if (!h_id_out) return fail(LQ4_ERR_NULL, "id_out is NULL");
    const NcclApi& nc = nccl_api();
    if (!nc.ok) return fail(LQ4_ERR_UNSUPPORTED, "no NCCL library (libnccl.so.2) could be loaded");
    NcclId id;
    LQ4_NCCL(nc.GetUniqueId(&id));
    memcpy(h_id_out, &id, sizeof(id));
    return LQ4_OK;
}

lq4_status lq4_nccl_comm_create(const uint8_t* h_id, uint32_t world, uint32_t rank, void** comm_out) {
    if (!comm_out) return fail(LQ4_ERR_NULL, "comm_out is NULL");
    *comm_out = nullptr;
    if (!h_id) return fail(LQ4_ERR_NULL, "id is NULL");
    if (world == 0 || rank >= world) return fail(LQ4_ERR_SHAPE, "rank must be below world");
    const NcclApi& nc = nccl_api();
    if (!nc.ok) return fail(LQ4_ERR_UNSUPPORTED, "no NCCL library (libnccl.so.2) could be loaded");
    NcclId id;
    memcpy(&id, h_id, sizeof(id));
    NcclComm comm = nullptr;
    LQ4_NCCL(nc.CommInitRank(&comm, (int)world, id, (int)rank));
    *comm_out = comm;
    return LQ4_OK;
}

void lq4_nccl_comm_destroy(void* comm) {
    if (comm && nccl_api().ok) nccl_api().CommDestroy(comm);
}

lq4_status lq4_place_slices(const float* gathered, float* y_full, uint64_t ldy_full, uint32_t rows, uint64_t n_total,
                            uint32_t world, void* stream) {
    if (rows == 0 || n_total == 0) return LQ4_OK;
    if (!gathered || !y_full) return fail(LQ4_ERR_NULL, "gathered and y_full must be non-NULL");
    if (world == 0) return fail(LQ4_ERR_SHAPE, "world must be non-zero");
    const uint64_t ldy = ldy_full ? ldy_full : n_total;
    if (ldy < n_total) return fail(LQ4_ERR_SHAPE, "ldy_full is smaller than n_total");
    if (!aligned(gathered, 4) || !aligned(y_full, 4)) return fail(LQ4_ERR_ALIGN, "buffers need 4-byte alignment");
    int dev = 0, sms = 0;
    LQ4_CUDA(cudaGetDevice(&dev));
    LQ4_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    LQ4_CUDA(place_slices(gathered, y_full, ldy, rows, n_total, world, sms, (cudaStream_t)stream));
    return LQ4_OK;
}

lq4_status lq4_linear_sharded(lq4_ctx* ctx, const lq4_linear_args* local, const lq4_shard_desc* sh, void* stream) {
    if (!ctx) return fail(LQ4_ERR_NULL, "ctx is NULL");
    if (!local || !sh) return fail(LQ4_ERR_NULL, "local and shard must be non-NULL");
    if (sh->world == 0 || sh->rank >= sh->world) return fail(LQ4_ERR_SHAPE, "shard: rank must be below world");
    if (local->gather || local->wait_gather) return fail(LQ4_ERR_UNSUPPORTED, "lq4_linear_sharded gathers over NCCL: no fused all-gather fields");
    if (local->m == 0 || sh->n_total == 0) return LQ4_OK;
    if (local->k == 0 || local->k % 32 != 0) return fail(LQ4_ERR_K, "k must be non-zero and divisible by 32");
    const uint64_t n_total = sh->n_total, world = sh->world;
    if (n_total > 0xffffffffull) return fail(LQ4_ERR_OVERFLOW, "n_total does not fit");
    const uint64_t n0 = n_total * sh->rank / world, n1 = n_total * (sh->rank + 1) / world;
    if (local->n != n1 - n0) return fail(LQ4_ERR_SHAPE, "local->n must be this rank's rows of lq4_shard_plan(n_total, world, rank)");
    if (!sh->y_full) return fail(LQ4_ERR_NULL, "y_full is NULL");
    const uint64_t ldy = sh->ldy_full ? sh->ldy_full : n_total;
    if (ldy < n_total) return fail(LQ4_ERR_SHAPE, "ldy_full is smaller than n_total");
    if (!aligned(sh->y_full, 4)) return fail(LQ4_ERR_ALIGN, "y_full needs 4-byte alignment");
    if (world > 1 && !sh->nccl_comm) return fail(LQ4_ERR_NULL, "nccl_comm is NULL");
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t m = local->m;
    lq4_status st;

    if (world == 1) {                         // nothing to exchange: the slice is the output
        lq4_linear_args a = *local;
        a.y = sh->y_full;
        a.ldy = ldy;
        return lq4_linear(ctx, &a, stream);
    }
    const NcclApi& nc = nccl_api();
    if (!nc.ok) return fail(LQ4_ERR_UNSUPPORTED, "no NCCL library (libnccl.so.2) could be loaded");
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    LQ4_CUDA(cudaStreamIsCapturing(s, &cap));
    if (cap != cudaStreamCaptureStatusNone) return fail(LQ4_ERR_UNSUPPORTED, "lq4_linear_sharded cannot be captured in a CUDA graph");

    // tile-row blocks: as many as keep every block's product at about one wave of 256 x 256 tiles
    const uint64_t nl = n1 - n0;
    uint32_t blocks = 1;
    if (m > 256) {
        const uint64_t tiles = ((nl + 255) / 256) * ((m + 255) / 256);
        blocks = (uint32_t)((tiles + ctx->sm_count / 2) / ctx->sm_count);
        blocks = blocks < 1 ? 1 : (blocks > 4 ? 4 : blocks);
    }
    const uint32_t rows_per = ((m + blocks - 1) / blocks + 255) / 256 * 256;
    blocks = (m + rows_per - 1) / rows_per;

    if ((st = ensure(ctx, ctx->shard_send, (size_t)m * nl * 4, false, s))) return st;
    if ((st = ensure(ctx, ctx->shard_recv, (size_t)m * n_total * 4, false, s))) return st;
    if (!ctx->comm_stream) {
        LQ4_CUDA(cudaStreamCreateWithFlags(&ctx->comm_stream, cudaStreamNonBlocking));
        for (cudaEvent_t& e : ctx->ev_block) LQ4_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        LQ4_CUDA(cudaEventCreateWithFlags(&ctx->ev_comm, cudaEventDisableTiming));
    }
    bool equal = true;
    for (uint64_t r = 0; r < world; ++r) equal = equal && (n_total * (r + 1) / world - n_total * r / world) == nl;
    const size_t esz = local->x_dtype == LQ4_DTYPE_BF16 ? 2 : 4;

    for (uint32_t b = 0; b < blocks; ++b) {
        const uint32_t r0 = b * rows_per, rows = m - r0 < rows_per ? m - r0 : rows_per;
        float* send = (float*)ctx->shard_send.p + (size_t)r0 * nl;
        float* recv = (float*)ctx->shard_recv.p + (size_t)r0 * n_total;
        lq4_linear_args a = *local;
        a.x = static_cast<const uint8_t*>(local->x) + (size_t)r0 * local->k * esz;
        a.m = rows;
        a.y = send;
        a.ldy = nl;
        if ((st = lq4_linear(ctx, &a, stream))) return st;
        LQ4_CUDA(cudaEventRecord(ctx->ev_block[b], s));
        LQ4_CUDA(cudaStreamWaitEvent(ctx->comm_stream, ctx->ev_block[b], 0));
        if (equal) {
            LQ4_NCCL(nc.AllGather(send, recv, (size_t)rows * nl, kNcclFloat, sh->nccl_comm, ctx->comm_stream));
        } else {
            LQ4_NCCL(nc.GroupStart());
            for (uint64_t r = 0; r < world; ++r) {
                const uint64_t q0 = n_total * r / world, q1 = n_total * (r + 1) / world;
                int rc = nc.Broadcast(send, recv + q0 * rows, (size_t)rows * (q1 - q0), kNcclFloat, (int)r, sh->nccl_comm, ctx->comm_stream);
                if (rc != 0) { nc.GroupEnd(); return nccl_fail(rc, "ncclBroadcast"); }
            }
            LQ4_NCCL(nc.GroupEnd());
        }
        LQ4_CUDA(place_slices(recv, sh->y_full + (size_t)r0 * ldy, ldy, rows, n_total, (uint32_t)world, ctx->sm_count, ctx->comm_stream));
        ctx->launches += 1;
    }
    LQ4_CUDA(cudaEventRecord(ctx->ev_comm, ctx->comm_stream));
    LQ4_CUDA(cudaStreamWaitEvent(s, ctx->ev_comm, 0));
    return LQ4_OK;
}

}  // extern "C"
