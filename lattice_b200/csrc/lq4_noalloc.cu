// lq4_linear_decode_noalloc: the decode projection for callers that must not allocate.
//
// Who needs it: an engine that claimed all device memory for its own pool at start-up (a
// later cudaMalloc fails or eats into another tenant's share), and a latency-critical decode
// loop in which the device-wide synchronisation hidden inside cudaMalloc/cudaFree would
// stall every stream.  Neither can create an lq4_ctx, whose workspace lives in cudaMalloc'd
// buffers.  Here the kernel's scratch (stream-K partial-sum messages, the launch counter, the LoRA
// projection messages, the status word) sits in a fixed array that is part of the loaded module instead.
#include <cmath>
#include <mutex>

#include "lq4_kernels.cuh"

namespace {

using namespace lq4;

// Capacity of the built-in scratch.  Every GPU that loads this library holds these bytes
// until the process exits.
constexpr uint32_t kNaMaxGrid = 160;        // CTAs (one per SM; B200 has 148)
constexpr uint32_t kNaMaxM = 4;             // tokens per call
constexpr uint32_t kNaMaxN = 32768;         // output rows per call
constexpr uint32_t kNaMaxRank = 64;         // LoRA rank
constexpr size_t kNaCtrlBytes = 256;                                                              // status word at 0, launch counter at 64
constexpr size_t kNaPartialBytes = (size_t)kNaMaxGrid * 2 * kGemvTileRows * 4 * sizeof(float);    // 655,360
// t = A x messages: tokens x rank x k pieces x 8 B; the piece count is decode_tsplit()'s, clamped to kDecodeMaxTsplit
constexpr size_t kNaTpartBytes = (size_t)kNaMaxM * kNaMaxRank * kDecodeMaxTsplit * sizeof(uint2);  // 16,384
constexpr size_t kNaScratchBytes = kNaCtrlBytes + kNaPartialBytes + kNaTpartBytes;                 // 672,000
static_assert(kNaCtrlBytes % 256 == 0 && kNaPartialBytes % 256 == 0, "sections keep the array's 256-byte alignment");

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

}  // namespace

// Declared in include/lattice_q4.h.
extern "C" lq4_status lq4_linear_decode_noalloc(const lq4_linear_args* a, void* stream) {
    auto fail = [](lq4_status s, const char* msg) {
        set_last_error(msg);          // read back with lq4_last_error()
        return s;
    };
    if (!a) return fail(LQ4_ERR_NULL, "args is NULL");
    if (a->gather || a->wait_gather) return fail(LQ4_ERR_UNSUPPORTED, "lq4_linear_decode_noalloc has no fused all-gather");
    if (a->m == 0 || a->n == 0) return LQ4_OK;
    if (a->k == 0 || a->k % 32 != 0) return fail(LQ4_ERR_K, "k must be non-zero and divisible by 32");
    {
        // element counts are checked before anything is derived from them, as in lq4_linear
        const uint64_t lim = (uint64_t)1 << 40;
        if ((uint64_t)a->m * a->k > lim || (uint64_t)a->n * a->k > lim || (uint64_t)a->m * a->n > lim)
            return fail(LQ4_ERR_OVERFLOW, "m*k, n*k or m*n exceeds the supported element count");
    }
    if (!a->x || !a->w || !a->y) return fail(LQ4_ERR_NULL, "x, w and y must be non-NULL");
    if (a->x_dtype != LQ4_DTYPE_F32 && a->x_dtype != LQ4_DTYPE_BF16) return fail(LQ4_ERR_DTYPE, "unknown x_dtype");
    if (a->m > kNaMaxM) return fail(LQ4_ERR_NOSPACE, "lq4_linear_decode_noalloc handles at most 4 tokens per call");
    if (a->n > kNaMaxN) return fail(LQ4_ERR_NOSPACE, "lq4_linear_decode_noalloc handles at most 32768 output rows per call");
    const uint32_t rank = a->lora ? a->lora->rank : 0;
    if (a->lora) {
        if (!a->lora->a || !a->lora->b || rank == 0 || !std::isfinite(a->lora->scale))
            return fail(LQ4_ERR_LORA, "invalid LoRA descriptor");
        if (rank > kNaMaxRank) return fail(LQ4_ERR_NOSPACE, "lq4_linear_decode_noalloc handles LoRA rank up to 64");
        if ((reinterpret_cast<uintptr_t>(a->lora->a) & 3) || (reinterpret_cast<uintptr_t>(a->lora->b) & 3))
            return fail(LQ4_ERR_ALIGN, "LoRA factors need 4-byte alignment");
    }
    if (a->k % 128 != 0 || (reinterpret_cast<uintptr_t>(a->w) & 15) || (reinterpret_cast<uintptr_t>(a->x) & 15) ||
        (reinterpret_cast<uintptr_t>(a->y) & 3))
        return fail(LQ4_ERR_ALIGN, "needs k % 128 == 0 and 16-byte aligned w and x");
    if (a->ldy != 0 && a->ldy < a->n) return fail(LQ4_ERR_SHAPE, "ldy is smaller than n");
    const float* signs = nullptr;
    if (a->rot) {
        if (!a->rot->signs || a->rot->dim != a->k || (a->k & (a->k - 1))) return fail(LQ4_ERR_ROT, "invalid rotation descriptor");
        signs = a->rot->signs;
    }
    if (signs && a->lora)
        return fail(LQ4_ERR_UNSUPPORTED, "rotation together with LoRA needs a workspace: use lq4_linear");
    if (!gemv_resident_fits(a->m, a->k, signs != nullptr))
        return fail(LQ4_ERR_NOSPACE, "m * k too large: the activation row(s) must fit in shared memory for this entry point");

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(LQ4_ERR_UNSUPPORTED, "device index out of range");
    unsigned char* base;
    int sms;
    {
        // Set-up, once per device, with that device current: resolve the device address of the array.
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_scratch_ptr[dev]) {
            unsigned char* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) return fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
            int n = 0;
            e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
            g_sm_count[dev] = n;
            g_scratch_ptr[dev] = p;
        }
        base = g_scratch_ptr[dev];
        sms = g_sm_count[dev];
    }
    cudaStream_t s = (cudaStream_t)stream;

    GemvParams p{};
    p.w = a->w; p.y = a->y; p.ldy = a->ldy ? a->ldy : a->n;
    p.m = a->m; p.n = a->n; p.k = a->k;
    p.kb = a->k / 32; p.kg = p.kb / kGemvGranuleBlocks;
    p.tiles = (a->n + kGemvTileRows - 1) / kGemvTileRows;
    p.x = a->x; p.x_dtype = a->x_dtype; p.signs = signs;
    p.tsplit = 1;
    if (a->lora) { p.la = a->lora->a; p.lb = a->lora->b; p.rank = rank; p.lscale = a->lora->scale; p.tsplit = decode_tsplit(a->k); }
    p.sm_count = sms < (int)kNaMaxGrid ? sms : (int)kNaMaxGrid;

    // carve the array: [status | counters] [partial-sum messages] [t = A x]
    p.status = reinterpret_cast<int32_t*>(base);
    p.tsync = reinterpret_cast<uint32_t*>(base + 64);
    unsigned char* q = base + kNaCtrlBytes;
    p.partials = reinterpret_cast<float*>(q);
    p.tmsg = reinterpret_cast<uint2*>(q + kNaPartialBytes);               // t = A x messages
    p.use_pdl = 0;
    if ((size_t)p.m * p.rank * p.tsplit * sizeof(uint2) > kNaTpartBytes)
        return fail(LQ4_ERR_NOSPACE, "LoRA projection messages exceed the built-in array");
    // The array keeps whatever the previous call left, on purpose: every cross-CTA message in it is
    // tagged from the launch counter stored in the array, which each launch advances, so stale
    // messages are never mistaken for new ones.  The status word (zero when the module is loaded) is
    // only ever OR-ed into by kernels; lq4_noalloc_check reads and clears it.
    const size_t smem = decode_plan_smem(p);
    if (!smem) return fail(LQ4_ERR_NOSPACE, "shared-memory plan does not fit");
    const uint64_t units = decode_units(p);
    const uint64_t grid = units < (uint64_t)p.sm_count ? units : (uint64_t)p.sm_count;
    e = launch_decode(p, smem, (int)grid, s);
    if (e != cudaSuccess) return fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
    return LQ4_OK;
}

// Declared in include/lattice_q4.h.  A 4-byte copy out of the array and, if the word was set, a
// 4-byte clear: nothing is allocated.
extern "C" lq4_status lq4_noalloc_check(void* stream) {
    auto fail = [](lq4_status s, const char* msg) {
        set_last_error(msg);
        return s;
    };
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(LQ4_ERR_UNSUPPORTED, "device index out of range");
    unsigned char* base;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        base = g_scratch_ptr[dev];
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (!base) {
        // no call of the entry point on this device yet: nothing can have failed
        e = cudaStreamSynchronize(s);
        return e == cudaSuccess ? LQ4_OK : fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
    }
    int32_t word = 0;
    e = cudaMemcpyAsync(&word, base, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
    if (word != 0) {
        e = cudaMemsetAsync(base, 0, 4, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return fail(LQ4_ERR_CUDA, cudaGetErrorString(e));
        return fail(LQ4_ERR_DEVICE, "a kernel launched through lq4_linear_decode_noalloc gave up on a bounded wait");
    }
    return LQ4_OK;
}
