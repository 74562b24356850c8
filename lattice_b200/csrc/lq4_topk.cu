// Exact top-k over a logit row, the selection half of the reference's two-stage lm_head path
// (crates/inference/src/forward/shaders/qwen35.metal:1688-1770 candidate order and merge pass,
// :1866-1979 block top-k).
//
// The reference fuses the block-local selection into its lm_head GEMV because that GEMV is one
// vocabulary row per thread: a threadgroup owns 256 finished logits.  Here the GEMV is the
// stream-K decode kernel, whose row tiles finish on different CTAs, and the full logit row is
// 1 MB next to ~800 MB of Q4 rows; so the selection reads the logit row the GEMV wrote (still in
// L2) and is a separate, tiny launch chain:
//
//   pass 0   one CTA per 1024 logits: NaN -> sentinel, 64-bit sort keys in shared memory, full
//            bitonic sort (descending), the first k keys go to scratch
//   pass i   one CTA per 2048 / k groups of k keys: load, sort, emit the first k; repeated until one
//            group is left, which is decoded to (logit, token_id) pairs
//
// Order (topk_better): higher logit first, ties -> lower token id; NaN never ranks (it becomes the
// sentinel (-inf, UINT32_MAX), as in the reference).  The key packs exactly that order into one
// unsigned compare: the high word is the logit mapped monotonically to u32 (-0.0 folded into +0.0,
// which compare equal), the low word is ~token_id.  Every block's list is an exact local top-k,
// so the union of the lists contains the global top-k whatever the distribution (all winners in
// one block included).
#include "lq4_kernels.cuh"

namespace lq4 {

namespace {

constexpr uint64_t kSentinelKey = 0x007fffff00000000ull;      // (-inf, UINT32_MAX)

__device__ __forceinline__ uint64_t candidate_key(float v, uint32_t id) {
    if (v != v) return kSentinelKey;
    if (v == 0.0f) v = 0.0f;                                  // -0.0 == +0.0: one key for both
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((uint64_t)u << 32) | (uint32_t)~id;
}

__device__ __forceinline__ lq4_topk_candidate key_candidate(uint64_t key) {
    const uint32_t u = (uint32_t)(key >> 32);
    lq4_topk_candidate c;
    c.logit = __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
    c.token_id = ~(uint32_t)key;
    return c;
}

__device__ __forceinline__ uint64_t pick(uint64_t a, uint64_t b, bool take_max) {
    return ((a > b) == take_max) ? a : b;
}

// Sorts ITEMS keys (descending) with ITEMS / 2 threads.  Thread t keeps elements 2t and 2t + 1 of the
// bitonic network in registers: distance 1 is a compare inside the thread, distances 2..32 are lane
// exchanges (the partner element sits in lane ^ (j / 2), same slot), and only distances >= 64 go
// through shared memory (two buffers in turn, so that one block barrier per step is enough).
// Block b takes source items [b * per_block, (b + 1) * per_block) (clipped to `count`): logits when
// `logits` is non-NULL (item index = token id), else keys.  Writes the first k keys to
// out_keys + b * k, or, for the last pass (one block), the decoded candidates to `out`.
template <int ITEMS>
__global__ void __launch_bounds__(ITEMS / 2) topk_sort_kernel(const float* __restrict__ logits,
                                                              const uint64_t* __restrict__ in_keys, uint32_t count,
                                                              uint32_t per_block, uint32_t k,
                                                              uint64_t* __restrict__ out_keys,
                                                              lq4_topk_candidate* __restrict__ out) {
    __shared__ uint64_t xch[2][ITEMS];
    const uint32_t tid = threadIdx.x, e0 = 2 * tid;
    const uint64_t first = (uint64_t)blockIdx.x * per_block;
    uint64_t key[2];
#pragma unroll
    for (uint32_t slot = 0; slot < 2; ++slot) {
        const uint32_t i = e0 + slot;
        const uint64_t src = first + i;
        key[slot] = kSentinelKey;
        if (i < per_block && src < count) key[slot] = logits ? candidate_key(logits[src], (uint32_t)src) : in_keys[src];
    }
    uint32_t buf = 0;
    for (uint32_t size = 2; size <= ITEMS; size <<= 1) {
        const bool descending = (e0 & size) == 0;             // bit `size` is the same for both elements
        for (uint32_t j = size >> 1; j >= 64; j >>= 1) {
            xch[buf][e0] = key[0];
            xch[buf][e0 + 1] = key[1];
            __syncthreads();
            const bool take_max = ((e0 & j) == 0) == descending;
            key[0] = pick(key[0], xch[buf][e0 ^ j], take_max);
            key[1] = pick(key[1], xch[buf][(e0 + 1) ^ j], take_max);
            buf ^= 1;
        }
        for (uint32_t j = size >> 1 < 32 ? size >> 1 : 32; j >= 2; j >>= 1) {
            const bool take_max = ((e0 & j) == 0) == descending;
#pragma unroll
            for (uint32_t slot = 0; slot < 2; ++slot) {
                const uint64_t other = __shfl_xor_sync(0xffffffffu, key[slot], j >> 1);
                key[slot] = pick(key[slot], other, take_max);
            }
        }
        {
            const uint64_t hi = key[0] > key[1] ? key[0] : key[1], lo = key[0] > key[1] ? key[1] : key[0];
            key[0] = descending ? hi : lo;
            key[1] = descending ? lo : hi;
        }
    }
#pragma unroll
    for (uint32_t slot = 0; slot < 2; ++slot) {
        const uint32_t o = e0 + slot;
        if (o < k) {
            if (out) out[o] = key_candidate(key[slot]);
            else out_keys[(uint64_t)blockIdx.x * k + o] = key[slot];
        }
    }
}

constexpr uint32_t kBlockItems = 1024, kMergeItems = 2048;

}  // namespace

size_t topk_scratch_bytes(uint32_t n, uint32_t k) {
    const size_t groups = ((size_t)n + kBlockItems - 1) / kBlockItems;
    return 2 * ((groups * k * sizeof(uint64_t) + 255) / 256 * 256);
}

cudaError_t launch_topk(const float* logits, uint32_t n, uint32_t k, void* scratch, lq4_topk_candidate* out,
                        cudaStream_t s, int* launches) {
    const uint32_t groups0 = (n + kBlockItems - 1) / kBlockItems;
    const size_t half = topk_scratch_bytes(n, k) / 2;
    uint64_t* buf[2] = {static_cast<uint64_t*>(scratch), reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(scratch) + half)};
    int nl = 0;
    topk_sort_kernel<kBlockItems><<<groups0, kBlockItems / 2, 0, s>>>(logits, nullptr, n, kBlockItems, k, buf[0],
                                                                     groups0 == 1 ? out : nullptr);
    ++nl;
    uint32_t groups = groups0, cur = 0;
    const uint32_t fan_in = kMergeItems / k;                  // k <= 256: at least 8 groups per merge block
    while (groups > 1) {
        const uint32_t next = (groups + fan_in - 1) / fan_in;
        topk_sort_kernel<kMergeItems><<<next, kMergeItems / 2, 0, s>>>(nullptr, buf[cur], groups * k, fan_in * k, k,
                                                                       buf[cur ^ 1], next == 1 ? out : nullptr);
        ++nl;
        groups = next;
        cur ^= 1;
    }
    if (launches) *launches = nl;
    return cudaGetLastError();
}

}  // namespace lq4
