// Exact top-k over a logit row, the selection half of the reference's two-stage lm_head path
// (crates/inference/src/forward/shaders/qwen35.metal:1688-1770 candidate order and merge pass,
// :1866-1979 block top-k).
//
// The reference fuses the block-local selection into its lm_head GEMV because that GEMV is one
// vocabulary row per thread: a threadgroup owns 256 finished logits.  Here the GEMV is the
// stream-K decode kernel, whose row tiles finish on different CTAs, and the full logit row is
// 1 MB next to ~800 MB of Q4 rows; so the selection reads the logit row the GEMV wrote (still in
// L2) and is one small launch of its own:
//
//   every CTA      takes 2048 logits (NaN -> sentinel, 64-bit keys in registers), sorts them in chunks of
//                  K' = max(64, next power of two >= k) and halves the chunks pairwise (keep the K'
//                  largest of two chunks) until one is left: its first k keys are list `b` of level 0
//   tickets        lists are grouped 2048 / K' at a time; a CTA that has stored its list takes a ticket
//                  on its group's counter and exits, except the one that drew the last ticket: it
//                  loads the group's lists as chunks, halves them in the same way and carries the
//                  first k on as a list of the next level.  Nobody waits for anybody; the CTA that ends up with the only list of
//                  the top level decodes it to (logit, token_id) pairs.
//
// One launch instead of one per level: between dependent launches this GPU spends about 5 us, more
// than all the sorting of a 248,320-entry row.
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

constexpr uint32_t kItems = 2048, kThreads = kItems / 2;

// Chunk length of the selection network: the power of two >= k, at least 64 (one warp per chunk).
__host__ __device__ inline uint32_t chunk_len(uint32_t k) {
    uint32_t kp = 64;
    while (kp < k) kp <<= 1;
    return kp;
}

// The CTA holds 2048 keys; thread t keeps elements 2t and 2t + 1 in registers.  Exchanges at distance 1
// are a compare inside the thread, distances 2..32 are lane exchanges (the partner element sits in
// lane ^ (j / 2), same slot), distances >= 64 go through shared memory (two buffers in turn, so that
// one block barrier per step is enough).
struct Net {
    uint64_t (*xch)[kItems];
    uint32_t e0, buf;

    // One bitonic step at distance j >= 64 for the threads with `active`; all threads must call it.
    __device__ __forceinline__ void far_step(uint64_t (&key)[2], uint32_t j, bool take_max, bool active) {
        xch[buf][e0] = key[0];
        xch[buf][e0 + 1] = key[1];
        __syncthreads();
        if (active) {
            key[0] = pick(key[0], xch[buf][e0 ^ j], take_max);
            key[1] = pick(key[1], xch[buf][(e0 + 1) ^ j], take_max);
        }
        buf ^= 1;
    }
    // Steps at distances j0, j0 / 2, ..., 1 (j0 <= 32) of a merge in direction `descending`.
    __device__ __forceinline__ void near_steps(uint64_t (&key)[2], uint32_t j0, bool descending) {
        for (uint32_t j = j0; j >= 2; j >>= 1) {
            const bool take_max = ((e0 & j) == 0) == descending;
#pragma unroll
            for (uint32_t slot = 0; slot < 2; ++slot) {
                const uint64_t other = __shfl_xor_sync(0xffffffffu, key[slot], j >> 1);
                key[slot] = pick(key[slot], other, take_max);
            }
        }
        const uint64_t hi = key[0] > key[1] ? key[0] : key[1], lo = key[0] > key[1] ? key[1] : key[0];
        key[0] = descending ? hi : lo;
        key[1] = descending ? lo : hi;
    }

    // Sorts every chunk of kp keys, even chunks descending, odd chunks ascending (the bitonic network up
    // to sequence length kp).
    __device__ __forceinline__ void sort_chunks(uint64_t (&key)[2], uint32_t kp) {
        for (uint32_t size = 2; size <= kp; size <<= 1) {
            const bool descending = (e0 & size) == 0;
            for (uint32_t j = size >> 1; j >= 64; j >>= 1) far_step(key, j, ((e0 & j) == 0) == descending, true);
            near_steps(key, size >> 1 < 32 ? size >> 1 : 32, descending);
        }
    }

    // Chunks sorted as sort_chunks leaves them -> the kp largest keys of all, descending, in chunk 0.
    // Round r pairs the surviving chunks c and c + 2^r: the element-wise maximum of a descending and an
    // ascending list holds the kp largest of both as a bitonic sequence; it stays in the lower chunk,
    // which is then merged into the direction the next round needs.  The other chunk is dead from then
    // on: its warps only keep the block barriers company, so the work halves every round.
    __device__ __forceinline__ void select_top(uint64_t (&key)[2], uint32_t kp) {
        for (uint32_t stride = kp; stride < kItems; stride <<= 1) {
            const bool live = (e0 & ((stride << 1) - 1) & ~(kp - 1)) == 0;     // lower chunk of a surviving pair
            far_step(key, stride, true, live);
            const bool descending = (e0 & (stride << 1)) == 0;
            for (uint32_t j = kp >> 1; j >= 64; j >>= 1) far_step(key, j, ((e0 & j) == 0) == descending, live);
            if (live) near_steps(key, 32, descending);
        }
    }
};

// lists:    [level 0: gridDim.x lists | level 1: ceil(gridDim.x / fan_in) lists | ...], k keys each, descending
// counters: one per list of every level above 0 (indexed like the lists), zero between launches:
//           the CTA that draws the last ticket of a group puts the counter back to zero.
__global__ void __launch_bounds__(kThreads) topk_kernel(const float* __restrict__ logits, uint32_t n, uint32_t k,
                                                        uint64_t* lists, uint32_t* counters,
                                                        lq4_topk_candidate* __restrict__ out) {
    __shared__ uint64_t xch[2][kItems];
    __shared__ uint32_t s_last;
    const uint32_t tid = threadIdx.x, e0 = 2 * tid;
    const uint32_t kp = chunk_len(k), fan_in = kItems / kp;
    Net net{xch, e0, 0};
    pdl_wait_prior_grids();                                   // the logits come from the launch before this one
    uint64_t key[2];
#pragma unroll
    for (uint32_t slot = 0; slot < 2; ++slot) {
        const uint64_t src = (uint64_t)blockIdx.x * kItems + e0 + slot;
        key[slot] = src < n ? candidate_key(logits[src], (uint32_t)src) : kSentinelKey;
    }
    net.sort_chunks(key, kp);
    net.select_top(key, kp);

    uint32_t groups = gridDim.x, my = blockIdx.x, base = 0;   // lists on this level, this CTA's, first list of the level
    while (groups > 1) {
#pragma unroll
        for (uint32_t slot = 0; slot < 2; ++slot)
            if (e0 + slot < k) __stcg(&lists[(uint64_t)(base + my) * k + e0 + slot], key[slot]);
        const uint32_t parent = my / fan_in, next_base = base + groups;
        const uint32_t members = groups - parent * fan_in < fan_in ? groups - parent * fan_in : fan_in;
        __syncthreads();                                      // every thread's keys are stored
        if (tid == 0) {
            __threadfence();
            const uint32_t ticket = atomicAdd(&counters[next_base + parent], 1u);
            s_last = ticket == members - 1;
            if (s_last) {
                counters[next_base + parent] = 0;             // nobody else touches it in this launch
                __threadfence();
            }
        }
        __syncthreads();
        if (!s_last) return;
        // The group's lists are complete (other CTAs of this launch wrote them: L2 loads).  List c goes to
        // chunk c, reversed in the odd chunks, padded with sentinels: the state sort_chunks leaves.
        const uint64_t* src = lists + (uint64_t)(base + parent * fan_in) * k;
#pragma unroll
        for (uint32_t slot = 0; slot < 2; ++slot) {
            const uint32_t i = e0 + slot, c = i / kp, p = i & (kp - 1), q = (c & 1u) ? kp - 1 - p : p;
            key[slot] = (c < members && q < k) ? __ldcg(&src[(uint64_t)c * k + q]) : kSentinelKey;
        }
        __syncthreads();                                      // s_last is rewritten on the next level
        net.select_top(key, kp);
        my = parent;
        base = next_base;
        groups = (groups + fan_in - 1) / fan_in;
    }
#pragma unroll
    for (uint32_t slot = 0; slot < 2; ++slot)
        if (e0 + slot < k) out[e0 + slot] = key_candidate(key[slot]);
}

uint32_t total_lists(uint32_t n, uint32_t k) {
    uint32_t groups = (n + kItems - 1) / kItems, total = groups;
    const uint32_t fan_in = kItems / chunk_len(k);
    while (groups > 1) {
        groups = (groups + fan_in - 1) / fan_in;
        total += groups;
    }
    return total;
}

}  // namespace

size_t topk_list_bytes(uint32_t n, uint32_t k) { return (size_t)total_lists(n, k) * k * sizeof(uint64_t); }

// Enough counters for any k: the fan-in is at least 8 (chunks of at most 256 keys), so the levels above 0 hold fewer than groups / 7 + 32 lists.
size_t topk_counter_bytes(uint32_t n) {
    const size_t groups = ((size_t)n + kItems - 1) / kItems;
    return (groups + groups / 7 + 34) * sizeof(uint32_t);
}

cudaError_t launch_topk(const float* logits, uint32_t n, uint32_t k, void* lists, uint32_t* counters,
                        lq4_topk_candidate* out, int use_pdl, cudaStream_t s, int* launches) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((n + kItems - 1) / kItems);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (use_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (launches) *launches = 1;
    return cudaLaunchKernelEx(&cfg, topk_kernel, logits, n, k, static_cast<uint64_t*>(lists), counters, out);
}

}  // namespace lq4
