// Pieces shared by the two decode kernels (lq4_decode.cu: one token, activations resident in
// shared memory; lq4_dense.cu: 2..16 tokens, activation limbs staged beside the weights).
#pragma once

#include <cuda.h>

#include "lq4_gemv_common.cuh"

namespace lq4 {
namespace dec {

using namespace gemv;

constexpr int kBigBlocks = 20;                                   // blocks per row in a big stage
constexpr int kSmallBlocks = kGemvGranuleBlocks;                 // 4
constexpr uint32_t kSlotBytes = kGemvTileRows * kBigBlocks * kBlockBytes;      // 51,200
constexpr uint32_t kSmallBytes = kGemvTileRows * kSmallBlocks * kBlockBytes;   // 10,240
constexpr int kMaxStages = 8;
constexpr uint32_t kZeroOffset = 2 * kMaxStages * 8;   // 32 zero bytes after the mbarriers

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Cross-CTA messages are 8-byte {value, tag} pairs written with one store: the tag arrives with
// the value, so neither side needs a fence (a gpu-scope fence in mid-stream would wait for the
// hundreds of kilobytes of weight loads the SM has in flight).  The tag identifies the launch.
// Both sides use relaxed gpu-scope accesses, which are served by L2.
__device__ __forceinline__ void msg_store(uint2* p, float v, uint32_t tag) {
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 msg_load(const uint2* p) {
    uint2 r;
    asm volatile("ld.relaxed.gpu.global.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p) : "memory");
    return r;
}
// Launch tags.  Every launch adds exactly 256 to a 64-bit counter: CTA c adds its share of 256
// virtual arrivals with a fire-and-forget reduction when it is done.  (counter >> 8) + 1, read after
// the previous launch has completed and before the reading CTA has added its own share, is
// therefore the same in every CTA of a launch and new in every launch, and no CTA has to wait for
// an atomic's return value on its way out.
__device__ __forceinline__ uint32_t launch_tag(const uint32_t* counter) {
    unsigned long long c;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(c) : "l"(counter) : "memory");
    return (uint32_t)(c >> 8) + 1u;
}
__device__ __forceinline__ void launch_done(uint32_t* counter, uint32_t cta, uint32_t grid) {
    const unsigned long long share = 256u / grid + (cta < 256u % grid ? 1u : 0u);
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(counter), "l"(share) : "memory");
}

// Output store; with a fused all-gather the value also goes to the same place in every peer.
__device__ __forceinline__ void store_out(const GemvParams& q, size_t idx, float v) {
    q.y[idx] = v;
    if (q.world > 1) {
        char* own = reinterpret_cast<char*>(q.y + idx);
        for (uint32_t r = 0; r < q.world; ++r)
            if (r != q.grank) *reinterpret_cast<float*>(own + q.peer_off[r]) = v;
    }
}
// One thread per CTA, after the CTA's last output store (and a CTA barrier).  The CTAs of a launch
// count themselves on a counter in this GPU's own memory (each adds its share of 256); the one
// that completes the 256 tells every peer, with a single remote reduction each, that the launch's
// results have arrived, and advances this rank's sequence counter.  Remote reductions to one
// address are slow, hence one per launch and peer rather than one per CTA.
__device__ __forceinline__ void gather_done(const GemvParams& q, uint32_t cta, uint32_t grid) {
    if (q.world <= 1) return;
    const unsigned long long share = 256u / grid + (cta < 256u % grid ? 1u : 0u);
    // Release chain: this CTA's stores (after the CTA barrier) -> gpu-scope fence + add on the local
    // counter -> observed by the launch's last CTA -> its system-scope fence + remote reduction ->
    // the peer's system-scope acquire of the arrival counter.
    __threadfence();
    if (share == 0) return;
    const unsigned long long old = atomicAdd(q.gseq + 1, share);
    if (((old + share) & 255ull) != 0) return;
    // one system-scope release fence for the whole launch, then relaxed signals (a release on every
    // remote reduction would repeat the fence once per peer)
    __threadfence_system();
    for (uint32_t r = 0; r < q.world; ++r)
        if (r != q.grank)
            asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(q.peer_arrive[r]), "l"(256ull) : "memory");
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(q.gseq), "l"(256ull) : "memory");
}

// u8 x s8 -> s32 warp MMA: D(16x8) += A(16x32, u8, row) * B(32x8, s8, col).
__device__ __forceinline__ void imma_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr float kLimb1Ratio = 254.0f;    // limb 1 is in units of scale / 254

// Eight activations of one Q4 block (a quad of threads holds its 32) -> two int8 limbs with the
// block's common scale s = max|x| / 127:  x ~= s * (l0 + l1 / 254), |l0|, |l1| <= 127, so the
// representation error is below max|x| / 64516 and integer dot products with the 4-bit codes are
// exact.  `amax` is the block's max |x| (already reduced over the quad).  Rounding uses the
// 1.5 * 2^23 trick: after the add, the low byte of the float's bit pattern is the two's-complement
// integer, so no float-to-int conversions are needed.  Output words hold the limbs of
// {v0, v2, v4, v6} (a) and {v1, v3, v5, v7} (b): the order of the MMA's k slots.
struct Limbs8 { uint32_t l0a, l0b, l1a, l1b; float scale; };

__device__ __forceinline__ uint32_t low_bytes4(float a, float b, float c, float d) {
    const uint32_t lo = __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x0040);
    const uint32_t hi = __byte_perm(__float_as_uint(c), __float_as_uint(d), 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

__device__ __forceinline__ Limbs8 make_limbs8(const float (&v)[8], float amax) {
    constexpr float kMagic = 12582912.0f;              // 1.5 * 2^23
    const bool tiny = !(amax > 1e-30f);
    Limbs8 r;
    r.scale = tiny ? 1.0f : amax * (1.0f / 127.0f);
    const float inv0 = tiny ? 0.0f : 127.0f / amax;
    const float inv1 = inv0 * kLimb1Ratio;
    float f0[8], f1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        f0[i] = fmaf(v[i], inv0, kMagic);                               // |v * inv0| <= 127
        const float res = fmaf(-(f0[i] - kMagic), r.scale, v[i]);       // what limb 0 leaves over
        f1[i] = fminf(fmaxf(res * inv1, -127.0f), 127.0f) + kMagic;
    }
    r.l0a = low_bytes4(f0[0], f0[2], f0[4], f0[6]);
    r.l0b = low_bytes4(f0[1], f0[3], f0[5], f0[7]);
    r.l1a = low_bytes4(f1[0], f1[2], f1[4], f1[6]);
    r.l1b = low_bytes4(f1[1], f1[3], f1[5], f1[7]);
    return r;
}

// Limbs of eight activations (octet `o` of token slot `mp`) into the resident layout:
// limbs [block][token][limb 0, limb 1][32 B], per-block info {scale, sum of the 32 activations}.
__device__ __forceinline__ void store_limbs(uint8_t* xs, float2* sx, uint32_t MT, uint32_t mp, uint32_t o,
                                            bool active, const float (&v)[8]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
    sum += __shfl_xor_sync(kFull, sum, 1);
    sum += __shfl_xor_sync(kFull, sum, 2);
    if (!active) return;
    const Limbs8 l = make_limbs8(v, amax);
    const uint32_t blk = o >> 2, j = o & 3;
    uint8_t* dst = xs + ((size_t)blk * MT + mp) * 64 + j * 8;
    *reinterpret_cast<uint2*>(dst) = make_uint2(l.l0a, l.l0b);
    *reinterpret_cast<uint2*>(dst + 32) = make_uint2(l.l1a, l.l1b);
    if (j == 0) sx[(size_t)blk * MT + mp] = make_float2(l.scale, sum);
}

// Granules (4 blocks each) the next stage takes when `left` remain in the segment: 5, 3 or 1.
// Row strides of 100, 60 and 20 words keep the consumer loads free of bank conflicts.
__device__ __forceinline__ uint32_t stage_granules(uint32_t left) { return left >= 5 ? 5u : (left >= 3 ? 3u : 1u); }

// Arguments of one launch: NP problems (NP = 1 for a single projection).  The shared-memory
// offsets, the stage count, the workspace pointers and the PDL flag are taken from p[0]; the
// problems differ in weights, shapes, activations, output and adapter.
template <int NP>
struct DecodeArgs {
    GemvParams p[NP];
    CUtensorMap maps[NP][3];      // boxes of 20, 12 and 4 blocks x 128 rows
    uint32_t cta_begin[NP + 1];   // CTAs [cta_begin[i], cta_begin[i+1]) work on problem i and on nothing else
    uint32_t dot_start[NP + 1];   // resident kernel: first LoRA projection dot (token, rank row) of each problem
    uint32_t count;
    uint32_t any_rank;            // some problem has a LoRA adapter
};


// One CTA of 256 threads computes t[pr] = sum_k A[j][k] * x[tok][k] for pr = tok * rank + j, with a
// fixed reduction order.
// With x_mul the input is silu(x) * x_mul (f32, rows ldx floats apart).
__device__ __forceinline__ void project_one(const void* __restrict__ x, int x_dtype, uint32_t k,
                                            const float* __restrict__ la, uint32_t rank, float* __restrict__ t,
                                            uint32_t pr, int vec4, const float* __restrict__ x_mul = nullptr,
                                            uint32_t ldx = 0) {
    const uint32_t tok = pr / rank, j = pr - tok * rank;
    const float* arow = la + (size_t)j * k;
    float s = 0.0f;
    if (x_mul) {
        const float* g = static_cast<const float*>(x) + (size_t)tok * ldx;
        const float* u = x_mul + (size_t)tok * ldx;
#pragma unroll 4
        for (uint32_t i = threadIdx.x; i < k; i += 256) s = fmaf(__ldg(arow + i), silu_mul(g[i], u[i]), s);
    } else if (vec4) {
        const float4* a4 = reinterpret_cast<const float4*>(arow);
        const float4* x4 = reinterpret_cast<const float4*>(static_cast<const float*>(x) + (size_t)tok * k);
#pragma unroll 4
        for (uint32_t i = threadIdx.x; i < k / 4; i += 256) {
            const float4 a = __ldg(a4 + i), b = x4[i];
            s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
        }
    } else {
#pragma unroll 4
        for (uint32_t i = threadIdx.x; i < k; i += 256) s = fmaf(__ldg(arow + i), load_act(x, x_dtype, (size_t)tok * k + i), s);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __shared__ float part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) t[pr] = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
}

// Host side: hands each problem a contiguous share of the grid's CTAs, proportional to its cost
// (work units of 4 blocks x 128 rows, plus a fixed charge per tile for the fix-up and epilogue), so
// that no CTA has to switch problems.  Needs grid >= count; a problem never gets more CTAs than
// it has units.
void split_ctas(const GemvParams* ps, uint32_t count, uint32_t grid, uint32_t* cta_begin, uint32_t tile_charge = 8);

// Host side: the three tensor maps of a payload (boxes of 20, 12 and 4 blocks x 128 rows), from a
// per-thread cache keyed by (pointer, n, k).  NULL if the driver entry point is missing or the
// encode fails.
struct MapEntry { const uint8_t* w; uint32_t n, kb; CUtensorMap m[3]; };
const MapEntry* maps_for(const uint8_t* w, uint32_t n, uint32_t kb);

}  // namespace dec
}  // namespace lq4
