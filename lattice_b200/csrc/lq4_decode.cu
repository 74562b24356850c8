// Resident decode kernel: y[m, n] = x[m, k] * Wq4[n, k]^T (+ LoRA) (+ rotation of x) for one token
// (up to four through the allocation-free entry point), and for groups of such projections in
// one launch.
//
// HBM-bound: the packed weights are read once, everything else is small.
//  * One persistent CTA per SM.  A producer warp streams weight tiles with TMA
//    (cp.async.bulk.tensor.2d, one instruction per stage) into a shared-memory ring;
//    completion is counted on mbarriers.  A stage is 128 rows x 20, 12 or 4 blocks (51,200 B at
//    most); rows stay densely packed, and the 100-, 60- and 20-word row strides keep every
//    consumer load free of bank conflicts.
//  * Eight consumer warps own 16 rows each.  Within a group of four Q4 blocks, the four
//    threads of an MMA quad take one block each: the 32 k-slots of a u8 x s8 warp MMA (m16n8k32)
//    hold eight codes of each of the four blocks, and the B operand is zero outside the column
//    pair (limb 0, limb 1) that belongs to the thread's block.  After four MMAs each thread holds
//    the exact integer dot products of its own block for two rows, so the per-block scale/bias
//    step is done once per four blocks per thread.
//  * The activation row is converted once per CTA into two int8 limbs with a per-block f32 scale
//    kept in shared memory (optionally after the randomized Hadamard rotation, also done in the
//    CTA); only the k range(s) the CTA touches are converted.
//  * Work is split stream-K style in units of 4 blocks x 128 rows (or in whole tiles when that
//    keeps the SMs busy).  The CTA that owns a tile's first k part finishes the tile: the others
//    publish their partial sums as 8-byte {value, launch tag} messages and the finisher adds them
//    in CTA order (bounded wait).  No fences, no atomics with a returned value on the way.
//  * In a grouped launch every problem gets a contiguous share of the CTAs in proportion to its
//    cost; a CTA works on one problem only.
//  * LoRA: once the ring is full for the first time, the producer warps compute the projection
//    t = A x (work items of one dot-product piece each, spread over all CTAs) and publish it as
//    tagged messages; finishers gather t into shared memory and add s * B * t in the epilogue.
//  * With a fused all-gather the epilogue also stores into every peer GPU's output buffer and
//    the launch's last CTA signals the peers' arrival counters.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "lq4_decode_common.cuh"

namespace lq4 {

namespace {

using namespace gemv;
using namespace dec;

// Randomized Hadamard transform of one activation row of K = 256 * R elements by the 256 consumer
// threads: x'[i] = (1 / sqrt(K)) * sum_j H[i][j] * signs[j] * x[j].  The log2(K) butterfly levels
// are independent of one another, so they are taken in the order that needs the least traffic:
// thread (warp w, lane l) first holds elements l + 32 w + 256 r and does the levels of the r bits
// in registers and those of the lane bits with shuffles; one trip through shared memory regroups
// the row so that the three warp bits sit in registers for the last three levels.
template <int R>
__device__ __forceinline__ void fwht_row_fast(const void* x, int x_dtype, const float* signs, float* xrot, uint32_t x_off,
                                              int ctid) {
    const uint32_t lane = ctid & 31, w = ctid >> 5, K = 256u * R;
    float v[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const uint32_t i = lane + 32 * w + 256 * r;
        v[r] = load_act(x, x_dtype, (size_t)x_off + i) * signs[i];
    }
#pragma unroll
    for (int h = 1; h < R; h <<= 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r & h) continue;
            const float a = v[r], b = v[r + h];
            v[r] = a + b;
            v[r + h] = a - b;
        }
    }
#pragma unroll
    for (int mask = 1; mask < 32; mask <<= 1) {
        const bool upper = (lane & mask) != 0;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float o = __shfl_xor_sync(kFull, v[r], mask);
            v[r] = upper ? o - v[r] : v[r] + o;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) xrot[lane + 32 * w + 256 * r] = v[r];
    named_bar_sync(kBarConsumers, kConsumerThreads);
    // regroup: register q + 8 s holds element lane + 32 q + 256 (w + 8 s)
#pragma unroll
    for (int s = 0; s < R / 8; ++s)
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q + 8 * s] = xrot[lane + 32 * q + 256 * (w + 8 * s)];
#pragma unroll
    for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r & h) continue;
            const float a = v[r], b = v[r + h];
            v[r] = a + b;
            v[r + h] = a - b;
        }
    }
    const float sc = 1.0f / sqrtf((float)K);
#pragma unroll
    for (int s = 0; s < R / 8; ++s)
#pragma unroll
        for (int q = 0; q < 8; ++q) xrot[lane + 32 * q + 256 * (w + 8 * s)] = v[q + 8 * s] * sc;
    named_bar_sync(kBarConsumers, kConsumerThreads);
}

// Prologue of the 256 consumer threads: rotation, LoRA partial projection, activation limbs.
template <int MT>
__device__ void decode_prologue(const GemvParams& p, uint8_t* smem, int ctid, uint64_t r0, uint64_t r1) {
    const uint32_t K = p.k, M = p.m;
    float* xrot = reinterpret_cast<float*>(smem + p.off_xrot);
    const bool rot = p.signs != nullptr;

    if (rot) {
        const uint32_t R = K / kConsumerThreads;          // elements per thread in the fast transform
        if (R == 8 || R == 16 || R == 32 || R == 64) {
            for (uint32_t row = 0; row < M; ++row) {
                switch (R) {
                    case 8: fwht_row_fast<8>(p.x, p.x_dtype, p.signs, xrot + (size_t)row * K, row * K, ctid); break;
                    case 16: fwht_row_fast<16>(p.x, p.x_dtype, p.signs, xrot + (size_t)row * K, row * K, ctid); break;
                    case 32: fwht_row_fast<32>(p.x, p.x_dtype, p.signs, xrot + (size_t)row * K, row * K, ctid); break;
                    default: fwht_row_fast<64>(p.x, p.x_dtype, p.signs, xrot + (size_t)row * K, row * K, ctid); break;
                }
            }
        } else {
            // short rows: one butterfly level per pass over shared memory
            for (uint32_t i = ctid; i < M * K; i += kConsumerThreads)
                xrot[i] = __fmul_rn(load_act(p.x, p.x_dtype, i), p.signs[i % K]);
            named_bar_sync(kBarConsumers, kConsumerThreads);
            const uint32_t half = K / 2;
            for (uint32_t h = 1; h < K; h <<= 1) {
                for (uint32_t bi = ctid; bi < M * half; bi += kConsumerThreads) {
                    const uint32_t row = bi / half, bb = bi - row * half;
                    const uint32_t j = row * K + (bb / h) * 2 * h + (bb % h);
                    const float a = xrot[j], b = xrot[j + h];
                    xrot[j] = __fadd_rn(a, b);
                    xrot[j + h] = __fsub_rn(a, b);
                }
                named_bar_sync(kBarConsumers, kConsumerThreads);
            }
            const float sc = __fdiv_rn(1.0f, __fsqrt_rn((float)K));
            for (uint32_t i = ctid; i < M * K; i += kConsumerThreads) xrot[i] = __fmul_rn(xrot[i], sc);
            named_bar_sync(kBarConsumers, kConsumerThreads);
        }
    }

    // limbs: [block][token][limb 0, limb 1][32 B]; per-block info {scale, sum}: [block][token]
    // Only the k range(s) this CTA's share of the work touches are converted: with a long k and
    // stream-K splitting that is a fraction of the row.  Ranges are in octets (8 activations).
    uint8_t* xs = smem + p.off_xs;
    float2* sx = reinterpret_cast<float2*>(smem + p.off_sx);
    const uint32_t opg = kGemvGranuleBlocks * 4;              // octets per granule
    uint32_t a0 = 0, a1 = K / 8, b0 = 0, b1 = 0;              // two octet ranges [a0,a1) and [b0,b1)
    if (r1 - r0 < p.kg) {
        const uint32_t g0 = (uint32_t)(r0 % p.kg), len = (uint32_t)(r1 - r0);
        if (g0 + len <= p.kg) { a0 = g0 * opg; a1 = (g0 + len) * opg; }
        else { a0 = g0 * opg; a1 = p.kg * opg; b0 = 0; b1 = (g0 + len - p.kg) * opg; }
    }
    const uint32_t na = a1 - a0, noct = na + (b1 - b0);
    for (uint32_t mp = 0; mp < (uint32_t)MT; ++mp) {
        // several octets per thread and pass: all global loads are issued before the first use
        constexpr int kBatch = MT <= 2 ? 8 : 4;
        for (uint32_t o0 = 0; o0 < noct; o0 += kBatch * kConsumerThreads) {
            float v[kBatch][8];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint32_t i = o0 + u * kConsumerThreads + ctid;
                const uint32_t o = i < na ? a0 + i : b0 + (i - na);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[u][e] = 0.0f;
                if (i < noct) {
                    if (rot) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[u][e] = xrot[mp * K + o * 8 + e];
                    } else {
                        load8(p.x, p.x_dtype, (size_t)mp * K + (size_t)o * 8, v[u]);
                    }
                }
            }
            if (p.x_mul) {                                    // gated input (one f32 token): silu(gate) * up
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const uint32_t i = o0 + u * kConsumerThreads + ctid;
                    const uint32_t o = i < na ? a0 + i : b0 + (i - na);
                    if (i < noct) {
                        float up[8];
                        load8(p.x_mul, LQ4_DTYPE_F32, (size_t)o * 8, up);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[u][e] = silu_mul(v[u][e], up[e]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint32_t i = o0 + u * kConsumerThreads + ctid;
                const uint32_t o = i < na ? a0 + i : b0 + (i - na);
                store_limbs(xs, sx, MT, mp, o, i < noct, v[u]);
            }
        }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
}

template <int MT, int NP>
__global__ void __launch_bounds__(kGemvThreads, 1) decode_kernel(const __grid_constant__ DecodeArgs<NP> ga) {
    const GemvParams& p = ga.p[0];
    const uint32_t count = NP == 1 ? 1u : ga.count;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    __shared__ int s_err;
    __shared__ int s_twait_failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t NST = p.nstages;
    if (tid == 0) {
        for (uint32_t s = 0; s < NST; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 8);
        }
        s_err = 0;
        s_twait_failed = 0;
        for (int i = 0; i < 8; ++i) reinterpret_cast<uint32_t*>(smem + kZeroOffset)[i] = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (p.use_pdl) pdl_launch_dependents();

    // this CTA's problem, and its share of that problem's work units among the problem's CTAs
    uint32_t pi = 0;
    if (NP > 1)
        while (pi + 1 < count && blockIdx.x >= ga.cta_begin[pi + 1]) ++pi;
    const GemvParams& q = ga.p[pi];
    const uint32_t cta0 = NP == 1 ? 0u : ga.cta_begin[pi];
    const uint64_t G = NP == 1 ? gridDim.x : ga.cta_begin[pi + 1] - cta0;
    const uint32_t cl = blockIdx.x - cta0;
    const uint64_t total = (uint64_t)q.tiles * q.kg;
    // whole-tile mode hands out entire tiles (no partial sums); otherwise equal shares of granules
    const bool whole = NP == 1 && p.whole_tiles;
    const uint64_t r0 = whole ? range_begin(cl, q.tiles, G) * q.kg : range_begin(cl, total, G);
    const uint64_t r1 = whole ? range_begin(cl + 1, q.tiles, G) * q.kg : range_begin(cl + 1, total, G);
    uint32_t issued = 0;

    if (warp == 8) {
        // ------------------------------ producer ------------------------------
        // All 32 lanes walk the same loop; lane 0 issues the copies.  Once the ring is full for the
        // first time (the consumers are still converting activations), the warp takes its share of
        // the LoRA projections t = A x and publishes them as tagged messages.
        const uint64_t pol = l2_policy_evict_first();
        const bool any_rank = NP == 1 ? p.rank != 0 : ga.any_rank != 0;
        bool projected = !any_rank;
        auto project = [&]() {
            projected = true;
            if (p.use_pdl) pdl_wait_prior_grids();          // x may come from the launch before this one
            if (p.wait_world > 1) {       // one lane polls the arrival counter, the warp follows
                if (lane == 0 && !wait_gather_arrivals(p.wait_arrive, p.wait_world)) atomicOr(p.status, kDevErrGridWaitTimeout);
                __syncwarp();
            }
            const uint32_t tag = launch_tag(p.tsync);
            // work item e = (problem, token, rank row, k piece); item e belongs to CTA e mod grid
            const uint32_t nitems = NP == 1 ? p.m * p.rank * p.tsplit : ga.dot_start[count];
            uint32_t pj = 0;
            for (uint32_t e = blockIdx.x; e < nitems; e += gridDim.x) {
                if (NP > 1)
                    while (pj + 1 < count && e >= ga.dot_start[pj + 1]) ++pj;
                const GemvParams& qq = ga.p[pj];
                const uint32_t local = NP == 1 ? e : e - ga.dot_start[pj];
                const uint32_t dot = local / qq.tsplit, sp = local - dot * qq.tsplit;
                const uint32_t tok = dot / qq.rank, j = dot - tok * qq.rank;
                const uint32_t k4 = qq.k / 4;
                const uint32_t chunk4 = ((k4 + qq.tsplit - 1) / qq.tsplit + 31u) & ~31u;
                const uint32_t i0 = sp * chunk4, i1 = min(k4, i0 + chunk4);
                const float* arow = qq.la + (size_t)j * qq.k;
                float s = 0.0f;
                const bool vec4 = qq.x_dtype == LQ4_DTYPE_F32 && ((reinterpret_cast<uintptr_t>(qq.x) | reinterpret_cast<uintptr_t>(qq.la)) & 15u) == 0;
                if (qq.x_mul) {
                    // gated input: the adapter sees silu(gate) * up like the Q4 rows do
                    const float4* a4 = reinterpret_cast<const float4*>(arow);
                    const float4* g4 = reinterpret_cast<const float4*>(qq.x);
                    const float4* u4 = reinterpret_cast<const float4*>(qq.x_mul);
#pragma unroll 8
                    for (uint32_t i = i0 + lane; i < i1; i += 32) {
                        const float4 a = __ldg(a4 + i), g = g4[i], u = u4[i];
                        s = fmaf(a.x, silu_mul(g.x, u.x), s); s = fmaf(a.y, silu_mul(g.y, u.y), s);
                        s = fmaf(a.z, silu_mul(g.z, u.z), s); s = fmaf(a.w, silu_mul(g.w, u.w), s);
                    }
                } else if (vec4) {
                    const float4* a4 = reinterpret_cast<const float4*>(arow);
                    const float4* x4 = reinterpret_cast<const float4*>(static_cast<const float*>(qq.x) + (size_t)tok * qq.k);
#pragma unroll 8
                    for (uint32_t i = i0 + lane; i < i1; i += 32) {
                        const float4 a = __ldg(a4 + i), b = x4[i];
                        s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
                    }
                } else {
#pragma unroll 8
                    for (uint32_t i = i0 * 4 + lane; i < i1 * 4; i += 32)
                        s = fmaf(__ldg(arow + i), load_act(qq.x, qq.x_dtype, (size_t)tok * qq.k + i), s);
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
                if (lane == 0) msg_store(qq.tmsg + local, s, tag);
            }
        };
        uint32_t it = 0;
        bool ok = true;
        for (uint64_t pos = r0; pos < r1 && ok;) {
            const uint32_t tile = (uint32_t)(pos / q.kg);
            const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * q.kg);
            const uint64_t left = r1 - pos;
            const uint32_t g1 = (uint64_t)(q.kg - g0) < left ? q.kg : (uint32_t)(g0 + left);
            for (uint32_t gs = g0; gs < g1; ++it) {
                if (it == NST && !projected) project();
                const uint32_t ngr = stage_granules(g1 - gs);
                const uint32_t s = it % NST;
                bool got = true;
                if (lane == 0) got = mbar_wait(&empty[s], ((it / NST) & 1u) ^ 1u);
                if (!__shfl_sync(kFull, got, 0)) { ok = false; break; }
                if (lane == 0) {
                    uint8_t* st = smem + p.off_stage + (size_t)s * kSlotBytes;
                    mbar_arrive_expect_tx(&full[s], ngr * kSmallBytes);
                    // coordinates: x in 4-byte elements along the row, y = first row of the tile
                    tma_load_2d(st, &ga.maps[pi][ngr == 5 ? 0 : (ngr == 3 ? 1 : 2)], (int32_t)(gs * kGemvGranuleBlocks * 5),
                                (int32_t)(tile * kGemvTileRows), &full[s], pol);
                }
                gs += ngr;
            }
            pos += g1 - g0;
        }
        if (!projected) project();
        issued = it;
        if (!ok && lane == 0) {
            atomicOr(p.status, kDevErrBarrierTimeout);
            s_err = 1;
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int g = lane >> 2, t = lane & 3;
        // x may come from the launch before this one, or from the peers of a fused all-gather
        if (p.use_pdl) pdl_wait_prior_grids();
        if (p.wait_world > 1) {           // one thread polls the arrival counter, the consumers follow
            if (tid == 0 && !wait_gather_arrivals(p.wait_arrive, p.wait_world)) atomicOr(p.status, kDevErrGridWaitTimeout);
            named_bar_sync(kBarConsumers, kConsumerThreads);
        }
        // a message written by an earlier launch never carries this launch's tag
        const uint32_t tag = launch_tag(p.tsync);

        // A lane supplies B-operand registers only for the column pair (limb 0, limb 1) of its own
        // block; every other lane reads a block of zeros, so that its columns contribute nothing.
        const bool has_b = (g >> 1) == t;
        const uint8_t* xs_lane = smem + p.off_xs + (size_t)(g & 1) * 32;
        const uint8_t* zeros = smem + kZeroOffset;
        const float2* sx_all = reinterpret_cast<const float2*>(smem + p.off_sx);

        uint32_t it = 0;
        bool ok = true;
        bool t_loaded = false;
        float* t_sm = reinterpret_cast<float*>(smem + p.off_t);
        // Gathers t = A x from the producer warps' messages (written in the first microseconds of the
        // launch) into shared memory, adding the k pieces of every dot product in order.  All eight
        // consumer warps call it at the same point of their (identical) walk.  Bounded wait.
        auto gather_t = [&]() {
            bool good = true;
            for (uint32_t idx = tid; idx < q.m * q.rank; idx += kConsumerThreads) {
                const uint2* src = q.tmsg + (size_t)idx * q.tsplit;
                float sum = 0.0f;
                for (uint32_t s0 = 0; s0 < q.tsplit; s0 += 8) {
                    uint2 msg[8];
                    const long long t0 = wait_clock();
                    for (;;) {
                        bool all = true;
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            if (s0 + u >= q.tsplit) continue;
                            msg[u] = msg_load(src + s0 + u);
                            all = all && (msg[u].y == tag);
                        }
                        if (all) break;
                        if (wait_expired(t0)) { good = false; break; }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (s0 + u < q.tsplit) sum += __uint_as_float(msg[u].x);
                }
                t_sm[idx] = sum;
            }
            if (!good) atomicOr(p.status, kDevErrGridWaitTimeout);
            named_bar_sync(kBarConsumers, kConsumerThreads);
            t_loaded = true;
        };
        decode_prologue<MT>(q, smem, tid, r0, r1);
        for (uint64_t pos = r0; pos < r1 && ok;) {
            const uint32_t tile = (uint32_t)(pos / q.kg);
            const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * q.kg);
            const uint64_t left = r1 - pos;
            const uint32_t g1 = (uint64_t)(q.kg - g0) < left ? q.kg : (uint32_t)(g0 + left);
            pos += g1 - g0;

            float acc[MT][2];
#pragma unroll
            for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = 0.0f;
            if (q.rank && g0 == 0) {
                // this CTA will finish the tile: pull the warp's 16 rows of LoRA B towards L2 now
                const uint32_t rfirst = tile * kGemvTileRows + warp * 16;
                const uint32_t rows = rfirst < q.n ? min(16u, q.n - rfirst) : 0u;
                const char* bb = reinterpret_cast<const char*>(q.lb + (size_t)rfirst * q.rank);
                for (uint32_t off = lane * 128; off < rows * q.rank * 4; off += 32 * 128)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(bb + off));
            }

            for (uint32_t gs = g0; gs < g1; ++it) {
                const uint32_t ngr = stage_granules(g1 - gs);
                const uint32_t rs = ngr * (kGemvGranuleBlocks * kBlockBytes);
                const uint32_t s = it % NST;
                if (!mbar_wait(&full[s], (it / NST) & 1u)) { ok = false; break; }
                // by now the projections are published; fetching them here keeps the round trip off
                // the end of the tile (the ring keeps the memory pipe busy meanwhile)
                if (it == 6 && q.rank && !t_loaded) gather_t();
                const uint8_t* st = smem + p.off_stage + (size_t)s * kSlotBytes;
                const uint8_t* row0 = st + (warp * 16 + g) * rs + t * kBlockBytes;
                const uint8_t* row1 = row0 + 8 * rs;
#pragma unroll 1
                for (uint32_t gi = 0; gi < ngr; ++gi) {
                    const uint32_t blk = (gs + gi) * kGemvGranuleBlocks + t;     // this thread's block
                    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(row0 + gi * (4 * kBlockBytes));
                    const uint32_t* q1 = reinterpret_cast<const uint32_t*>(row1 + gi * (4 * kBlockBytes));
                    const uint32_t meta0 = q0[0], meta1 = q1[0];
                    uint32_t w0[4], w1[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) { w0[j] = q0[1 + j]; w1[j] = q1[1 + j]; }
                    uint4 bq[MT][2];
                    float2 info[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint8_t* xb = has_b ? xs_lane + ((size_t)blk * MT + mt) * 64 : zeros;
                        bq[mt][0] = *reinterpret_cast<const uint4*>(xb);
                        bq[mt][1] = *reinterpret_cast<const uint4*>(xb + 16);
                        info[mt] = sx_all[(size_t)blk * MT + mt];
                    }
                    int c[MT][4];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) c[mt][0] = c[mt][1] = c[mt][2] = c[mt][3] = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // bytes {n0,n2,n4,n6} fill k-slots 4t..4t+3, bytes {n1,n3,n5,n7} slots 4t+16..4t+19
                        uint32_t a[4];
                        a[0] = w0[j] & 0x0F0F0F0Fu;
                        a[1] = w1[j] & 0x0F0F0F0Fu;
                        a[2] = (w0[j] >> 4) & 0x0F0F0F0Fu;
                        a[3] = (w1[j] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint4 q = bq[mt][j >> 1];
                            imma_16832(c[mt], a, (j & 1) ? q.z : q.x, (j & 1) ? q.w : q.y);
                        }
                    }
                    const float d0 = h2f_bits(meta0 & 0xffffu), b0 = h2f_bits(meta0 >> 16);
                    const float d1 = h2f_bits(meta1 & 0xffffu), b1 = h2f_bits(meta1 >> 16);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        // columns 2t (limb 0) and 2t+1 (limb 1) hold this thread's block: exact integers
                        const float dot0 = fmaf((float)c[mt][1], 1.0f / kLimb1Ratio, (float)c[mt][0]);
                        const float dot1 = fmaf((float)c[mt][3], 1.0f / kLimb1Ratio, (float)c[mt][2]);
                        acc[mt][0] = fmaf(d0 * info[mt].x, dot0, fmaf(b0, info[mt].y, acc[mt][0]));
                        acc[mt][1] = fmaf(d1 * info[mt].x, dot1, fmaf(b1, info[mt].y, acc[mt][1]));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                gs += ngr;
            }
            if (!ok) break;

            // each thread of a quad covered blocks = t (mod 4): add the four
            float v[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float s = acc[mt][r];
                    s += __shfl_xor_sync(kFull, s, 1);
                    s += __shfl_xor_sync(kFull, s, 2);
                    v[mt][r] = s;
                }
            }
            const bool complete = (g0 == 0 && g1 == q.kg);
            const uint32_t rowa = tile * kGemvTileRows + warp * 16 + g, rowb = rowa + 8;
            const float* bra = q.lb + (size_t)(rowa < q.n ? rowa : 0) * q.rank;
            const float* brb = q.lb + (size_t)(rowb < q.n ? rowb : 0) * q.rank;
            // first 16 rank columns of B (four per quad lane), requested before the fix-up wait so that
            // the two round trips overlap
            float ba0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, bb0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (q.rank && (complete || g0 == 0)) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t j = t + 4 * u;
                    if (j < q.rank) { ba0[u] = __ldg(bra + j); bb0[u] = __ldg(brb + j); }
                }
            }
            if (!complete && g0 != 0) {
                // Contributor: this CTA's range starts inside the tile, so this is its first segment.
                // Publish the partial sums as tagged messages and go on; no reply is needed.
                uint2* dst = reinterpret_cast<uint2*>(p.partials) + ((size_t)blockIdx.x * kGemvTileRows + warp * 16) * MT;
                if (t == 0) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        msg_store(dst + g * MT + mt, v[mt][0], tag);
                        msg_store(dst + (g + 8) * MT + mt, v[mt][1], tag);
                    }
                }
                continue;
            }
            if (!complete) {
                // Finisher: the CTA that owns the tile's first k part reaches it at the END of its own
                // range, when the contributors (who met the tile at the START of theirs) are long done.
                // The wait below is bounded and normally falls through at once.
                const uint32_t c_last = cta0 + owner_of((uint64_t)(tile + 1) * q.kg - 1, total, G);
                // Every thread fetches the messages of its own two rows from each contributor (the four
                // threads of a quad read the same words); the loop is warp-uniform, so the warp never
                // splits, and contributors are added in CTA order: the sum does not depend on arrival order.
                constexpr int CB = 4;                          // contributors polled together
                bool good = true;
                for (uint32_t c0 = blockIdx.x + 1; c0 <= c_last && good; c0 += CB) {
                    uint2 msg[CB][2 * MT];
                    const long long t0 = wait_clock();
                    for (;;) {
                        bool all = true;
#pragma unroll
                        for (int cb = 0; cb < CB; ++cb) {
                            if (c0 + cb > c_last) continue;
                            const uint2* src = reinterpret_cast<const uint2*>(p.partials) +
                                               ((size_t)(c0 + cb) * kGemvTileRows + warp * 16) * MT;
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                msg[cb][2 * mt] = msg_load(src + g * MT + mt);
                                msg[cb][2 * mt + 1] = msg_load(src + (g + 8) * MT + mt);
                            }
                        }
                        // all loads of a sweep are in flight together; the tags are looked at afterwards
#pragma unroll
                        for (int cb = 0; cb < CB; ++cb) {
                            if (c0 + cb > c_last) continue;
#pragma unroll
                            for (int i = 0; i < 2 * MT; ++i) all = all && msg[cb][i].y == tag;
                        }
                        if (__all_sync(kFull, all)) break;
                        if (__any_sync(kFull, wait_expired(t0))) { good = false; break; }
                    }
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb) {
                        if (c0 + cb > c_last) continue;
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            v[mt][0] += __uint_as_float(msg[cb][2 * mt].x);
                            v[mt][1] += __uint_as_float(msg[cb][2 * mt + 1].x);
                        }
                    }
                }
                if (!good && lane == 0) atomicOr(p.status, kDevErrGridWaitTimeout);
            }

            // epilogue: LoRA term (the quad splits the rank), then quad thread t stores token t
            if (q.rank) {
                if (!t_loaded) gather_t();
                float la[MT], lb2[MT];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) la[mt] = lb2[mt] = 0.0f;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t j = t + 4 * u;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const float tv = j < q.rank ? t_sm[mt * q.rank + j] : 0.0f;
                        la[mt] = fmaf(ba0[u], tv, la[mt]);
                        lb2[mt] = fmaf(bb0[u], tv, lb2[mt]);
                    }
                }
#pragma unroll 4
                for (uint32_t j = t + 16; j < q.rank; j += 4) {
                    const float ba = __ldg(bra + j), bb = __ldg(brb + j);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const float tv = t_sm[mt * q.rank + j];
                        la[mt] = fmaf(ba, tv, la[mt]);
                        lb2[mt] = fmaf(bb, tv, lb2[mt]);
                    }
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    la[mt] += __shfl_xor_sync(kFull, la[mt], 1);
                    la[mt] += __shfl_xor_sync(kFull, la[mt], 2);
                    lb2[mt] += __shfl_xor_sync(kFull, lb2[mt], 1);
                    lb2[mt] += __shfl_xor_sync(kFull, lb2[mt], 2);
                    v[mt][0] += q.lscale * la[mt];
                    v[mt][1] += q.lscale * lb2[mt];
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                if (mt != t || (uint32_t)mt >= q.m) continue;
                if (rowa < q.n) store_out(q, (size_t)mt * q.ldy + rowa, v[mt][0]);
                if (rowb < q.n) store_out(q, (size_t)mt * q.ldy + rowb, v[mt][1]);
            }
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, kDevErrBarrierTimeout);
            s_err = 1;
        }
    }

    // After a failed wait some TMA loads may still be in flight towards this CTA's shared
    // memory: wait (bounded) for the stages that were issued before leaving.
    __syncthreads();
    if (tid == 0) {
        gather_done(p, blockIdx.x, gridDim.x);
        launch_done(p.tsync, blockIdx.x, gridDim.x);
    }
    if (s_err && warp == 8 && lane == 0) {
        const uint32_t first = issued > NST ? issued - NST : 0;
        for (uint32_t j = first; j < issued; ++j) mbar_wait(&full[j % NST], (j / NST) & 1u);
    }
}

// ---- host: tensor maps ----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Weights as a 2-D tensor of 4-byte elements: inner = k/32*5 words per row, outer = n rows.
bool make_weight_map(CUtensorMap* map, const uint8_t* w, uint32_t n, uint32_t kb, uint32_t box_blocks) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)kb * 5, (cuuint64_t)n};
    const cuuint64_t strides[1] = {(cuuint64_t)kb * kBlockBytes};
    const cuuint32_t box[2] = {box_blocks * 5, (cuuint32_t)kGemvTileRows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(w), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

template <int MT, int NP>
cudaError_t launch_mt(const DecodeArgs<NP>& ga, size_t smem, int grid, cudaStream_t s) {
    auto kern = decode_kernel<MT, NP>;
    static DeviceOnce once;            // the shared-memory opt-in is per device and per kernel instantiation
    {
        cudaError_t e = opt_in_smem(reinterpret_cast<const void*>(kern), kMaxSmem - 1024, once);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (ga.p[0].use_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kern, ga);
}

// Single problems of up to four tokens (the library's own dispatch sends only one token here; the
// allocation-free entry point uses all four); groups are one token per problem.
cudaError_t launch_args(const DecodeArgs<1>& ga, size_t smem, int grid, cudaStream_t s) {
    switch (ga.p[0].m) {
        case 1: return launch_mt<1, 1>(ga, smem, grid, s);
        case 2: return launch_mt<2, 1>(ga, smem, grid, s);
        case 3: return launch_mt<3, 1>(ga, smem, grid, s);
        case 4: return launch_mt<4, 1>(ga, smem, grid, s);
        default: return cudaErrorInvalidValue;
    }
}
cudaError_t launch_args(const DecodeArgs<kMaxGroup>& ga, size_t smem, int grid, cudaStream_t s) {
    if (ga.p[0].m != 1) return cudaErrorInvalidValue;
    return launch_mt<1, kMaxGroup>(ga, smem, grid, s);
}

}  // namespace

namespace dec {
void split_ctas(const GemvParams* ps, uint32_t count, uint32_t grid, uint32_t* cta_begin, uint32_t tile_charge) {
    // fix-up and epilogue of a tile, in work units (a work unit streams in about 0.24 us).  Measured on the
    // large-layer set: 8 suits a launch per set, whose tail the next launch covers; the step kernel, where a
    // CTA walks straight into the next group and the shares inside a problem carry a charge of their own,
    // passes 5 (LQ4_TILE_CHARGE overrides both).
    static const int env_charge = [] {
        const char* e = getenv("LQ4_TILE_CHARGE");
        return e ? atoi(e) : -1;
    }();
    const uint64_t kTileCharge = env_charge >= 0 ? (uint64_t)env_charge : (uint64_t)tile_charge;
    constexpr uint32_t kMaxSplit = 32;           // problems of one launch: a group (8) or a step's group (24)
    if (count > kMaxSplit) count = kMaxSplit;
    uint64_t cost[kMaxSplit], units[kMaxSplit];
    uint32_t n[kMaxSplit];
    for (uint32_t i = 0; i < count; ++i) {
        units[i] = (uint64_t)ps[i].tiles * ps[i].kg;
        cost[i] = (uint64_t)ps[i].tiles * (ps[i].kg + kTileCharge);
        n[i] = 1;
    }
    for (uint32_t left = grid > count ? grid - count : 0; left > 0; --left) {
        // the next CTA goes to the problem whose CTAs carry the most
        uint32_t best = count;
        for (uint32_t i = 0; i < count; ++i) {
            if (n[i] >= units[i]) continue;
            if (best == count || cost[i] * n[best] > cost[best] * n[i]) best = i;
        }
        if (best == count) break;
        ++n[best];
    }
    cta_begin[0] = 0;
    for (uint32_t i = 0; i < count; ++i) cta_begin[i + 1] = cta_begin[i] + n[i];
}
// Encoding a tensor map costs about a microsecond of host time and weights are long-lived, so
// the three maps of a payload are kept in a per-thread direct-mapped cache keyed by
// (pointer, n, k).
const MapEntry* maps_for(const uint8_t* w, uint32_t n, uint32_t kb) {
    constexpr uint32_t kSlots = 512;
    thread_local MapEntry* cache = nullptr;
    if (!cache) cache = new MapEntry[kSlots]();
    uint64_t h = reinterpret_cast<uintptr_t>(w) * 0x9E3779B97F4A7C15ull;
    h ^= ((uint64_t)n << 32 | kb) * 0xC2B2AE3D27D4EB4Full;
    MapEntry& e = cache[(h >> 40) % kSlots];
    if (e.w == w && e.n == n && e.kb == kb) return &e;
    e.w = nullptr;
    if (!make_weight_map(&e.m[0], w, n, kb, 20) || !make_weight_map(&e.m[1], w, n, kb, 12) ||
        !make_weight_map(&e.m[2], w, n, kb, 4))
        return nullptr;
    e.w = w; e.n = n; e.kb = kb;
    return &e;
}

}  // namespace dec

size_t decode_plan_smem(GemvParams& p) {
    if (p.m == 0 || p.m > 4 || p.kb == 0 || p.kb % kGemvGranuleBlocks != 0) return 0;
    const uint32_t MT = p.m;
    uint32_t off = 2 * kMaxStages * 8 + 128;      // mbarriers, then the block of zeros
    p.off_t = off;                                // t = A x of the problem being finished
    off += align_up(p.m * p.rank * 4, 128);
    p.off_xrot = 0;
    if (p.signs) {
        p.off_xrot = off;
        off += align_up(p.m * p.k * 4, 128);
    }
    p.off_xs = off;
    off += align_up(p.kb * MT * 64, 128);
    p.off_sx = off;
    off += align_up(p.kb * MT * 8, 128);
    p.off_stage = off;
    const uint32_t budget = (uint32_t)kMaxSmem - 1024;    // static shared memory and driver reserve
    if (off + 2 * kSlotBytes > budget) return 0;
    uint32_t nst = (budget - off) / kSlotBytes;
    if (nst > 4) nst = 4;
    p.nstages = nst;
    p.kg = p.kb / kGemvGranuleBlocks;
    // Whole tiles per CTA need no cross-CTA sums; take that when it keeps at least 88 % of the SMs busy.
    const uint64_t sms = p.sm_count > 0 ? (uint64_t)p.sm_count : 148;
    const uint64_t rounds = (p.tiles + sms - 1) / sms;
    p.whole_tiles = (rounds > 0 && (double)p.tiles / (double)(rounds * sms) >= 0.88) ? 1u : 0u;
    return (size_t)off + (size_t)nst * kSlotBytes;
}

uint64_t decode_units(const GemvParams& p) { return p.whole_tiles ? (uint64_t)p.tiles : (uint64_t)p.tiles * p.kg; }

cudaError_t launch_decode(const GemvParams& p, size_t smem, int grid, cudaStream_t s) {
    const MapEntry* e = maps_for(p.w, p.n, p.kb);
    if (!e) return cudaErrorInvalidValue;
    DecodeArgs<1> ga{};
    ga.p[0] = p;
    for (int i = 0; i < 3; ++i) ga.maps[0][i] = e->m[i];
    ga.cta_begin[0] = 0;
    ga.cta_begin[1] = (uint32_t)grid;
    ga.dot_start[0] = 0;
    ga.dot_start[1] = p.m * p.rank * p.tsplit;
    ga.count = 1;
    ga.any_rank = p.rank != 0;
    return launch_args(ga, smem, grid, s);
}

size_t decode_group_plan_smem(GemvParams* ps, uint32_t count) {
    if (count == 0 || count > (uint32_t)kMaxGroup) return 0;
    const uint32_t MT = ps[0].m;
    if (MT != 1) return 0;
    uint32_t max_kb = 0;
    for (uint32_t i = 0; i < count; ++i) {
        const GemvParams& p = ps[i];
        if (p.m != MT || p.kb == 0 || p.kb % kGemvGranuleBlocks != 0 || p.signs) return 0;
        max_kb = p.kb > max_kb ? p.kb : max_kb;
    }
    uint32_t off = 2 * kMaxStages * 8 + 128;      // mbarriers, then the block of zeros
    uint32_t max_t = 0;
    for (uint32_t i = 0; i < count; ++i) max_t = ps[i].m * ps[i].rank > max_t ? ps[i].m * ps[i].rank : max_t;
    const uint32_t off_t = off;
    off += align_up(max_t * 4, 128);
    const uint32_t off_xs = off;
    off += align_up(max_kb * MT * 64, 128);
    const uint32_t off_sx = off;
    off += align_up(max_kb * MT * 8, 128);
    const uint32_t budget = (uint32_t)kMaxSmem - 1024;
    if (off + 2 * kSlotBytes > budget) return 0;
    uint32_t nst = (budget - off) / kSlotBytes;
    if (nst > 4) nst = 4;
    for (uint32_t i = 0; i < count; ++i) {
        GemvParams& p = ps[i];
        p.off_xrot = 0;
        p.off_t = off_t;
        p.off_xs = off_xs;
        p.off_sx = off_sx;
        p.off_stage = off;
        p.nstages = nst;
        p.kg = p.kb / kGemvGranuleBlocks;
        p.whole_tiles = 0;
    }
    return (size_t)off + (size_t)nst * kSlotBytes;
}

uint64_t decode_group_units(const GemvParams* ps, uint32_t count) {
    uint64_t total = 0;
    for (uint32_t i = 0; i < count; ++i) total += (uint64_t)ps[i].tiles * ps[i].kg;
    return total;
}

cudaError_t launch_decode_group(const GemvParams* ps, uint32_t count, size_t smem, int grid, cudaStream_t s) {
    if (count == 0 || count > (uint32_t)kMaxGroup) return cudaErrorInvalidValue;
    // the argument block is a few kilobytes: keep it off the stack of deep callers
    thread_local DecodeArgs<kMaxGroup> ga;
    ga.count = count;
    ga.any_rank = 0;
    split_ctas(ps, count, (uint32_t)grid, ga.cta_begin);
    for (uint32_t i = count; i < (uint32_t)kMaxGroup; ++i) ga.cta_begin[i + 1] = ga.cta_begin[count];
    ga.dot_start[0] = 0;
    for (uint32_t i = 0; i < (uint32_t)kMaxGroup; ++i) {
        const GemvParams& p = ps[i < count ? i : count - 1];
        ga.p[i] = p;
        if (i < count) {
            const MapEntry* e = maps_for(p.w, p.n, p.kb);
            if (!e) return cudaErrorInvalidValue;
            for (int j = 0; j < 3; ++j) ga.maps[i][j] = e->m[j];
            ga.dot_start[i + 1] = ga.dot_start[i] + p.m * p.rank * p.tsplit;
            ga.any_rank |= p.rank != 0;
        } else {
            ga.dot_start[i + 1] = ga.dot_start[i];
        }
    }
    return launch_args(ga, smem, grid, s);
}

}  // namespace lq4
