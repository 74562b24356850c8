// Decode kernel for 2..16 tokens (and for one token whose row is too long to sit in shared
// memory): y[m, n] = x[m, k] * Wq4[n, k]^T (+ LoRA).
//
// HBM-bound like the one-token kernel, and built on the same frame: one persistent CTA per SM, a
// producer warp that streams 128-row weight stages with TMA into a shared-memory ring, eight
// consumer warps of 16 rows each, stream-K work split in units of 4 blocks x 128 rows with
// tagged 8-byte messages for the partial sums of shared tiles.  What differs is the MMA mapping:
//  * One u8 x s8 warp MMA (m16n8k32) covers ONE Q4 block (its 32 codes are the k dimension) of 16
//    rows for FOUR tokens: the eight B columns are (token 0..3) x (limb 0, limb 1).  Nothing in
//    the operand is padding, so a block costs one MMA per four tokens.
//  * Each thread then owns the exact integer dot products of its token (quad lane) for two rows
//    and applies that block's scale and bias at once: acc += d * s * (c0 + c1 / 254) + b * sum(x).
//  * The int8 limbs of the activations are prepared once per call by a small kernel (which also
//    projects the LoRA adapter) into per-block records in global memory; the producer copies the
//    records of a stage's blocks beside its weights with one bulk copy.  The token count does not
//    limit k.
#include "lq4_decode_common.cuh"

namespace lq4 {

namespace {

using namespace gemv;
using namespace dec;

// Activation record of one Q4 block for NG groups of four tokens:
//   NG x [half 0 | half 1][column g = 2 * token + limb][4 bytes per quad lane t]  (256 B per group)
//   NG x 4 x {scale, sum}                                                          (32 B per group)
// Half 0 holds the activations that meet the low nibbles of block bytes 4t..4t+3 (k = 8t+0,2,4,6),
// half 1 those of the high nibbles (k = 8t+1,3,5,7): the order of the MMA's k slots.
__host__ __device__ constexpr uint32_t rec_bytes(uint32_t ng) { return ng * 288u; }

struct PrepArgs {
    const void* x[kMaxGroup];
    const float* x_mul[kMaxGroup];           // non-NULL: the input is silu(x) * x_mul, rows ldx floats apart
    uint32_t ldx[kMaxGroup];
    const float* la[kMaxGroup];
    float* t[kMaxGroup];
    uint8_t* rec[kMaxGroup];
    uint32_t k[kMaxGroup], rank[kMaxGroup];
    uint32_t limb_start[kMaxGroup + 1];     // first CTA of each problem's limb work
    uint32_t proj_start[kMaxGroup + 1];     // first CTA (after all limb CTAs) of each problem's projection
    int32_t x_dtype[kMaxGroup], vec4[kMaxGroup];
    uint32_t count, m, ng;
    int32_t use_pdl;
    const unsigned long long* wait_arrive;   // x holds gathered results: wait for the peers first (wait_world > 1)
    uint32_t wait_world;
    int32_t* status;
};

// Limb records for every (block, token slot) and t = A x for every adapter, in one launch.
__global__ void __launch_bounds__(256) dense_prep_kernel(const __grid_constant__ PrepArgs a) {
    // The decode kernel behind this one may start at once: it only streams weights until it has
    // waited for this grid, which in turn waits here for whatever produced x.
    if (a.use_pdl) {
        pdl_launch_dependents();
        pdl_wait_prior_grids();
    }
    if (a.wait_world > 1) {               // one thread polls the arrival counter, the CTA follows
        if (threadIdx.x == 0 && !wait_gather_arrivals(a.wait_arrive, a.wait_world)) atomicOr(a.status, kDevErrGridWaitTimeout);
        __syncthreads();
    }
    const uint32_t nlimb = a.limb_start[a.count];
    if (blockIdx.x >= nlimb) {
        const uint32_t b = blockIdx.x - nlimb;
        uint32_t pi = 0;
        while (pi + 1 < a.count && b >= a.proj_start[pi + 1]) ++pi;
        project_one(a.x[pi], a.x_dtype[pi], a.k[pi], a.la[pi], a.rank[pi], a.t[pi], b - a.proj_start[pi], a.vec4[pi],
                    a.x_mul[pi], a.ldx[pi]);
        return;
    }
    uint32_t pi = 0;
    while (pi + 1 < a.count && blockIdx.x >= a.limb_start[pi + 1]) ++pi;
    const uint32_t slots = a.ng * 4, K = a.k[pi], kb = K / 32;
    const uint32_t idx = (blockIdx.x - a.limb_start[pi]) * 256 + threadIdx.x;
    const uint32_t t = idx & 3, slot = (idx >> 2) % slots, blk = (idx >> 2) / slots;
    const bool in_range = blk < kb;              // whole quads are in or out together
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    if (in_range && slot < a.m) {
        if (a.x_mul[pi]) {                       // gated input: silu(gate) * up, f32
            const size_t at = (size_t)slot * a.ldx[pi] + (size_t)blk * 32 + t * 8;
            float up[8];
            load8(a.x[pi], LQ4_DTYPE_F32, at, v);
            load8(a.x_mul[pi], LQ4_DTYPE_F32, at, up);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = silu_mul(v[i], up[i]);
        } else {
            load8(a.x[pi], a.x_dtype[pi], (size_t)slot * K + (size_t)blk * 32 + t * 8, v);
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
    sum += __shfl_xor_sync(kFull, sum, 1);
    sum += __shfl_xor_sync(kFull, sum, 2);
    if (!in_range) return;
    const Limbs8 l = make_limbs8(v, amax);
    uint8_t* rec = a.rec[pi] + (size_t)blk * rec_bytes(a.ng);
    uint8_t* grp = rec + (slot >> 2) * 256 + (slot & 3) * 32 + t * 4;      // column g = 2 * (slot & 3): 16 B per column
    *reinterpret_cast<uint32_t*>(grp) = l.l0a;
    *reinterpret_cast<uint32_t*>(grp + 128) = l.l0b;
    *reinterpret_cast<uint32_t*>(grp + 16) = l.l1a;
    *reinterpret_cast<uint32_t*>(grp + 16 + 128) = l.l1b;
    if (t == 0) *reinterpret_cast<float2*>(rec + a.ng * 256 + slot * 8) = make_float2(l.scale, sum);
}

template <int NG>
__host__ __device__ constexpr uint32_t dense_slot_bytes() { return kSlotBytes + kBigBlocks * rec_bytes(NG); }

template <int NG, int NP>
__global__ void __launch_bounds__(kGemvThreads, 1) dense_kernel(const __grid_constant__ DecodeArgs<NP> ga) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    __shared__ int s_err;
    constexpr uint32_t kSlot = dense_slot_bytes<NG>();
    constexpr uint32_t kRec = rec_bytes(NG);

    const GemvParams& p = ga.p[0];
    const uint32_t count = NP == 1 ? 1u : ga.count;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t NST = p.nstages;
    if (tid == 0) {
        for (uint32_t s = 0; s < NST; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 8);
        }
        s_err = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // The limb records and t come from the launch before this one, but the weights do not: the
    // producer starts streaming them at once and waits for that launch only before it copies the
    // first records; the consumers wait for it before they touch anything.
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
    const uint64_t r0 = range_begin(cl, total, G), r1 = range_begin(cl + 1, total, G);
    uint32_t issued = 0;

    if (warp == 8) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            const uint64_t pol = l2_policy_evict_first();
            uint32_t it = 0;
            bool ok = true;
            // The first weight stage is requested before the previous launch is known to be done; its
            // records follow as soon as it is (and go out before the later weight stages, which would
            // otherwise sit in front of them in the copy queue).
            struct Pending { uint8_t* dst; const uint8_t* src; uint32_t bytes; uint64_t* bar; } pend[kMaxStages];
            uint32_t npend = 0;
            bool prior_done = !p.use_pdl;
            auto flush = [&]() {
                pdl_wait_prior_grids();
                prior_done = true;
                for (uint32_t i = 0; i < npend; ++i) bulk_g2s(pend[i].dst, pend[i].src, pend[i].bytes, pend[i].bar);
                npend = 0;
            };
            for (uint64_t pos = r0; pos < r1 && ok;) {
                const uint32_t tile = (uint32_t)(pos / q.kg);
                const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * q.kg);
                const uint64_t left = r1 - pos;
                const uint32_t g1 = (uint64_t)(q.kg - g0) < left ? q.kg : (uint32_t)(g0 + left);
                for (uint32_t gs = g0; gs < g1; ++it) {
                    const uint32_t ngr = stage_granules(g1 - gs);
                    const uint32_t s = it % NST;
                    if (!mbar_wait(&empty[s], ((it / NST) & 1u) ^ 1u)) { ok = false; break; }
                    uint8_t* st = smem + p.off_stage + (size_t)s * kSlot;
                    const uint32_t xbytes = ngr * kGemvGranuleBlocks * kRec;
                    mbar_arrive_expect_tx(&full[s], ngr * kSmallBytes + xbytes);
                    tma_load_2d(st, &ga.maps[pi][ngr == 5 ? 0 : (ngr == 3 ? 1 : 2)], (int32_t)(gs * kGemvGranuleBlocks * 5),
                                (int32_t)(tile * kGemvTileRows), &full[s], pol);
                    const uint8_t* xsrc = q.xs_g + (size_t)gs * kGemvGranuleBlocks * kRec;
                    if (prior_done) {
                        bulk_g2s(st + kSlotBytes, xsrc, xbytes, &full[s]);
                    } else {
                        pend[npend++] = Pending{st + kSlotBytes, xsrc, xbytes, &full[s]};
                        if (npend == 1) flush();
                    }
                    gs += ngr;
                }
                pos += g1 - g0;
            }
            if (!prior_done) flush();
            issued = it;
            if (!ok) {
                atomicOr(p.status, kDevErrBarrierTimeout);
                s_err = 1;
            }
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int g = lane >> 2, t = lane & 3;
        if (p.use_pdl) pdl_wait_prior_grids();
        const uint32_t tag = launch_tag(p.tsync);
        uint32_t it = 0;
        bool ok = true;
        for (uint64_t pos = r0; pos < r1 && ok;) {
            const uint32_t tile = (uint32_t)(pos / q.kg);
            const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * q.kg);
            const uint64_t left = r1 - pos;
            const uint32_t g1 = (uint64_t)(q.kg - g0) < left ? q.kg : (uint32_t)(g0 + left);
            pos += g1 - g0;

            float acc[NG][2];
#pragma unroll
            for (int i = 0; i < NG; ++i) acc[i][0] = acc[i][1] = 0.0f;
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
                const uint8_t* st = smem + p.off_stage + (size_t)s * kSlot;
                const uint8_t* row0 = st + (warp * 16 + g) * rs;
                const uint8_t* row1 = row0 + 8 * rs;
                const uint8_t* xrec = st + kSlotBytes + g * 16 + t * 4;
                const uint8_t* info = st + kSlotBytes + NG * 256 + t * 8;
                const uint32_t nblk = ngr * kGemvGranuleBlocks;
#pragma unroll 4
                for (uint32_t bi = 0; bi < nblk; ++bi) {
                    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(row0 + bi * kBlockBytes);
                    const uint32_t* q1 = reinterpret_cast<const uint32_t*>(row1 + bi * kBlockBytes);
                    const uint32_t meta0 = q0[0], meta1 = q1[0];
                    const uint32_t w0 = q0[1 + t], w1 = q1[1 + t];
                    // low nibbles fill k slots 4t..4t+3, high nibbles slots 16+4t..16+4t+3
                    uint32_t a[4];
                    a[0] = w0 & 0x0F0F0F0Fu;
                    a[1] = w1 & 0x0F0F0F0Fu;
                    a[2] = (w0 >> 4) & 0x0F0F0F0Fu;
                    a[3] = (w1 >> 4) & 0x0F0F0F0Fu;
                    const float d0 = h2f_bits(meta0 & 0xffffu), b0 = h2f_bits(meta0 >> 16);
                    const float d1 = h2f_bits(meta1 & 0xffffu), b1 = h2f_bits(meta1 >> 16);
                    const uint8_t* xr = xrec + bi * kRec;
                    const uint8_t* ir = info + bi * kRec;
#pragma unroll
                    for (int ng = 0; ng < NG; ++ng) {
                        int c[4] = {0, 0, 0, 0};
                        imma_16832(c, a, *reinterpret_cast<const uint32_t*>(xr + ng * 256),
                                   *reinterpret_cast<const uint32_t*>(xr + ng * 256 + 128));
                        const float2 sx = *reinterpret_cast<const float2*>(ir + ng * 32);   // token 4 ng + t
                        // columns 2t (limb 0) and 2t+1 (limb 1) belong to this thread's token: exact integers
                        const float dot0 = fmaf((float)c[1], 1.0f / kLimb1Ratio, (float)c[0]);
                        const float dot1 = fmaf((float)c[3], 1.0f / kLimb1Ratio, (float)c[2]);
                        acc[ng][0] = fmaf(d0 * sx.x, dot0, fmaf(b0, sx.y, acc[ng][0]));
                        acc[ng][1] = fmaf(d1 * sx.x, dot1, fmaf(b1, sx.y, acc[ng][1]));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                gs += ngr;
            }
            if (!ok) break;

            // thread (g, t) holds rows g and g+8 of the warp's 16 for tokens 4 ng + t
            const bool complete = (g0 == 0 && g1 == q.kg);
            constexpr uint32_t kTok = NG * 4;
            if (!complete && g0 != 0) {
                // Contributor: the range of this CTA starts inside the tile (its first segment);
                // publish the partial sums and go on.
                uint2* dst = reinterpret_cast<uint2*>(p.partials) + ((size_t)blockIdx.x * kGemvTileRows + warp * 16) * kTok;
#pragma unroll
                for (int ng = 0; ng < NG; ++ng) {
                    msg_store(dst + g * kTok + ng * 4 + t, acc[ng][0], tag);
                    msg_store(dst + (g + 8) * kTok + ng * 4 + t, acc[ng][1], tag);
                }
                continue;
            }
            if (!complete) {
                // Finisher: owns the tile's first k part and meets it at the END of its range, when the
                // contributors (who met it at the START of theirs) are normally done.  Bounded wait.
                const uint32_t c_last = cta0 + owner_of((uint64_t)(tile + 1) * q.kg - 1, total, G);
                constexpr int CB = NG == 1 ? 8 : 4;     // contributors polled together
                bool good = true;
                for (uint32_t c0 = blockIdx.x + 1; c0 <= c_last && good; c0 += CB) {
                    uint2 msg[CB][2 * NG];
                    const long long t0 = wait_clock();
                    for (;;) {
                        bool all = true;
#pragma unroll
                        for (int cb = 0; cb < CB; ++cb) {
                            if (c0 + cb > c_last) continue;
                            const uint2* src = reinterpret_cast<const uint2*>(p.partials) +
                                               ((size_t)(c0 + cb) * kGemvTileRows + warp * 16) * kTok;
#pragma unroll
                            for (int ng = 0; ng < NG; ++ng) {
                                msg[cb][2 * ng] = msg_load(src + g * kTok + ng * 4 + t);
                                msg[cb][2 * ng + 1] = msg_load(src + (g + 8) * kTok + ng * 4 + t);
                            }
                        }
#pragma unroll
                        for (int cb = 0; cb < CB; ++cb) {
                            if (c0 + cb > c_last) continue;
#pragma unroll
                            for (int i = 0; i < 2 * NG; ++i) all = all && (msg[cb][i].y == tag);
                        }
                        if (__all_sync(kFull, all)) break;                 // warp-uniform: the warp never splits
                        if (__any_sync(kFull, wait_expired(t0))) { good = false; break; }
                    }
                    // contributors are added in CTA order: the sum does not depend on arrival order
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb) {
                        if (c0 + cb > c_last) continue;
#pragma unroll
                        for (int ng = 0; ng < NG; ++ng) {
                            acc[ng][0] += __uint_as_float(msg[cb][2 * ng].x);
                            acc[ng][1] += __uint_as_float(msg[cb][2 * ng + 1].x);
                        }
                    }
                }
                if (!good && lane == 0) atomicOr(p.status, kDevErrGridWaitTimeout);
            }

            // epilogue: LoRA term for the thread's two rows and NG tokens, then the stores
            const uint32_t rowa = tile * kGemvTileRows + warp * 16 + g, rowb = rowa + 8;
            if (q.rank) {
                float la[NG], lb2[NG];
                const float* tt[NG];
#pragma unroll
                for (int ng = 0; ng < NG; ++ng) {
                    la[ng] = lb2[ng] = 0.0f;
                    const uint32_t tok = ng * 4 + t;
                    tt[ng] = q.t_g + (size_t)(tok < q.m ? tok : 0) * q.rank;
                }
                const float* bra = q.lb + (size_t)(rowa < q.n ? rowa : 0) * q.rank;
                const float* brb = q.lb + (size_t)(rowb < q.n ? rowb : 0) * q.rank;
                const bool vec = (q.rank & 3u) == 0 && ((reinterpret_cast<uintptr_t>(q.lb) | reinterpret_cast<uintptr_t>(q.t_g)) & 15u) == 0;
                if (vec) {
                    // 16-byte loads, eight rank columns per step and two steps in flight: the whole
                    // term costs one or two memory round trips instead of one per few columns
                    const float4* a4 = reinterpret_cast<const float4*>(bra);
                    const float4* b4 = reinterpret_cast<const float4*>(brb);
                    const uint32_t r4 = q.rank >> 2;
#pragma unroll 2
                    for (uint32_t j = 0; j < r4; j += 2) {
                        const bool two = j + 1 < r4;
                        const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        const float4 ba0 = __ldg(a4 + j), bb0 = __ldg(b4 + j);
                        const float4 ba1 = two ? __ldg(a4 + j + 1) : z, bb1 = two ? __ldg(b4 + j + 1) : z;
                        float4 t0[NG], t1[NG];
#pragma unroll
                        for (int ng = 0; ng < NG; ++ng) {
                            const float4* t4 = reinterpret_cast<const float4*>(tt[ng]);
                            t0[ng] = __ldcg(t4 + j);
                            t1[ng] = two ? __ldcg(t4 + j + 1) : z;
                        }
#pragma unroll
                        for (int ng = 0; ng < NG; ++ng) {
                            la[ng] = fmaf(ba0.x, t0[ng].x, fmaf(ba0.y, t0[ng].y, fmaf(ba0.z, t0[ng].z, fmaf(ba0.w, t0[ng].w, la[ng]))));
                            la[ng] = fmaf(ba1.x, t1[ng].x, fmaf(ba1.y, t1[ng].y, fmaf(ba1.z, t1[ng].z, fmaf(ba1.w, t1[ng].w, la[ng]))));
                            lb2[ng] = fmaf(bb0.x, t0[ng].x, fmaf(bb0.y, t0[ng].y, fmaf(bb0.z, t0[ng].z, fmaf(bb0.w, t0[ng].w, lb2[ng]))));
                            lb2[ng] = fmaf(bb1.x, t1[ng].x, fmaf(bb1.y, t1[ng].y, fmaf(bb1.z, t1[ng].z, fmaf(bb1.w, t1[ng].w, lb2[ng]))));
                        }
                    }
                } else {
#pragma unroll 4
                    for (uint32_t j = 0; j < q.rank; ++j) {
                        const float ba = __ldg(bra + j), bb = __ldg(brb + j);
#pragma unroll
                        for (int ng = 0; ng < NG; ++ng) {
                            const float tv = __ldcg(tt[ng] + j);
                            la[ng] = fmaf(ba, tv, la[ng]);
                            lb2[ng] = fmaf(bb, tv, lb2[ng]);
                        }
                    }
                }
#pragma unroll
                for (int ng = 0; ng < NG; ++ng) {
                    acc[ng][0] += q.lscale * la[ng];
                    acc[ng][1] += q.lscale * lb2[ng];
                }
            }
#pragma unroll
            for (int ng = 0; ng < NG; ++ng) {
                const uint32_t tok = ng * 4 + t;
                if (tok >= q.m) continue;
                if (rowa < q.n) store_out(q, (size_t)tok * q.ldy + rowa, acc[ng][0]);
                if (rowb < q.n) store_out(q, (size_t)tok * q.ldy + rowb, acc[ng][1]);
            }
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, kDevErrBarrierTimeout);
            s_err = 1;
        }
    }

    __syncthreads();
    if (tid == 0) {
        gather_done(p, blockIdx.x, gridDim.x);
        launch_done(p.tsync, blockIdx.x, gridDim.x);
    }
    // After a failed wait some copies may still be in flight towards this CTA's shared memory:
    // wait (bounded) for the stages that were issued before leaving.
    if (s_err && warp == 8 && lane == 0) {
        const uint32_t first = issued > NST ? issued - NST : 0;
        for (uint32_t j = first; j < issued; ++j) mbar_wait(&full[j % NST], (j / NST) & 1u);
    }
}

template <int NG, int NP>
cudaError_t launch_ng(const DecodeArgs<NP>& ga, size_t smem, int grid, cudaStream_t s) {
    auto kern = dense_kernel<NG, NP>;
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

template <int NP>
cudaError_t launch_args(const DecodeArgs<NP>& ga, size_t smem, int grid, cudaStream_t s) {
    switch ((ga.p[0].m + 3) / 4) {
        case 1: return launch_ng<1, NP>(ga, smem, grid, s);
        case 2: return launch_ng<2, NP>(ga, smem, grid, s);
        case 3: return launch_ng<3, NP>(ga, smem, grid, s);
        case 4: return launch_ng<4, NP>(ga, smem, grid, s);
        default: return cudaErrorInvalidValue;
    }
}

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

}  // namespace

size_t dense_record_bytes(uint32_t m, uint32_t k) { return (size_t)(k / 32) * rec_bytes((m + 3) / 4); }

size_t dense_plan_smem(GemvParams* ps, uint32_t count) {
    if (count == 0 || count > (uint32_t)kMaxGroup) return 0;
    const uint32_t m = ps[0].m;
    if (m == 0 || m > (uint32_t)kGemvMaxM) return 0;
    const uint32_t ng = (m + 3) / 4;
    for (uint32_t i = 0; i < count; ++i)
        if (ps[i].m != m || ps[i].kb == 0 || ps[i].kb % kGemvGranuleBlocks != 0 || ps[i].signs) return 0;
    const uint32_t off = align_up(2 * kMaxStages * 8, 128);
    const uint32_t slot = kSlotBytes + kBigBlocks * rec_bytes(ng);
    const uint32_t budget = (uint32_t)kMaxSmem - 1024;
    uint32_t nst = (budget - off) / slot;
    if (nst < 2) return 0;
    if (nst > 4) nst = 4;
    for (uint32_t i = 0; i < count; ++i) {
        GemvParams& p = ps[i];
        p.off_stage = off;
        p.nstages = nst;
        p.kg = p.kb / kGemvGranuleBlocks;
        p.whole_tiles = 0;
    }
    return (size_t)off + (size_t)nst * slot;
}

cudaError_t launch_dense_prep(const GemvParams* ps, uint32_t count, uint8_t* const* rec, float* const* t, int use_pdl,
                              cudaStream_t s) {
    if (count == 0 || count > (uint32_t)kMaxGroup) return cudaErrorInvalidValue;
    PrepArgs a{};
    a.count = count;
    a.m = ps[0].m;
    a.ng = (ps[0].m + 3) / 4;
    a.use_pdl = use_pdl;
    a.wait_arrive = ps[0].wait_arrive;
    a.wait_world = ps[0].wait_world;
    a.status = ps[0].status;
    a.limb_start[0] = a.proj_start[0] = 0;
    for (uint32_t i = 0; i < count; ++i) {
        const GemvParams& p = ps[i];
        a.x[i] = p.x; a.x_dtype[i] = p.x_dtype; a.k[i] = p.k;
        a.x_mul[i] = p.x_mul; a.ldx[i] = p.ldx ? p.ldx : p.k;
        a.la[i] = p.la; a.rank[i] = p.rank; a.t[i] = t[i]; a.rec[i] = rec[i];
        a.vec4[i] = p.x_dtype == LQ4_DTYPE_F32 && p.k % 4 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(p.la) & 15) == 0;
        const uint32_t threads = p.kb * a.ng * 4 * 4;       // one quad per (block, token slot)
        a.limb_start[i + 1] = a.limb_start[i] + (threads + 255) / 256;
        a.proj_start[i + 1] = a.proj_start[i] + p.m * p.rank;
    }
    for (uint32_t i = count; i < (uint32_t)kMaxGroup; ++i) {
        a.limb_start[i + 1] = a.limb_start[count];
        a.proj_start[i + 1] = a.proj_start[count];
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(a.limb_start[count] + a.proj_start[count]);
    cfg.blockDim = dim3(256);
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
    return cudaLaunchKernelEx(&cfg, dense_prep_kernel, a);
}

cudaError_t launch_dense(const GemvParams* ps, uint32_t count, size_t smem, int grid, cudaStream_t s) {
    if (count == 0 || count > (uint32_t)kMaxGroup) return cudaErrorInvalidValue;
    if (count == 1) {
        const GemvParams& p = ps[0];
        const MapEntry* e = maps_for(p.w, p.n, p.kb);
        if (!e) return cudaErrorInvalidValue;
        DecodeArgs<1> ga{};
        ga.p[0] = p;
        for (int j = 0; j < 3; ++j) ga.maps[0][j] = e->m[j];
        ga.cta_begin[0] = 0;
        ga.cta_begin[1] = (uint32_t)grid;
        ga.dot_start[0] = ga.dot_start[1] = 0;
        ga.count = 1;
        ga.any_rank = p.rank != 0;
        return launch_args<1>(ga, smem, grid, s);
    }
    thread_local DecodeArgs<kMaxGroup> ga;
    ga.count = count;
    ga.any_rank = 0;
    split_ctas(ps, count, (uint32_t)grid, ga.cta_begin);
    for (uint32_t i = count; i < (uint32_t)kMaxGroup; ++i) ga.cta_begin[i + 1] = ga.cta_begin[count];
    for (uint32_t i = 0; i <= (uint32_t)kMaxGroup; ++i) ga.dot_start[i] = 0;
    for (uint32_t i = 0; i < (uint32_t)kMaxGroup; ++i) {
        const GemvParams& p = ps[i < count ? i : count - 1];
        ga.p[i] = p;
        if (i < count) {
            const MapEntry* e = maps_for(p.w, p.n, p.kb);
            if (!e) return cudaErrorInvalidValue;
            for (int j = 0; j < 3; ++j) ga.maps[i][j] = e->m[j];
            ga.any_rank |= p.rank != 0;
        }
    }
    return launch_args<kMaxGroup>(ga, smem, grid, s);
}

}  // namespace lq4
