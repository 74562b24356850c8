// Decode path (m <= 16): y[m, n] = x[m, k] * Wq4[n, k]^T (+ LoRA), HBM-bound.
//
// One persistent CTA per SM.  A producer warp streams the packed Q4 rows from HBM
// into a shared-memory ring with bulk async copies (one 320-byte piece per row and
// stage, completion on an mbarrier); eight consumer warps each own 16 of the tile's
// 128 output rows, turn the nibbles into exact f16 integers in registers and feed
// warp-level MMAs whose B operand holds the activations split into an f16 "hi" and
// an f16 "lo" limb (two columns per token).  Per Q4 block the 16x8 product is
// scaled by the block's f16 scale and the bias is applied through the block sum of
// the activations, all in f32:
//     y[row] += d * sum_k(q_k * x_k) + b * sum_k(x_k)
// which is the factorisation the reference's decode shader uses
// (crates/inference/src/forward/shaders/qwen35.metal:799-866).
//
// Work is split stream-K style: the (tile, k-granule) space is cut into equal
// contiguous ranges, one per CTA, so every CTA streams the same number of bytes.
// A tile whose k range is shared by several CTAs is finished by whichever of them
// arrives last; it adds the partial sums in CTA order, so the result does not
// depend on arrival order.
//
// The LoRA delta s * B (A x) is added in the tile epilogue.  In the resident
// variant (whole activation row kept in shared memory, m small) each CTA computes
// the partial projection A x over its own slice of k in the prologue and the CTAs
// exchange the partials through global memory; in the staged variant a small
// preparation kernel has produced the activation fragments and t = A x beforehand.
#include "lq4_gemv_common.cuh"

namespace lq4 {

namespace {

using namespace gemv;

// ---------------------------------------------------------------------------
// Resident-variant prologue, run by the 256 consumer threads: optional Hadamard
// rotation in shared memory, LoRA partial projection over this CTA's k slice,
// activation fragments for the whole row.
// ---------------------------------------------------------------------------
template <int NT>
__device__ void resident_prologue(const GemvParams& p, uint8_t* smem, int ctid) {
    const uint32_t K = p.k, M = p.m;
    const int cw = ctid >> 5, lane = ctid & 31;
    float* xrot = reinterpret_cast<float*>(smem + p.off_xrot);
    const bool rot = p.signs != nullptr;

    if (rot) {
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

    if (p.rank) {
        const uint64_t G = gridDim.x;
        const uint32_t k0 = (uint32_t)(((uint64_t)blockIdx.x * p.kb) / G) * 32;
        const uint32_t k1 = (uint32_t)(((uint64_t)(blockIdx.x + 1) * p.kb) / G) * 32;
        const uint32_t pairs = M * p.rank;
        for (uint32_t pr = cw; pr < pairs; pr += 8) {
            const uint32_t mm = pr / p.rank, j = pr - mm * p.rank;
            const float* arow = p.la + (size_t)j * K;
            float s = 0.0f;
            for (uint32_t kk = k0 + lane; kk < k1; kk += 32) {
                const float xv = rot ? xrot[mm * K + kk] : load_act(p.x, p.x_dtype, (size_t)mm * K + kk);
                s = fmaf(__ldg(arow + kk), xv, s);
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
            if (lane == 0) {
                p.tpart[(size_t)blockIdx.x * pairs + pr] = s;
                __threadfence();
            }
        }
        named_bar_sync(kBarConsumers, kConsumerThreads);
        if (ctid == 0) atomicAdd(p.tsync, 1u);
    }

    uint8_t* xs = smem + p.off_xs;
    float* sx = reinterpret_cast<float*>(smem + p.off_sx);
    const uint32_t noct = K / 8;
    for (uint32_t mp = 0; mp < NT * 4; ++mp) {
        if ((mp & 3) * 2 >= p.gmax) continue;
        for (uint32_t o0 = 0; o0 < noct; o0 += kConsumerThreads) {
            const uint32_t o = o0 + ctid;
            const bool active = o < noct;
            float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (active && mp < M) {
                if (rot) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = xrot[mp * K + o * 8 + i];
                } else {
                    load8(p.x, p.x_dtype, (size_t)mp * K + (size_t)o * 8, v);
                }
            }
            store_fragments(xs, sx, NT, p.gmax, mp, o, active, v, NT * 4);
        }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
}

template <int NT, bool RESIDENT>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_mma_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + 8;
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
        mbar_fence_init();
    }
    __syncthreads();
    if (p.use_pdl) pdl_launch_dependents();

    const uint64_t G = gridDim.x;
    const uint64_t total = (uint64_t)p.tiles * p.kg;
    const uint64_t r0 = range_begin(blockIdx.x, total, G), r1 = range_begin(blockIdx.x + 1, total, G);
    const uint32_t gmax = p.gmax;
    uint32_t issued = 0;   // producer: stages issued

    if (warp == 8) {
        // ------------------------------ producer ------------------------------
        const uint64_t pol = l2_policy_evict_first();
        if (!RESIDENT && p.use_pdl) pdl_wait_prior_grids();
        const size_t row_bytes = (size_t)p.kb * kBlockBytes;
        uint32_t it = 0;
        bool ok = true;
        for (uint64_t pos = r0; pos < r1 && ok;) {
            const uint32_t tile = (uint32_t)(pos / p.kg);
            const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * p.kg);
            const uint64_t left = r1 - pos;
            const uint32_t g1 = (uint64_t)(p.kg - g0) < left ? p.kg : (uint32_t)(g0 + left);
            const uint32_t rows_valid = min((uint32_t)kGemvTileRows, p.n - tile * kGemvTileRows);
            for (uint32_t gs = g0; gs < g1; gs += 4, ++it) {
                const uint32_t nbs = min(4u, g1 - gs) * kGemvGranuleBlocks;
                const uint32_t s = it % NST;
                if (!mbar_wait(&empty[s], ((it / NST) & 1u) ^ 1u)) { ok = false; break; }
                uint8_t* st = smem + p.off_stage + (size_t)s * p.stage_bytes;
                uint32_t bytes = rows_valid * nbs * kBlockBytes;
                if (!RESIDENT) bytes += nbs * NT * gmax * 64 + nbs * NT * 16;
                if (lane == 0) mbar_arrive_expect_tx(&full[s], bytes);
                __syncwarp();
                const uint8_t* src = p.w + (size_t)tile * kGemvTileRows * row_bytes + (size_t)gs * kGemvGranuleBlocks * kBlockBytes;
                for (uint32_t r = lane; r < rows_valid; r += 32)
                    bulk_g2s_evict_first(st + r * kGemvRowStride, src + r * row_bytes, nbs * kBlockBytes, &full[s], pol);
                if (!RESIDENT) {
                    const size_t blk0 = (size_t)gs * kGemvGranuleBlocks;
                    if (lane == 0)
                        bulk_g2s(st + p.off_stage_xs, p.xs_g + blk0 * NT * gmax * 64, nbs * NT * gmax * 64, &full[s]);
                    if (lane == 1)
                        bulk_g2s(st + p.off_stage_sx, p.sx_g + blk0 * NT * 4, nbs * NT * 16, &full[s]);
                }
            }
            pos += g1 - g0;
        }
        issued = it;
        if (!ok) {
            if (lane == 0) atomicOr(p.status, kDevErrBarrierTimeout);
            s_err = 1;
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int g = lane >> 2, t = lane & 3;
        float* t_s = reinterpret_cast<float*>(smem + p.off_t);
        if (RESIDENT) {
            if (p.use_pdl) pdl_wait_prior_grids();
            resident_prologue<NT>(p, smem, tid);
        } else if (p.rank) {
            if (p.use_pdl) pdl_wait_prior_grids();
            for (uint32_t i = tid; i < p.m * p.rank; i += kConsumerThreads) t_s[i] = p.t_g[i];
            named_bar_sync(kBarConsumers, kConsumerThreads);
        }
        bool t_ready = !(RESIDENT && p.rank);

        // Waits for every CTA's partial projection and sums them in CTA order.
        auto gather_t = [&]() {
            if (tid == 0) {
                const long long t0 = wait_clock();
                while (ld_acquire_u32(p.tsync) < (uint32_t)G) {
                    if (wait_expired(t0)) {
                        s_twait_failed = 1;
                        atomicOr(p.status, kDevErrGridWaitTimeout);
                        break;
                    }
                }
            }
            named_bar_sync(kBarConsumers, kConsumerThreads);
            const uint32_t pairs = p.m * p.rank;
            const bool failed = s_twait_failed != 0;
            for (uint32_t pr = tid; pr < pairs; pr += kConsumerThreads) {
                float s = 0.0f;
                if (!failed)
                    for (uint32_t c = 0; c < (uint32_t)G; ++c) s += __ldcg(p.tpart + (size_t)c * pairs + pr);
                t_s[pr] = s;
            }
            named_bar_sync(kBarConsumers, kConsumerThreads);
            if (tid == 0) {
                // the last CTA to finish reading re-arms both counters for the next launch
                const uint32_t old = atomicAdd(p.tsync + 1, 1u);
                if (old == (uint32_t)G - 1) {
                    p.tsync[0] = 0;
                    p.tsync[1] = 0;
                    __threadfence();
                }
            }
            t_ready = true;
        };

        uint32_t it = 0;
        bool ok = true;
        for (uint64_t pos = r0; pos < r1 && ok;) {
            const uint32_t tile = (uint32_t)(pos / p.kg);
            const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * p.kg);
            const uint64_t left = r1 - pos;
            const uint32_t g1 = (uint64_t)(p.kg - g0) < left ? p.kg : (uint32_t)(g0 + left);
            pos += g1 - g0;

            float acc[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

            for (uint32_t gs = g0; gs < g1; gs += 4, ++it) {
                const uint32_t nbs = min(4u, g1 - gs) * kGemvGranuleBlocks;
                const uint32_t s = it % NST;
                if (!mbar_wait(&full[s], (it / NST) & 1u)) { ok = false; break; }
                const uint8_t* st = smem + p.off_stage + (size_t)s * p.stage_bytes;
                const uint8_t* rowp = st + (warp * 16 + g) * kGemvRowStride;
                const uint8_t* xsb;
                const float* sxb;
                if (RESIDENT) {
                    const size_t blk0 = (size_t)gs * kGemvGranuleBlocks;
                    xsb = smem + p.off_xs + blk0 * NT * gmax * 64;
                    sxb = reinterpret_cast<const float*>(smem + p.off_sx) + blk0 * NT * 4;
                } else {
                    xsb = st + p.off_stage_xs;
                    sxb = reinterpret_cast<const float*>(st + p.off_stage_sx);
                }
                const uint8_t* xlane = xsb + g * 64 + t * 16;
                const bool has_b = (uint32_t)g < gmax;
#pragma unroll 4
                for (uint32_t b = 0; b < nbs; ++b) {
                    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(rowp + b * kBlockBytes);
                    const uint32_t* q1 = reinterpret_cast<const uint32_t*>(rowp + 8 * kGemvRowStride + b * kBlockBytes);
                    const uint32_t meta0 = q0[0], w0 = q0[1 + t];
                    const uint32_t meta1 = q1[0], w1 = q1[1 + t];
                    uint32_t a1[4], a2[4];
                    nibbles_to_h2(w0, a1[0], a1[2], a2[0], a2[2]);
                    nibbles_to_h2(w1, a1[1], a1[3], a2[1], a2[3]);
                    const float d0 = h2f_bits(meta0 & 0xffffu), b0 = h2f_bits(meta0 >> 16);
                    const float d1 = h2f_bits(meta1 & 0xffffu), b1 = h2f_bits(meta1 >> 16);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        uint4 bf = make_uint4(0, 0, 0, 0);
                        if (has_b) bf = *reinterpret_cast<const uint4*>(xlane + (size_t)(b * NT + nt) * gmax * 64);
                        const float sxv = sxb[(b * NT + nt) * 4 + t];
                        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        mma_16816(c, a1, bf.x, bf.y, c);
                        mma_16816(c, a2, bf.z, bf.w, c);
                        acc[nt][0] = fmaf(d0, c[0], acc[nt][0]);
                        acc[nt][1] = fmaf(d0, c[1], acc[nt][1]);
                        acc[nt][2] = fmaf(d1, c[2], acc[nt][2]);
                        acc[nt][3] = fmaf(d1, c[3], acc[nt][3]);
                        acc[nt][0] = fmaf(b0, sxv, acc[nt][0]);
                        acc[nt][2] = fmaf(b1, sxv, acc[nt][2]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
            if (!t_ready) gather_t();

            // columns 2t (hi limb) and 2t+1 (lo limb) belong to token nt*4 + t
            float v[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                v[nt][0] = acc[nt][0] + acc[nt][1];
                v[nt][1] = acc[nt][2] + acc[nt][3];
            }
            const bool complete = (g0 == 0 && g1 == p.kg);
            if (!complete) {
                const uint32_t slot = (tile == (uint32_t)(r0 / p.kg)) ? 0u : 1u;
                float* dst = p.partials + ((size_t)(blockIdx.x * 2 + slot) * kGemvTileRows + warp * 16) * (NT * 4);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    dst[g * (NT * 4) + nt * 4 + t] = v[nt][0];
                    dst[(g + 8) * (NT * 4) + nt * 4 + t] = v[nt][1];
                }
                __threadfence();
                __syncwarp();
                uint32_t last = 0, c_first = 0, c_last = 0;
                if (lane == 0) {
                    c_first = owner_of((uint64_t)tile * p.kg, total, G);
                    c_last = owner_of((uint64_t)(tile + 1) * p.kg - 1, total, G);
                    const uint32_t old = atomicAdd(&p.tickets[tile * 8 + warp], 1u);
                    last = (old == c_last - c_first) ? 1u : 0u;
                    if (last) p.tickets[tile * 8 + warp] = 0;
                }
                last = __shfl_sync(kFull, last, 0);
                if (!last) continue;
                c_first = __shfl_sync(kFull, c_first, 0);
                c_last = __shfl_sync(kFull, c_last, 0);
                __threadfence();
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) v[nt][0] = v[nt][1] = 0.0f;
                for (uint32_t c = c_first; c <= c_last; ++c) {
                    const uint32_t sl = ((uint32_t)(range_begin(c, total, G) / p.kg) == tile) ? 0u : 1u;
                    const float* src = p.partials + ((size_t)(c * 2 + sl) * kGemvTileRows + warp * 16) * (NT * 4);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        v[nt][0] += __ldcg(src + g * (NT * 4) + nt * 4 + t);
                        v[nt][1] += __ldcg(src + (g + 8) * (NT * 4) + nt * 4 + t);
                    }
                }
            }

            const uint32_t row0 = tile * kGemvTileRows + warp * 16 + g, row1 = row0 + 8;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t tok = nt * 4 + t;
                if (tok >= p.m) continue;
                float y0 = v[nt][0], y1 = v[nt][1];
                if (p.rank) {
                    const float* tt = t_s + tok * p.rank;
                    if (row0 < p.n) {
                        const float* br = p.lb + (size_t)row0 * p.rank;
                        float dsum = 0.0f;
                        for (uint32_t j = 0; j < p.rank; ++j) dsum = fmaf(__ldg(br + j), tt[j], dsum);
                        y0 += p.lscale * dsum;
                    }
                    if (row1 < p.n) {
                        const float* br = p.lb + (size_t)row1 * p.rank;
                        float dsum = 0.0f;
                        for (uint32_t j = 0; j < p.rank; ++j) dsum = fmaf(__ldg(br + j), tt[j], dsum);
                        y1 += p.lscale * dsum;
                    }
                }
                if (row0 < p.n) p.y[(size_t)tok * p.ldy + row0] = y0;
                if (row1 < p.n) p.y[(size_t)tok * p.ldy + row1] = y1;
            }
        }
        if (ok && !t_ready) gather_t();
        if (!ok) {
            if (lane == 0) atomicOr(p.status, kDevErrBarrierTimeout);
            s_err = 1;
        }
    }

    // After a failed wait some bulk copies may still be in flight towards this CTA's
    // shared memory: wait (bounded) for the stages that were issued before leaving.
    __syncthreads();
    if (s_err && warp == 8 && lane == 0) {
        const uint32_t first = issued > NST ? issued - NST : 0;
        for (uint32_t j = first; j < issued; ++j) mbar_wait(&full[j % NST], (j / NST) & 1u);
    }
}

}  // namespace

// ---------------------------------------------------------------------------
// Host side: shared-memory plan and launch.
// ---------------------------------------------------------------------------
static inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

size_t gemv_plan_smem(GemvParams& p, bool resident) {
    if (resident) return decode_plan_smem(p);
    uint32_t off = 128;                       // 2 x 8 mbarriers
    p.off_t = off;
    off += align_up(p.m * p.rank * 4, 128);
    p.off_xrot = p.off_xs = p.off_sx = 0;
    p.off_stage_xs = p.off_stage_sx = 0;
    uint32_t stage = kGemvStageWBytes;
    if (resident) {
        if (p.signs) {
            p.off_xrot = off;
            off += align_up(p.m * p.k * 4, 128);
        }
        p.off_xs = off;
        off += align_up(p.kb * p.nt * p.gmax * 64, 128);
        p.off_sx = off;
        off += align_up(p.kb * p.nt * 16, 128);
    } else {
        p.off_stage_xs = stage;
        stage += kGemvStageBlocks * p.nt * p.gmax * 64;
        p.off_stage_sx = stage;
        stage += kGemvStageBlocks * p.nt * 16;
        stage = align_up(stage, 128);
    }
    p.off_stage = off;
    p.stage_bytes = stage;
    const uint32_t budget = (uint32_t)kMaxSmem - 1024;   // static shared memory and driver reserve
    if (off + 2 * stage > budget) return 0;
    uint32_t nst = (budget - off) / stage;
    if (nst > 5) nst = 5;
    p.nstages = nst;
    return (size_t)off + (size_t)nst * stage;
}

bool gemv_resident_fits(uint32_t m, uint32_t k, bool rot) {
    if (m == 0 || m > 4 || k % 128 != 0) return false;
    GemvParams q{};
    q.m = m; q.n = 1u << 20; q.k = k; q.kb = k / 32; q.nt = 1; q.gmax = 2 * m; q.rank = kGemvMaxRank;
    q.tiles = q.n / kGemvTileRows;
    static float dummy;
    q.signs = rot ? &dummy : nullptr;
    return decode_plan_smem(q) != 0;
}

template <int NT, bool RESIDENT>
static cudaError_t launch_one(const GemvParams& p, size_t smem, int grid, cudaStream_t s) {
    auto kern = gemv_mma_kernel<NT, RESIDENT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (p.use_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

cudaError_t launch_gemv_mma(const GemvParams& p, bool resident, size_t smem, int grid, cudaStream_t s) {
    if (resident) return launch_decode(p, smem, grid, s);
    switch (p.nt) {
        case 1: return launch_one<1, false>(p, smem, grid, s);
        case 2: return launch_one<2, false>(p, smem, grid, s);
        case 3: return launch_one<3, false>(p, smem, grid, s);
        case 4: return launch_one<4, false>(p, smem, grid, s);
        default: return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------------------
// Preparation kernels of the staged variant.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) prep_xs_kernel(const void* __restrict__ x, int x_dtype, uint32_t m, uint32_t k,
                                                      uint32_t NT, uint32_t gmax, uint8_t* __restrict__ xs,
                                                      float* __restrict__ sx) {
    const uint32_t mp = blockIdx.y;
    if ((mp & 3) * 2 >= gmax) return;
    const uint32_t o = blockIdx.x * 256 + threadIdx.x;
    const bool active = o < k / 8;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active && mp < m) load8(x, x_dtype, (size_t)mp * k + (size_t)o * 8, v);
    store_fragments(xs, sx, NT, gmax, mp, o, active, v, NT * 4);
}

void launch_prep_xs(const void* x, int x_dtype, uint32_t m, uint32_t k, uint32_t nt, uint32_t gmax, uint8_t* xs_g,
                    float* sx_g, cudaStream_t s) {
    dim3 grid((k / 8 + 255) / 256, nt * 4);
    prep_xs_kernel<<<grid, 256, 0, s>>>(x, x_dtype, m, k, nt, gmax, xs_g, sx_g);
}

// t[tok][j] = sum_k A[j][k] * x[tok][k]; one warp per (tok, j), fixed reduction tree.
__global__ void __launch_bounds__(256) lora_t_kernel(const void* __restrict__ x, int x_dtype, uint32_t m, uint32_t k,
                                                     const float* __restrict__ la, uint32_t rank,
                                                     float* __restrict__ t) {
    const uint32_t pr = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (pr >= m * rank) return;
    const uint32_t tok = pr / rank, j = pr - tok * rank;
    const float* arow = la + (size_t)j * k;
    float s0 = 0.0f, s1 = 0.0f;
    uint32_t kk = lane;
    for (; kk + 32 < k; kk += 64) {
        s0 = fmaf(__ldg(arow + kk), load_act(x, x_dtype, (size_t)tok * k + kk), s0);
        s1 = fmaf(__ldg(arow + kk + 32), load_act(x, x_dtype, (size_t)tok * k + kk + 32), s1);
    }
    for (; kk < k; kk += 32) s0 = fmaf(__ldg(arow + kk), load_act(x, x_dtype, (size_t)tok * k + kk), s0);
    float sum = s0 + s1;
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
    if (lane == 0) t[pr] = sum;
}

void launch_lora_t(const void* x, int x_dtype, uint32_t m, uint32_t k, const float* la, uint32_t rank, float* t,
                   cudaStream_t s) {
    const uint32_t pairs = m * rank;
    if (pairs == 0) return;
    lora_t_kernel<<<(pairs + 7) / 8, 256, 0, s>>>(x, x_dtype, m, k, la, rank, t);
}

// ---------------------------------------------------------------------------
// Generic kernel: any k % 32 == 0, 4-byte aligned payload, any m.  One warp per
// output row and token; lanes stride over nibble words.  Also serves the
// standalone LoRA accumulate (base term skipped).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gemv_generic_kernel(const void* __restrict__ x, int x_dtype,
                                                           const uint8_t* __restrict__ w, float* __restrict__ y,
                                                           uint64_t ldy, uint32_t m, uint32_t n, uint32_t k,
                                                           const float* __restrict__ t, const float* __restrict__ lb,
                                                           uint32_t rank, float lscale, int accumulate_only) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= n) return;
    const uint32_t kb = k / 32, nwords = k / 8;
    const uint8_t* wrow = w ? w + (size_t)row * kb * kBlockBytes : nullptr;
    for (uint32_t tok = blockIdx.y; tok < m; tok += gridDim.y) {
        float acc = 0.0f;
        if (!accumulate_only) {
            for (uint32_t wi = lane; wi < nwords; wi += 32) {
                const uint32_t* bp = reinterpret_cast<const uint32_t*>(wrow + (size_t)(wi >> 2) * kBlockBytes);
                const uint32_t meta = __ldg(bp), q = __ldg(bp + 1 + (wi & 3));
                const float d = h2f_bits(meta & 0xffffu), b = h2f_bits(meta >> 16);
                const size_t xb = (size_t)tok * k + (size_t)wi * 8;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float wv = __fmaf_rn((float)((q >> (4 * i)) & 15u), d, b);
                    acc = fmaf(wv, load_act(x, x_dtype, xb + i), acc);
                }
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
        }
        if (lane == 0) {
            float out = accumulate_only ? y[(size_t)tok * ldy + row] : acc;
            if (rank) {
                float dsum = 0.0f;
                for (uint32_t j = 0; j < rank; ++j) dsum = fmaf(lb[(size_t)row * rank + j], t[(size_t)tok * rank + j], dsum);
                out += lscale * dsum;
            }
            y[(size_t)tok * ldy + row] = out;
        }
    }
}

void launch_gemv_generic(const void* x, int x_dtype, const uint8_t* w, float* y, uint64_t ldy, uint32_t m,
                         uint32_t n, uint32_t k, const float* t, const float* lb, uint32_t rank, float lscale,
                         int accumulate_only, cudaStream_t s) {
    if (m == 0 || n == 0) return;
    dim3 grid((n + 7) / 8, m < 65535u ? m : 65535u);
    gemv_generic_kernel<<<grid, 256, 0, s>>>(x, x_dtype, w, y, ldy, m, n, k, t, lb, rank, lscale, accumulate_only);
}

}  // namespace lq4
