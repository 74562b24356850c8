// Resident decode kernel (m <= 4): y[m, n] = x[m, k] * Wq4[n, k]^T (+ LoRA) (+ rotation of x).
//
// HBM-bound: the packed weights are read once, everything else is small.
//  * One persistent CTA per SM.  A producer warp streams weight tiles with TMA
//    (cp.async.bulk.tensor.2d, one instruction per stage) into a shared-memory ring;
//    completion is counted on mbarriers.  A "big" stage is 128 rows x 20 blocks (51,200 B),
//    a "small" one 128 rows x 4 blocks; rows stay densely packed, and 100- and 20-word row
//    strides keep every consumer load free of bank conflicts.
//  * Eight consumer warps own 16 rows each.  Within a group of four Q4 blocks, the four
//    threads of an MMA quad take one block each: the 16 k-slots of every warp MMA then hold
//    four k-values of four different blocks, and the B operand is zero outside the column
//    pair (hi limb, lo limb) that belongs to the thread's block.  After eight MMAs each
//    thread holds the full 32-element dot products of its own block for two rows, so the
//    per-block scale/bias step (f16 -> f32 conversions, three FMAs per row) is done once per
//    four blocks per thread instead of once per block by every thread.
//  * The activation row(s) are converted once per CTA into f16 hi/lo limbs kept in shared
//    memory (optionally after the randomized Hadamard rotation, also done in shared memory).
//  * Work is split stream-K style in units of 4 blocks x 128 rows; tiles shared by several
//    CTAs are finished by the last arriver, which adds the partials in CTA order.
//  * LoRA: each CTA projects its own k slice onto A, the partials are exchanged through
//    global memory (bounded wait) and s * B * t is added in the tile epilogue.
#include <cuda.h>

#include <mutex>

#include "lq4_gemv_common.cuh"

namespace lq4 {

namespace {

using namespace gemv;

constexpr int kBigBlocks = 20;                                   // blocks per row in a big stage
constexpr int kSmallBlocks = kGemvGranuleBlocks;                 // 4
constexpr int kBigGranules = kBigBlocks / kGemvGranuleBlocks;    // 5
constexpr uint32_t kSlotBytes = kGemvTileRows * kBigBlocks * kBlockBytes;      // 51,200
constexpr uint32_t kSmallBytes = kGemvTileRows * kSmallBlocks * kBlockBytes;   // 10,240
constexpr int kMaxStages = 8;

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Prologue of the 256 consumer threads: rotation, LoRA partial projection, activation limbs.
template <int MT>
__device__ void decode_prologue(const GemvParams& p, uint8_t* smem, int ctid) {
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

    // limbs: [block][token][hi, lo][64 B]; block sums: [block][token]
    uint8_t* xs = smem + p.off_xs;
    float* sx = reinterpret_cast<float*>(smem + p.off_sx);
    const uint32_t noct = K / 8;
    for (uint32_t mp = 0; mp < (uint32_t)MT; ++mp) {
        // four octets per thread and pass: all global loads are issued before the first use
        for (uint32_t o0 = 0; o0 < noct; o0 += 4 * kConsumerThreads) {
            float v[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t o = o0 + u * kConsumerThreads + ctid;
#pragma unroll
                for (int i = 0; i < 8; ++i) v[u][i] = 0.0f;
                if (o < noct) {
                    if (rot) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[u][i] = xrot[mp * K + o * 8 + i];
                    } else {
                        load8(p.x, p.x_dtype, (size_t)mp * K + (size_t)o * 8, v[u]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t o = o0 + u * kConsumerThreads + ctid;
                store_fragments(xs, sx, 1, 2 * MT, mp, o, o < noct, v[u], MT);
            }
        }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
}

template <int MT>
__global__ void __launch_bounds__(kGemvThreads, 1)
decode_kernel(const GemvParams p, const __grid_constant__ CUtensorMap tm_big,
              const __grid_constant__ CUtensorMap tm_small) {
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
        mbar_fence_init();
    }
    __syncthreads();
    if (p.use_pdl) pdl_launch_dependents();

    const uint64_t G = gridDim.x;
    const uint64_t total = (uint64_t)p.tiles * p.kg;
    const uint64_t r0 = range_begin(blockIdx.x, total, G), r1 = range_begin(blockIdx.x + 1, total, G);
    uint32_t issued = 0;

    if (warp == 8) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            const uint64_t pol = l2_policy_evict_first();
            uint32_t it = 0;
            bool ok = true;
            for (uint64_t pos = r0; pos < r1 && ok;) {
                const uint32_t tile = (uint32_t)(pos / p.kg);
                const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * p.kg);
                const uint64_t left = r1 - pos;
                const uint32_t g1 = (uint64_t)(p.kg - g0) < left ? p.kg : (uint32_t)(g0 + left);
                for (uint32_t gs = g0; gs < g1; ++it) {
                    const bool big = g1 - gs >= (uint32_t)kBigGranules;
                    const uint32_t s = it % NST;
                    if (!mbar_wait(&empty[s], ((it / NST) & 1u) ^ 1u)) { ok = false; break; }
                    uint8_t* st = smem + p.off_stage + (size_t)s * kSlotBytes;
                    mbar_arrive_expect_tx(&full[s], big ? kSlotBytes : kSmallBytes);
                    // coordinates: x in 4-byte elements along the row, y = first row of the tile
                    tma_load_2d(st, big ? &tm_big : &tm_small, (int32_t)(gs * kGemvGranuleBlocks * 5),
                                (int32_t)(tile * kGemvTileRows), &full[s], pol);
                    gs += big ? kBigGranules : 1;
                }
                pos += g1 - g0;
            }
            issued = it;
            if (!ok) {
                atomicOr(p.status, kDevErrBarrierTimeout);
                s_err = 1;
            }
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int g = lane >> 2, t = lane & 3;
        float* t_s = reinterpret_cast<float*>(smem + p.off_t);
        if (p.use_pdl) pdl_wait_prior_grids();
        decode_prologue<MT>(p, smem, tid);
        bool t_ready = p.rank == 0;

        auto gather_t = [&]() {
            if (tid == 0) {
                const unsigned long long t0 = globaltimer_ns();
                while (ld_acquire_u32(p.tsync) < (uint32_t)G) {
                    if (globaltimer_ns() - t0 > kWaitLimitNs) {
                        s_twait_failed = 1;
                        atomicOr(p.status, kDevErrGridWaitTimeout);
                        break;
                    }
                    __nanosleep(64);
                }
            }
            named_bar_sync(kBarConsumers, kConsumerThreads);
            // one warp per (token, rank) pair: lanes fetch different CTAs' partials at once, then a
            // fixed shuffle tree adds them (same result whatever the arrival order)
            const uint32_t pairs = p.m * p.rank;
            const bool failed = s_twait_failed != 0;
            for (uint32_t pr = warp; pr < pairs; pr += 8) {
                float s = 0.0f;
                if (!failed)
                    for (uint32_t c = lane; c < (uint32_t)G; c += 32) s += __ldcg(p.tpart + (size_t)c * pairs + pr);
#pragma unroll
                for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
                if (lane == 0) t_s[pr] = s;
            }
            named_bar_sync(kBarConsumers, kConsumerThreads);
            if (tid == 0) {
                const uint32_t old = atomicAdd(p.tsync + 1, 1u);
                if (old == (uint32_t)G - 1) {     // last reader re-arms both counters
                    p.tsync[0] = 0;
                    p.tsync[1] = 0;
                    __threadfence();
                }
            }
            t_ready = true;
        };

        // this lane supplies B-operand registers only for the column pair of its own block
        const bool has_b = (g >> 1) == t;
        const uint8_t* xs_lane = smem + p.off_xs + (size_t)(g & 1) * 64;
        const float* sx_all = reinterpret_cast<const float*>(smem + p.off_sx);

        uint32_t it = 0;
        bool ok = true;
        for (uint64_t pos = r0; pos < r1 && ok;) {
            const uint32_t tile = (uint32_t)(pos / p.kg);
            const uint32_t g0 = (uint32_t)(pos - (uint64_t)tile * p.kg);
            const uint64_t left = r1 - pos;
            const uint32_t g1 = (uint64_t)(p.kg - g0) < left ? p.kg : (uint32_t)(g0 + left);
            pos += g1 - g0;

            float acc[MT][2];
#pragma unroll
            for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = 0.0f;

            for (uint32_t gs = g0; gs < g1; ++it) {
                const bool big = g1 - gs >= (uint32_t)kBigGranules;
                const uint32_t ngr = big ? kBigGranules : 1;
                const uint32_t rs = big ? kBigBlocks * kBlockBytes : kSmallBlocks * kBlockBytes;
                const uint32_t s = it % NST;
                if (!mbar_wait(&full[s], (it / NST) & 1u)) { ok = false; break; }
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
                    uint4 bf[MT][4];
                    float sxv[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint8_t* xb = xs_lane + ((size_t)blk * MT + mt) * 128;
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            bf[mt][j] = has_b ? *reinterpret_cast<const uint4*>(xb + j * 16) : make_uint4(0, 0, 0, 0);
                        sxv[mt] = sx_all[(size_t)blk * MT + mt];
                    }
                    float ca[MT][4], cb[MT][4];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) ca[mt][i] = cb[mt][i] = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t a1[4], a2[4];
                        nibbles_to_h2(w0[j], a1[0], a1[2], a2[0], a2[2]);
                        nibbles_to_h2(w1[j], a1[1], a1[3], a2[1], a2[3]);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            mma_16816(ca[mt], a1, bf[mt][j].x, bf[mt][j].y, ca[mt]);
                            mma_16816(cb[mt], a2, bf[mt][j].z, bf[mt][j].w, cb[mt]);
                        }
                    }
                    const float d0 = h2f_bits(meta0 & 0xffffu), b0 = h2f_bits(meta0 >> 16);
                    const float d1 = h2f_bits(meta1 & 0xffffu), b1 = h2f_bits(meta1 >> 16);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        // columns 2t (hi limb) and 2t+1 (lo limb) hold this thread's block
                        const float dot0 = (ca[mt][0] + cb[mt][0]) + (ca[mt][1] + cb[mt][1]);
                        const float dot1 = (ca[mt][2] + cb[mt][2]) + (ca[mt][3] + cb[mt][3]);
                        acc[mt][0] = fmaf(d0, dot0, fmaf(b0, sxv[mt], acc[mt][0]));
                        acc[mt][1] = fmaf(d1, dot1, fmaf(b1, sxv[mt], acc[mt][1]));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                gs += ngr;
            }
            if (!ok) break;
            if (!t_ready) gather_t();

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
            const bool complete = (g0 == 0 && g1 == p.kg);
            if (!complete) {
                const uint32_t slot = (tile == (uint32_t)(r0 / p.kg)) ? 0u : 1u;
                float* dst = p.partials + ((size_t)(blockIdx.x * 2 + slot) * kGemvTileRows + warp * 16) * MT;
                if (t == 0) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        dst[g * MT + mt] = v[mt][0];
                        dst[(g + 8) * MT + mt] = v[mt][1];
                    }
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
                // lanes fetch different CTAs' partials (all 16 rows each) in one round trip, a fixed
                // shuffle tree adds them, then every lane picks the rows it finishes
                float part[16 * MT];
#pragma unroll
                for (int i = 0; i < 16 * MT; ++i) part[i] = 0.0f;
                for (uint32_t c = c_first + lane; c <= c_last; c += 32) {
                    const uint32_t sl = ((uint32_t)(range_begin(c, total, G) / p.kg) == tile) ? 0u : 1u;
                    const float4* src = reinterpret_cast<const float4*>(
                        p.partials + ((size_t)(c * 2 + sl) * kGemvTileRows + warp * 16) * MT);
#pragma unroll
                    for (int i = 0; i < 4 * MT; ++i) {
                        const float4 q = __ldcg(src + i);
                        part[4 * i] += q.x; part[4 * i + 1] += q.y; part[4 * i + 2] += q.z; part[4 * i + 3] += q.w;
                    }
                }
#pragma unroll
                for (int i = 0; i < 16 * MT; ++i) {
#pragma unroll
                    for (int o = 16; o; o >>= 1) part[i] += __shfl_xor_sync(kFull, part[i], o);
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    v[mt][0] = v[mt][1] = 0.0f;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {        // select without dynamic register indexing
                        if (r == g) { v[mt][0] = part[r * MT + mt]; v[mt][1] = part[(r + 8) * MT + mt]; }
                    }
                }
            }

            // epilogue: quad thread t finishes token t (LoRA term, store)
            const uint32_t rowa = tile * kGemvTileRows + warp * 16 + g, rowb = rowa + 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                if (mt != t || (uint32_t)mt >= p.m) continue;
                float y0 = v[mt][0], y1 = v[mt][1];
                if (p.rank) {
                    const float* tt = t_s + mt * p.rank;
                    if (rowa < p.n) {
                        const float* br = p.lb + (size_t)rowa * p.rank;
                        float dsum = 0.0f;
                        for (uint32_t j = 0; j < p.rank; ++j) dsum = fmaf(__ldg(br + j), tt[j], dsum);
                        y0 += p.lscale * dsum;
                    }
                    if (rowb < p.n) {
                        const float* br = p.lb + (size_t)rowb * p.rank;
                        float dsum = 0.0f;
                        for (uint32_t j = 0; j < p.rank; ++j) dsum = fmaf(__ldg(br + j), tt[j], dsum);
                        y1 += p.lscale * dsum;
                    }
                }
                if (rowa < p.n) p.y[(size_t)mt * p.ldy + rowa] = y0;
                if (rowb < p.n) p.y[(size_t)mt * p.ldy + rowb] = y1;
            }
        }
        if (ok && !t_ready) gather_t();
        if (!ok) {
            if (lane == 0) atomicOr(p.status, kDevErrBarrierTimeout);
            s_err = 1;
        }
    }

    // After a failed wait some TMA loads may still be in flight towards this CTA's shared
    // memory: wait (bounded) for the stages that were issued before leaving.
    __syncthreads();
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

template <int MT>
cudaError_t launch_mt(const GemvParams& p, const CUtensorMap& big, const CUtensorMap& small, size_t smem, int grid,
                      cudaStream_t s) {
    auto kern = decode_kernel<MT>;
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
    return cudaLaunchKernelEx(&cfg, kern, p, big, small);
}

}  // namespace

size_t decode_plan_smem(GemvParams& p) {
    if (p.m == 0 || p.m > 4 || p.kb == 0 || p.kb % kGemvGranuleBlocks != 0) return 0;
    const uint32_t MT = p.m;
    uint32_t off = 2 * kMaxStages * 8;            // mbarriers
    p.off_t = off;
    off += align_up(p.m * p.rank * 4, 128);
    p.off_xrot = 0;
    if (p.signs) {
        p.off_xrot = off;
        off += align_up(p.m * p.k * 4, 128);
    }
    p.off_xs = off;
    off += align_up(p.kb * MT * 128, 128);
    p.off_sx = off;
    off += align_up(p.kb * MT * 4, 128);
    p.off_stage = off;
    p.stage_bytes = kSlotBytes;
    p.off_stage_xs = p.off_stage_sx = 0;
    const uint32_t budget = (uint32_t)kMaxSmem - 1024;    // static shared memory and driver reserve
    if (off + 2 * kSlotBytes > budget) return 0;
    uint32_t nst = (budget - off) / kSlotBytes;
    if (nst > 4) nst = 4;
    p.nstages = nst;
    p.kg = p.kb / kGemvGranuleBlocks;
    return (size_t)off + (size_t)nst * kSlotBytes;
}

uint64_t decode_units(const GemvParams& p) { return (uint64_t)p.tiles * p.kg; }

cudaError_t launch_decode(const GemvParams& p, size_t smem, int grid, cudaStream_t s) {
    CUtensorMap big, small;
    if (!make_weight_map(&big, p.w, p.n, p.kb, kBigBlocks) || !make_weight_map(&small, p.w, p.n, p.kb, kSmallBlocks))
        return cudaErrorInvalidValue;
    switch (p.m) {
        case 1: return launch_mt<1>(p, big, small, smem, grid, s);
        case 2: return launch_mt<2>(p, big, small, smem, grid, s);
        case 3: return launch_mt<3>(p, big, small, smem, grid, s);
        case 4: return launch_mt<4>(p, big, small, smem, grid, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace lq4
