// Prefill path (m > 16): Y[m, n] = X[m, k] * Wq4[n, k]^T (+ LoRA) on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// The product is computed transposed, D[n, m] = W[n, :] . X[m, :], so that the 128 TMEM lanes
// are weight rows and the columns are tokens: the epilogue then stores 32 consecutive output
// features per warp instruction (coalesced along n).
//
//   CTA tile      256 weight rows (two 128-row sub-tiles, one TMEM accumulator each) x TT tokens
//                 (TT = 256 with f16-exact activations, 128 when the activations are carried as two
//                 f16 limbs); both sub-tiles multiply the same activation tile, which is therefore
//                 loaded once per 256 weight rows; K loop in blocks of 64, three 64 KB stages
//   warp 0        TMA producer: activation tiles (and the dense LoRA tiles) -> shared memory
//   warp 1        TMEM allocation, then one elected lane issues tcgen05.mma / tcgen05.commit
//   warps 2..5    dequantizers of sub-tile 0, warps 6..9 of sub-tile 1: read the raw Q4 blocks of
//                 their rows from a small shared-memory ring, convert in registers (magic-number
//                 int4 -> f16, one HFMA2 per pair for q*d+b) and write the 128 x 64 f16 tile in the
//                 128-byte-swizzled K-major layout the MMA reads
//   warps 10..13  epilogue: tcgen05.ld the finished accumulators, store f32 to Y
//   warp 14       TMA producer of the raw Q4 ring (128 rows x 4 blocks per stage)
//
// Operands are f16 with f32 accumulation.  Dequantized weights are rounded once to f16; the
// activations are exact in f16 when they come as bf16, and are split into hi + lo f16 limbs
// (two MMAs on the same weight tile) when they come as f32.
// LoRA enters as extra K blocks: D += (s*B)[n, :] . T[m, :] with T = X A^T computed beforehand
// (f32) and both factors carried as hi/lo f16 pairs.  T itself comes from the same kernel in its
// all-dense mode with the roles swapped: the tokens are the 256-row operand (every row of the box
// is real work; a rank-64 adapter would fill a quarter of it), A is the narrow one, and the k range
// is cut into pieces, one output tile each, so that about one wave of CTAs shares a product that
// would otherwise be a long serial loop on m / 256 of them.  The pieces (of T^T) are summed in
// index order by the kernel that splits T into limbs.
//
// Within each group of 8 consecutive k the stored order is (k0,k4,k1,k5,k2,k6,k3,k7): that is
// the order in which the nibble extraction yields pairs, and the activation tiles are written
// in the same order by the conversion kernel, so no shuffling is needed on either side.
#include "lq4_gemm.cuh"
#include "lq4_kernels.cuh"

#include <cuda.h>

#include <mutex>

namespace lq4 {

namespace {

constexpr int kTileN = 128;          // weight rows per CTA tile (TMEM lanes)
constexpr int kBlockK = 64;          // k per pipeline stage (128 bytes of f16: one swizzle atom)
constexpr uint32_t kTileABytes = kTileN * kBlockK * 2;      // 16 KB dequantized weights
constexpr uint32_t kTileBBytes = 256 * kBlockK * 2;         // 32 KB activations (both limb modes)

// ---- tcgen05 wrappers ------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], f16 inputs, f32 accumulate; issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 32 consecutive columns of 32-bit accumulators -> 32 registers per thread.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle; groups of
// 8 rows are 1024 bytes apart.  Fields: start address >> 4 (bits 0-13), leading byte offset >> 4
// (16-29, unused for swizzled K-major), stride byte offset >> 4 (32-45), descriptor version 1
// (46-47), swizzle mode 2 = 128 B (61-63).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::f16: f32 accumulator (bits 4-5 = 1), f16 A and B (formats 0), both
// K-major, N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void tma_load_tile(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y,
                                              uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Byte offset of 16-byte chunk `c` (0..7) of row `r` inside a 128-byte-swizzled K-major tile.
__device__ __forceinline__ uint32_t swz128(uint32_t r, uint32_t c) {
    return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4);
}

// ---------------------------------------------------------------------------
// f16 conversion of an f32/bf16 matrix [rows, cols] (cols % 8 == 0): "hi" = round to nearest,
// optional "lo" = residual.  Each group of 8 consecutive columns is stored as
// (c0,c4,c1,c5,c2,c6,c3,c7).  Destination rows are `dst_stride` halves apart; lo goes
// `lo_off` halves to the right of hi (lo_off == 0: no lo limb).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) convert_rows_kernel(const void* __restrict__ x, int x_dtype, uint32_t rows,
                                                           uint32_t cols, __half* __restrict__ dst,
                                                           uint64_t dst_stride, uint64_t lo_off) {
    const uint64_t opr = cols / 8, n_oct = (uint64_t)rows * opr;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; o < n_oct; o += stride) {
        const uint64_t row = o / opr, oc = o - row * opr;
        float v[8];
        if (x_dtype == LQ4_DTYPE_BF16) {
            const uint4 r = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + o * 8);
            const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        } else {
            const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + o * 8);
            const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + o * 8 + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        __half h[8], l[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) split_f16(v[i], h[i], l[i]);
        auto pk = [](__half a, __half b) { return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16); };
        __half* d = dst + row * dst_stride + oc * 8;
        *reinterpret_cast<uint4*>(d) = make_uint4(pk(h[0], h[4]), pk(h[1], h[5]), pk(h[2], h[6]), pk(h[3], h[7]));
        if (lo_off)
            *reinterpret_cast<uint4*>(d + lo_off) = make_uint4(pk(l[0], l[4]), pk(l[1], l[5]), pk(l[2], l[6]), pk(l[3], l[7]));
    }
}

// dst[row][j] = hi(scale * src[row][j]), dst[row][cp + j] = lo(...), natural column order, zero
// padding for cols <= j < cp.  dst rows are 2 * cp halves long.
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ src, uint32_t rows, uint32_t cols,
                                                         uint32_t cp, float scale, __half* __restrict__ dst) {
    const uint64_t n = (uint64_t)rows * cp;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t row = i / cp;
        const uint32_t j = (uint32_t)(i - row * cp);
        __half h = __float2half_rn(0.0f), l = h;
        if (j < cols) split_f16(scale * src[row * cols + j], h, l);
        dst[row * 2 * cp + j] = h;
        dst[row * 2 * cp + cp + j] = l;
    }
}

// The same split for T = X A^T as the k-split projection leaves it: `pieces` partial sums of the TRANSPOSE,
// part[s][j][row] (rows of `ld` floats, pieces `piece_stride` floats apart).  Sums the pieces in index order
// and writes dst[row][j] = hi, dst[row][cp + j] = lo.  Block = 32 rows x 8 columns through shared memory:
// the reads run along `row` (128 bytes per warp and piece), the writes are 16-byte runs along `j`.
__global__ void __launch_bounds__(256) sum_split_transposed_kernel(const float* __restrict__ part, uint32_t pieces,
                                                                   uint64_t piece_stride, uint64_t ld, uint32_t rows,
                                                                   uint32_t cols, uint32_t cp, __half* __restrict__ dst) {
    __shared__ float tile[8][33];
    const uint32_t row0 = blockIdx.x * 32, j0 = blockIdx.y * 8;
    {
        const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
        const uint32_t j = j0 + ty, row = row0 + tx;
        float acc = 0.0f;
        if (j < cols && row < rows) {
            const float* src = part + (uint64_t)j * ld + row;
            uint32_t s = 0;
            for (; s + 4 <= pieces; s += 4) {
                const float v0 = src[(s + 0) * piece_stride], v1 = src[(s + 1) * piece_stride];
                const float v2 = src[(s + 2) * piece_stride], v3 = src[(s + 3) * piece_stride];
                acc = (((acc + v0) + v1) + v2) + v3;
            }
            for (; s < pieces; ++s) acc += src[s * piece_stride];
        }
        tile[ty][tx] = acc;
    }
    __syncthreads();
    const uint32_t r = threadIdx.x >> 3, jj = threadIdx.x & 7u;
    const uint32_t row = row0 + r, j = j0 + jj;
    if (row < rows && j < cp) {
        __half h, l;
        split_f16(tile[jj][r], h, l);
        dst[(uint64_t)row * 2 * cp + j] = h;
        dst[(uint64_t)row * 2 * cp + cp + j] = l;
    }
}

struct GemmParams {
    const uint8_t* w;
    float* y;
    uint64_t ldy;
    uint32_t m, n, k;
    uint32_t limbs;          // 1: activations exact in f16; 2: hi + lo limbs
    uint32_t tt;             // tokens per CTA tile = 256 / limbs
    uint32_t n_tiles, m_tiles;
    uint32_t kblocks;        // k / 64 (even)
    uint32_t lora_kblocks;   // dense (f16 x f16) k blocks appended after the Q4 blocks
    uint32_t seg_len;        // dense blocks per segment
    uint32_t seg_a_off[4];   // column offset of each dense segment in the A-operand matrix
    uint32_t seg_b_off[4];   // ... and in the B-operand matrix
    uint32_t ksplit;         // all-dense products only: the k range is cut into ksplit pieces, one output tile each;
    uint64_t split_stride;   // piece s adds s * seg_len blocks to every segment offset and writes y + s * split_stride
    int32_t* status;
    // fused all-gather of an N-sharded product: every result is also stored at the same place of each peer's
    // output buffer (plain stores over NVLink from the epilogue warps, tile by tile while the MMAs go on)
    uint32_t n_peers;
    int64_t peer_off[LQ4_MAX_PEERS - 1];     // bytes from an element of y to the same element in a peer
};

// A CTA works on TWO 128-row sub-tiles of the weights against one activation tile: the activation
// tile (the operand every n-tile has to re-read from L2) is loaded once per 256 weight rows.
constexpr int kSubTiles = 2;
constexpr int kCtaRows = kSubTiles * kTileN;                   // 256 weight rows per CTA tile
constexpr int kRawStages = 3;                                  // each: one sub-tile, 128 rows x 4 blocks (two k blocks)
constexpr uint32_t kRawBytes = kTileN * 4 * kBlockBytes;       // 10,240
constexpr int kStages2 = 3;                                    // pipeline stages of A0 | A1 | B
constexpr uint32_t kStage2Bytes = kSubTiles * kTileABytes + kTileBBytes;   // 64 KB
constexpr uint32_t kOffStages = 1024;                          // barriers and the TMEM pointer live below
constexpr uint32_t kOffRaw = kOffStages + kStages2 * kStage2Bytes;
constexpr uint32_t kGemmSmem = kOffRaw + kRawStages * kRawBytes;   // 228,352

// One nibble word (8 weights of one block) -> 8 f16 weights q*d+b in the order (k0,k4,k1,k5,k2,k6,k3,k7).
__device__ __forceinline__ uint4 dequant_word_f16(uint32_t w, __half2 d2, __half2 b2) {
    uint32_t q04, q15, q26, q37;
    nibbles_to_h2(w, q04, q15, q26, q37);
    __half2 r0 = __hfma2(*reinterpret_cast<__half2*>(&q04), d2, b2);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2*>(&q15), d2, b2);
    __half2 r2 = __hfma2(*reinterpret_cast<__half2*>(&q26), d2, b2);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2*>(&q37), d2, b2);
    return make_uint4(*reinterpret_cast<uint32_t*>(&r0), *reinterpret_cast<uint32_t*>(&r1),
                      *reinterpret_cast<uint32_t*>(&r2), *reinterpret_cast<uint32_t*>(&r3));
}

// warps: 0 TMA (activations, dense LoRA tiles), 1 MMA issue, 2-9 dequant sub-tile 0, 10-17 dequant
// sub-tile 1 (thread = one weight row x one Q4 block), 18-21 epilogue (warp % 4 = TMEM lane quarter),
// 22 TMA (packed Q4 rows)
constexpr int kDeqWarpsPerSub = 4;      // 4: a thread converts both Q4 blocks of its row; 8: one block each
constexpr int kGemmWarps = 2 + 2 * kDeqWarpsPerSub + 4 + 1;

__global__ void __launch_bounds__(kGemmWarps * 32, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_da, const __grid_constant__ CUtensorMap tm_db) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);          // [kStages2]  tile operands ready
    uint64_t* empty = full + kStages2;                           // [kStages2]  MMAs that read the stage are done
    uint64_t* raw_full = empty + kStages2;                       // [kRawStages]
    uint64_t* raw_empty = raw_full + kRawStages;                 // [kRawStages]
    uint64_t* acc_full = raw_empty + kRawStages;                 // [2] accumulator finished
    uint64_t* acc_empty = acc_full + 2;                          // [2] accumulator drained
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* s_err = reinterpret_cast<int*>(tmem_ptr + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kStages2; ++s) { mbar_init(&full[s], 1 + kDeqWarpsPerSub * kSubTiles); mbar_init(&empty[s], 1); }
        for (int s = 0; s < kRawStages; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], kDeqWarpsPerSub); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *s_err = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_ptr, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    const uint32_t tps = p.n_tiles * p.m_tiles;                  // tiles per k piece
    const uint32_t total_tiles = tps * p.ksplit;
    const uint32_t nkb = p.kblocks + p.lora_kblocks;
    const uint32_t xbytes = p.limbs * p.tt * 128;                // activation bytes per Q4 stage
    // accumulator buffers: two sub-tiles of tt columns each; double-buffered when they fit twice in 512 columns
    const uint32_t acc_cols = kSubTiles * p.tt;
    const uint32_t nbuf = acc_cols * 2 <= 512 ? 2u : 1u;

    if (warp == 0) {
        // ---------------- TMA: activation tiles, dense LoRA tiles ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int32_t n0 = (int32_t)(((tile % tps) / p.m_tiles) * kCtaRows), m0 = (int32_t)((tile % p.m_tiles) * p.tt);
                for (uint32_t kb = 0; kb < nkb; ++kb, ++it) {
                    const uint32_t s = it % kStages2;
                    if (!mbar_wait(&empty[s], ((it / kStages2) & 1u) ^ 1u)) { ok = false; break; }
                    uint8_t* st = smem + kOffStages + s * kStage2Bytes;
                    uint8_t* bt = st + kSubTiles * kTileABytes;
                    if (kb < p.kblocks) {
                        mbar_arrive_expect_tx(&full[s], xbytes);
                        // the converted activations hold the hi limb in columns [0, k), the lo limb in [k, 2k)
                        tma_load_tile(bt, &tm_x, (int32_t)(kb * kBlockK), m0, &full[s]);
                        if (p.limbs == 2) tma_load_tile(bt + p.tt * 128, &tm_x, (int32_t)(p.k + kb * kBlockK), m0, &full[s]);
                    } else {
                        // dense stage: both operands by TMA; the A box spans all 256 rows (two sub-tiles)
                        const uint32_t d = kb - p.kblocks, seg = d / p.seg_len;
                        const uint32_t within = d - seg * p.seg_len + (tile / tps) * p.seg_len;
                        mbar_arrive_expect_tx(&full[s], kSubTiles * kTileABytes + p.tt * 128);
                        tma_load_tile(st, &tm_da, (int32_t)(p.seg_a_off[seg] + within * kBlockK), n0, &full[s]);
                        tma_load_tile(bt, &tm_db, (int32_t)(p.seg_b_off[seg] + within * kBlockK), m0, &full[s]);
                    }
                }
            }
            if (!ok) { atomicOr(p.status, kDevErrBarrierTimeout); *s_err = 1; }
        }
    } else if (warp == kGemmWarps - 1) {
        // ---------------- TMA: packed Q4 rows, per sub-tile 4 blocks (two k blocks) per load ----------------
        if (lane == 0) {
            uint32_t rit = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const uint32_t n0 = ((tile % tps) / p.m_tiles) * kCtaRows;
                const uint32_t nsub = n0 + kTileN < p.n ? 2u : 1u;
                for (uint32_t pr = 0; pr < p.kblocks / 2 && ok; ++pr) {
                    for (uint32_t sub = 0; sub < nsub; ++sub, ++rit) {
                        const uint32_t rs = rit % kRawStages;
                        if (!mbar_wait(&raw_empty[rs], ((rit / kRawStages) & 1u) ^ 1u)) { ok = false; break; }
                        mbar_arrive_expect_tx(&raw_full[rs], kRawBytes);
                        tma_load_tile(smem + kOffRaw + rs * kRawBytes, &tm_w, (int32_t)(pr * 20), (int32_t)(n0 + sub * kTileN),
                                      &raw_full[rs]);
                    }
                }
            }
            if (!ok) { atomicOr(p.status, kDevErrBarrierTimeout); *s_err = 1; }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(kTileN, p.tt);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
                const uint32_t n0 = ((tile % tps) / p.m_tiles) * kCtaRows;
                const uint32_t nsub = n0 + kTileN < p.n ? 2u : 1u;
                const uint32_t buf = tcount % nbuf;
                if (!mbar_wait(&acc_empty[buf], ((tcount / nbuf) & 1u) ^ 1u)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * acc_cols;
                for (uint32_t kb = 0; kb < nkb; ++kb, ++it) {
                    const uint32_t s = it % kStages2;
                    if (!mbar_wait(&full[s], (it / kStages2) & 1u)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + kOffStages + s * kStage2Bytes);
                    const uint32_t b_addr = a_addr + kSubTiles * kTileABytes;
                    const uint32_t nl = kb < p.kblocks ? p.limbs : 1u;
                    for (uint32_t sub = 0; sub < nsub; ++sub) {
                        const uint64_t da = make_smem_desc(a_addr + sub * kTileABytes);
                        for (uint32_t l = 0; l < nl; ++l) {
                            const uint64_t db = make_smem_desc(b_addr + l * p.tt * 128);
#pragma unroll
                            for (uint32_t k4 = 0; k4 < 4; ++k4)      // 16 k per MMA = 32 bytes = 2 descriptor units
                                umma_f16(d_tmem + sub * p.tt, da + 2 * k4, db + 2 * k4, idesc, (kb | l | k4) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty[s]);
                }
                if (!ok) break;
                umma_commit(&acc_full[buf]);
            }
            if (!ok) { atomicOr(p.status, kDevErrBarrierTimeout); *s_err = 1; }
        }
    } else if (warp >= 2 && warp < 2 + 2 * kDeqWarpsPerSub) {
        // ---- dequantizers: group `sub`; thread = weight row n0 + sub*128 + r, Q4 block `blk` of the k block ----
        const uint32_t sub = (uint32_t)(warp - 2) / kDeqWarpsPerSub;
        const uint32_t gt = (uint32_t)(tid - 64) - sub * (kDeqWarpsPerSub * 32);
        const uint32_t r = gt & 127u, blk = gt >> 7;
        uint32_t it = 0, rit = 0;      // rit counts raw entries of ALL groups, as the raw producer does
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const uint32_t n0 = ((tile % tps) / p.m_tiles) * kCtaRows;
            const uint32_t nsub = n0 + kTileN < p.n ? 2u : 1u;
            const bool active = sub < nsub;
            for (uint32_t kb = 0; kb < nkb; ++kb, ++it) {
                const uint32_t s = it % kStages2;
                if (!mbar_wait(&empty[s], ((it / kStages2) & 1u) ^ 1u)) { ok = false; break; }
                if (kb < p.kblocks && active) {
                    const uint32_t my = rit + sub;                  // this group's entry of the current pair
                    const uint32_t rs = my % kRawStages;
                    if ((kb & 1u) == 0 && !mbar_wait(&raw_full[rs], (my / kRawStages) & 1u)) { ok = false; break; }
                    // rows past n were zero-filled by the TMA: scale 0, bias 0, codes 0 -> weights 0
                    uint8_t* a_tile = smem + kOffStages + s * kStage2Bytes + sub * kTileABytes;
#pragma unroll
                    for (uint32_t b = blk; b < 2; b += kDeqWarpsPerSub / 4) {
                        const uint32_t* src = reinterpret_cast<const uint32_t*>(smem + kOffRaw + rs * kRawBytes + r * 80 + (kb & 1u) * 40 + b * 20);
                        uint32_t q[5];
#pragma unroll
                        for (int i = 0; i < 5; ++i) q[i] = src[i];
                        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)(q[0] & 0xffffu)));
                        const __half2 b2 = __half2half2(__ushort_as_half((unsigned short)(q[0] >> 16)));
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<uint4*>(a_tile + swz128(r, 4 * b + j)) = dequant_word_f16(q[1 + j], d2, b2);
                    }
                    fence_async_smem();          // generic-proxy writes -> visible to the tensor core
                    if (kb & 1u) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&raw_empty[rs]);
                    }
                }
                if (kb < p.kblocks && (kb & 1u)) rit += nsub;
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
            }
        }
        if (!ok) { if (lane == 0) atomicOr(p.status, kDevErrBarrierTimeout); *s_err = 1; }
    } else if (warp >= 2 + 2 * kDeqWarpsPerSub && warp < kGemmWarps - 1) {
        // ---------------- epilogue: TMEM -> registers -> Y ----------------
        const uint32_t quarter = (uint32_t)warp & 3u;            // TMEM lanes this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
            const uint32_t buf = tcount % nbuf;
            const uint32_t n0 = ((tile % tps) / p.m_tiles) * kCtaRows;
            const uint32_t nsub = n0 + kTileN < p.n ? 2u : 1u;
            const uint32_t m0 = (tile % p.m_tiles) * p.tt;
            float* yout = p.y + (tile / tps) * p.split_stride;
            if (!mbar_wait(&acc_full[buf], (tcount / nbuf) & 1u)) { ok = false; break; }
            tc_fence_after();
            for (uint32_t sub = 0; sub < nsub; ++sub) {
                const uint32_t n = n0 + sub * kTileN + quarter * 32 + lane;
                for (uint32_t c0 = 0; c0 < p.tt; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ((quarter * 32) << 16) + buf * acc_cols + sub * p.tt + c0, v);
                    tmem_ld_wait();
                    if (n < p.n) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t m = m0 + c0 + j;
                            if (c0 + j < p.tt && m < p.m) yout[(size_t)m * p.ldy + n] = __uint_as_float(v[j]);
                        }
                        // fused all-gather: the same 32 values go to the same place of every peer's buffer (the
                        // accumulator is not double-buffered at 256 tokens per tile, so the stores are kept in
                        // straight runs per peer and out of the single-GPU path)
                        for (uint32_t r = 0; r < p.n_peers; ++r) {
                            float* py = reinterpret_cast<float*>(reinterpret_cast<char*>(yout) + p.peer_off[r]);
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const uint32_t m = m0 + c0 + j;
                                if (c0 + j < p.tt && m < p.m) py[(size_t)m * p.ldy + n] = __uint_as_float(v[j]);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (!ok) { if (lane == 0) atomicOr(p.status, kDevErrBarrierTimeout); *s_err = 1; }
    }

    tc_fence_before();
    __syncthreads();
    if (*s_err) {
        // a bounded wait gave up: let copies still in flight towards this CTA land before it exits
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn gemm_encode_fn() {
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

// f16 matrix [rows, cols] with `stride` halves between rows; box = 64 columns x box_rows, 128-byte swizzle.
bool make_f16_map(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t stride, uint32_t box_rows) {
    EncodeTiledFn fn = gemm_encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {stride * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Packed weights as 4-byte words: box = 4 blocks (20 words) x 128 rows, no swizzle.
bool make_raw_map(CUtensorMap* map, const uint8_t* w, uint32_t n, uint32_t k) {
    EncodeTiledFn fn = gemm_encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)(k / 32) * 5, n};
    const cuuint64_t strides[1] = {(cuuint64_t)(k / 32) * kBlockBytes};
    const cuuint32_t box[2] = {20, (cuuint32_t)kTileN};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(w), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }
inline uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

struct GemmWorkspace {
    size_t x16, al, t, tl, bl, total;
};

// Pieces the k range of the projection T = X A^T is cut into: the largest divisor of k / 64 that is at most
// 16 and keeps (256-token tiles) x pieces within about one wave of CTAs.
uint32_t projection_pieces(uint32_t m, uint32_t k) {
    const uint32_t tiles = (m + kCtaRows - 1) / kCtaRows, kb = k / kBlockK;
    uint32_t best = 1;
    for (uint32_t s = 2; s <= 16 && s <= kb; ++s)
        if (kb % s == 0 && tiles * s <= 160) best = s;
    return best;
}

GemmWorkspace plan_workspace(uint32_t m, uint32_t n, uint32_t k, uint32_t rank, uint32_t limbs) {
    GemmWorkspace ws{};
    const uint32_t rp = round_up(rank, kBlockK);
    size_t off = 0;
    ws.x16 = off; off += up256((size_t)m * limbs * k * 2);
    ws.al = off;  off += up256((size_t)rank * 2 * k * 2);
    ws.t = off;   off += up256((size_t)projection_pieces(m, k) * rank * round_up(m, 4) * 4);
    ws.tl = off;  off += up256((size_t)m * 2 * rp * 2);
    ws.bl = off;  off += up256((size_t)n * 2 * rp * 2);
    ws.total = off;
    return ws;
}

cudaError_t launch_kernel(const GemmParams& p, const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tda,
                          const CUtensorMap& tdb, int sm_count, cudaStream_t s) {
    static DeviceOnce once;            // the shared-memory opt-in is per device
    const size_t smem = kGemmSmem + 1024;
    {
        cudaError_t e = opt_in_smem(reinterpret_cast<const void*>(gemm_tc_kernel), (int)smem, once);
        if (e != cudaSuccess) return e;
    }
    const uint32_t tiles = p.n_tiles * p.m_tiles * p.ksplit;
    const uint32_t grid = tiles < (uint32_t)sm_count ? tiles : (uint32_t)sm_count;
    gemm_tc_kernel<<<grid, kGemmWarps * 32, smem, s>>>(p, tx, tw, tda, tdb);
    return cudaGetLastError();
}

}  // namespace

bool gemm_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t rank) {
    return m > 0 && n > 0 && k > 0 && k % 128 == 0 && rank <= (uint32_t)kGemmMaxRank;
}

size_t gemm_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, uint32_t rank) {
    return plan_workspace(m, n, k, rank, 2).total;
}

cudaError_t launch_gemm_tc(const void* x, int x_dtype, const uint8_t* w, float* y, uint64_t ldy, uint32_t m,
                           uint32_t n, uint32_t k, const float* la, const float* lb, uint32_t rank, float lscale,
                           void* workspace, size_t workspace_bytes, int32_t* status, int sm_count, cudaStream_t s,
                           int* launches, std::string* err, const int64_t* peer_off, uint32_t n_peers) {
    auto fail = [&](const char* what, cudaError_t e) {
        if (err) *err = what;
        return e;
    };
    const uint32_t limbs = x_dtype == LQ4_DTYPE_BF16 ? 1u : 2u;      // bf16 is exact in f16 (normal range)
    const GemmWorkspace ws = plan_workspace(m, n, k, rank, limbs);
    if (ws.total > workspace_bytes) return fail("workspace too small", cudaErrorInvalidValue);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    __half* x16 = reinterpret_cast<__half*>(base + ws.x16);
    const uint32_t rp = round_up(rank, kBlockK);
    int nl = 0;
    cudaError_t e;

    // 1. activations -> f16 limbs, [m][limbs * k]
    {
        const uint64_t n_oct = (uint64_t)m * k / 8;
        const unsigned blocks = (unsigned)((n_oct + 255) / 256 < (uint64_t)sm_count * 8 ? (n_oct + 255) / 256 : (uint64_t)sm_count * 8);
        convert_rows_kernel<<<blocks, 256, 0, s>>>(x, x_dtype, m, k, x16, (uint64_t)limbs * k, limbs == 2 ? k : 0);
        ++nl;
    }
    uint32_t tt = 256 / limbs;
    if (round_up(m, 32) < tt) tt = round_up(m, 32);

    CUtensorMap tm_x, tm_w, tm_da, tm_db;
    if (!make_f16_map(&tm_x, x16, (uint64_t)limbs * k, m, (uint64_t)limbs * k, tt)) return fail("tensor map (x)", cudaErrorInvalidValue);
    if (!make_raw_map(&tm_w, w, n, k)) return fail("tensor map (w)", cudaErrorInvalidValue);
    tm_da = tm_x;
    tm_db = tm_x;

    GemmParams p{};
    p.status = status;
    if (rank) {
        float* t = reinterpret_cast<float*>(base + ws.t);
        uint32_t pieces = 0;                        // 0: t holds T itself, [m][rank]
        const uint64_t mld = round_up(m, 4);        // row length of T^T (16-byte rows)
        if (m <= 32) {
            // few tokens: one warp per (token, rank row) dot product is quicker than a GEMM with one or two tiles
            launch_lora_t(x, x_dtype, m, k, la, rank, t, s);
            if ((e = cudaGetLastError()) != cudaSuccess) return fail("projection launch", e);
            ++nl;
        } else {
            // 2. A -> [Ah | Al] in the activations' column order; 3. T = X A^T on the tensor cores (f32)
            __half* al = reinterpret_cast<__half*>(base + ws.al);
            const uint64_t a_oct = (uint64_t)rank * k / 8;
            convert_rows_kernel<<<(unsigned)((a_oct + 255) / 256), 256, 0, s>>>(la, LQ4_DTYPE_F32, rank, k, al, 2ull * k, k);
            ++nl;
            // X is the 256-row operand (every row of the box is a token), A the narrow one; the k range is
            // cut into pieces so that about one wave of CTAs shares the work.  Output: pieces of T^T.
            CUtensorMap tm_al, tm_xw;
            const uint32_t ta = round_up(rank, 32);
            if (!make_f16_map(&tm_al, al, 2ull * k, rank, 2ull * k, ta)) return fail("tensor map (A)", cudaErrorInvalidValue);
            if (!make_f16_map(&tm_xw, x16, (uint64_t)limbs * k, m, (uint64_t)limbs * k, kCtaRows)) return fail("tensor map (x rows)", cudaErrorInvalidValue);
            pieces = projection_pieces(m, k);
            GemmParams q{};
            q.status = status;
            q.w = w; q.y = t; q.ldy = mld; q.m = rank; q.n = m; q.k = k;
            q.limbs = 1; q.tt = ta; q.n_tiles = (m + kCtaRows - 1) / kCtaRows; q.m_tiles = 1;
            q.kblocks = 0;
            q.ksplit = pieces; q.split_stride = (uint64_t)rank * mld;
            q.seg_len = k / kBlockK / pieces;
            q.seg_a_off[0] = 0; q.seg_b_off[0] = 0;          // Xh . Ah
            q.seg_a_off[1] = 0; q.seg_b_off[1] = k;          // Xh . Al
            q.seg_a_off[2] = k; q.seg_b_off[2] = 0;          // Xl . Ah (two-limb activations only)
            q.lora_kblocks = (limbs == 2 ? 3u : 2u) * q.seg_len;
            if ((e = launch_kernel(q, tm_xw, tm_w, tm_xw, tm_al, sm_count, s)) != cudaSuccess) return fail("projection GEMM launch", e);
            ++nl;
        }
        // 4. hi/lo limbs of T and of s * B
        __half* tl = reinterpret_cast<__half*>(base + ws.tl);
        __half* bl = reinterpret_cast<__half*>(base + ws.bl);
        if (pieces)
            sum_split_transposed_kernel<<<dim3((m + 31) / 32, rp / 8), 256, 0, s>>>(t, pieces, (uint64_t)rank * mld, mld, m, rank, rp, tl);
        else
            split_rows_kernel<<<(unsigned)(((uint64_t)m * rp + 255) / 256), 256, 0, s>>>(t, m, rank, rp, 1.0f, tl);
        const uint64_t bn = (uint64_t)n * rp;
        const unsigned bblocks = (unsigned)((bn + 255) / 256 < (uint64_t)sm_count * 16 ? (bn + 255) / 256 : (uint64_t)sm_count * 16);
        split_rows_kernel<<<bblocks, 256, 0, s>>>(lb, n, rank, rp, lscale, bl);
        nl += 2;
        if (!make_f16_map(&tm_da, bl, 2ull * rp, n, 2ull * rp, kCtaRows)) return fail("tensor map (B)", cudaErrorInvalidValue);
        if (!make_f16_map(&tm_db, tl, 2ull * rp, m, 2ull * rp, tt)) return fail("tensor map (T)", cudaErrorInvalidValue);
        p.seg_len = rp / kBlockK;
        p.seg_a_off[0] = 0;  p.seg_b_off[0] = 0;         // Bh . Th
        p.seg_a_off[1] = rp; p.seg_b_off[1] = 0;         // Bl . Th
        p.seg_a_off[2] = 0;  p.seg_b_off[2] = rp;        // Bh . Tl
        p.lora_kblocks = 3 * p.seg_len;
    } else {
        p.seg_len = 1;
    }
    // 5. the main product
    p.w = w; p.y = y; p.ldy = ldy; p.m = m; p.n = n; p.k = k;
    p.limbs = limbs; p.tt = tt;
    p.n_tiles = (n + kCtaRows - 1) / kCtaRows;
    p.m_tiles = (m + tt - 1) / tt;
    p.kblocks = k / kBlockK;
    p.ksplit = 1;
    if (n_peers > (uint32_t)(LQ4_MAX_PEERS - 1)) return fail("too many peers", cudaErrorInvalidValue);
    p.n_peers = peer_off ? n_peers : 0;
    for (uint32_t r = 0; r < p.n_peers; ++r) p.peer_off[r] = peer_off[r];
    if ((e = launch_kernel(p, tm_x, tm_w, tm_da, tm_db, sm_count, s)) != cudaSuccess) return fail("GEMM launch", e);
    ++nl;
    if (launches) *launches = nl;
    return cudaSuccess;
}

}  // namespace lq4
