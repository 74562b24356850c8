// Decode step kernel: an ordered list of groups of one-token Q4 (+LoRA) projections in ONE persistent
// launch.  The projections of a group are independent; a projection of a later group may read what an
// earlier group wrote (the next layer's input, or gate / up in front of down_proj), on this GPU or - with the
// output rows sharded over several GPUs - on the peers.
//
// Why one launch: a decode step is a chain of 20-microsecond weight streams, and per launch the resident
// kernel pays a fixed price (programmatic hand-over, activation prologue, the spread of CTA end times, and
// across GPUs a release / acquire round trip) that does not shrink with the shard.  Here the CTAs stay
// resident: the TMA warp keeps streaming the NEXT group's weights into the ring while the consumers finish
// the current group and wait for their inputs, so only the data dependency itself is left between groups.
//
// How groups hand data over without fences (a fence in mid-stream waits for the SM's loads in flight):
// every published output is an 8-byte {value, step tag} mailbox entry written with one store, into the
// mailbox of EVERY rank (plain stores over NVLink for the peers).  A reader polls the entries of the k range
// it needs until they carry this step's tag (bounded; a status bit on timeout).  The tag comes from a
// counter every step launch advances by exactly 256 on every rank, so it agrees across the ranks of a
// group; the two halves of the mailbox alternate between steps, so a rank that is one step ahead never
// overwrites what a slower rank still reads.  At the end of the launch every CTA moves its share of the
// gathered ranges from the mailbox to plain f32: when the launch completes on a rank, that rank holds the
// results of all ranks (no wait kernel, no collective).
//
// Inside a group the work is split as in the grouped decode kernel: every problem gets a contiguous share
// of the CTAs in proportion to its cost, stream-K over (128-row tile, 4-block granule), the owner of a
// tile's first k part adds the others' tagged partial sums in CTA order.  Warps: eight consumers (int8
// tensor-core MMAs on nibble codes x two-limb activations), one TMA producer, one projection warp that
// computes the adapters' t = A x for all groups and publishes it as tagged messages.
#include "lq4_step.cuh"

#include "lq4_decode_common.cuh"

namespace lq4 {

namespace {

using namespace gemv;
using namespace dec;

constexpr int kStepThreads = 384;      // 8 consumer warps + TMA warp + projection warp + 2 converter warps
constexpr int kConvWarps = 2;          // (ptxas sizes the register budget for 384 threads anyway: these warps are free)
constexpr int kConvThreads = kConvWarps * 32;
constexpr int kBarConverters = 2;      // named barrier of the converter warps
constexpr uint32_t kXBarOffset = 2 * kMaxStages * 8 + 32;      // xready, xfree, tready, tfree [2 each] after the ring's barriers and the zero block

// Development aid, compiled only with -DLQ4_STEP_TIMELINE: nanosecond stamps per CTA and group.
#ifdef LQ4_STEP_TIMELINE
constexpr int kTlSlots = 12;           // per (cta, group): 0 group start, 1 prologue done, 2 last stage consumed,
                                       // 3 last epilogue done, 4 projection start, 5 projection done, 6 first stage consumed,
                                       // 7 converters start, 8 limbs built, 9 projection gathered
__device__ unsigned long long g_step_timeline[160 * kStepMaxGroups * kTlSlots + 8];
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TL_STAMP(g, slot) do { g_step_timeline[((size_t)blockIdx.x * kStepMaxGroups + (g)) * kTlSlots + (slot)] = tl_now(); } while (0)
#else
#define TL_STAMP(g, slot) do { } while (0)
#endif

__device__ __forceinline__ unsigned long long mbox_pack(float v, uint32_t tag) {
    return ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
}
// One 8-byte store: the tag arrives with the value (single-copy atomic), on this GPU or on a peer.
__device__ __forceinline__ void mbox_store(unsigned long long* p, unsigned long long e) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(e) : "memory");
}
__device__ __forceinline__ unsigned long long mbox_load(const unsigned long long* p) {
    unsigned long long e;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(e) : "l"(p) : "memory");
    return e;
}
// Two entries with one 16-byte load that is served by L2 and never by this SM's L1 (.cg).  Deliberately not a
// system-scope "strong" load: measured on B200, strong loads of one thread complete one after the other
// (about 0.2 us each), which made a 90-load dot product take 20 us; the sweeps below need dozens of loads in
// flight.  L2 is where stores from this GPU and from the peers (over NVLink) land, each 8-byte entry is written
// by a single store, and every sweep is re-executed until the tags match, so what a sweep sees is either the
// old entry or the new one.
__device__ __forceinline__ void mbox_load2(const unsigned long long* p, unsigned long long& e0, unsigned long long& e1) {
    asm volatile("ld.global.cg.v2.u64 {%0, %1}, [%2];" : "=l"(e0), "=l"(e1) : "l"(p) : "memory");
}
// Eight consecutive entries (32-byte aligned), loads only: the caller issues the loads of a whole batch before
// it looks at the first tag, so a batch costs one L2 round trip.
__device__ __forceinline__ void mbox_load8_raw(const unsigned long long* p, unsigned long long (&e)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) mbox_load2(p + 2 * i, e[2 * i], e[2 * i + 1]);
}
__device__ __forceinline__ bool mbox_unpack8(const unsigned long long (&e)[8], uint32_t stag, float (&v)[8]) {
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        ok = ok && (uint32_t)(e[i] >> 32) == stag;
        v[i] = __uint_as_float((uint32_t)e[i]);
    }
    return ok;
}

// Cheap gate in front of a mailbox sweep: ONE lane of the warp polls ONE entry, with a growing pause,
// until it carries this step's tag; the warp follows.  Readers get here microseconds before their inputs
// exist; if every waiting thread swept its whole range meanwhile, the polling traffic of 148 CTAs would
// compete in L2 with the weight stream of the CTAs that still produce those inputs.  The probe says
// nothing about the other entries: the sweep after it still checks every tag.
__device__ __forceinline__ void mbox_probe_wait(const unsigned long long* p, uint32_t stag, volatile int* err) {
    if ((threadIdx.x & 31) == 0) {
        unsigned ns = 128;
        const long long t0 = wait_clock();
        while ((uint32_t)(mbox_load(p) >> 32) != stag) {
            if (*err || wait_expired(t0)) break;       // the sweep that follows reports the failure
            __nanosleep(ns);
            ns = ns < 1024 ? ns * 2 : 1024;
        }
    }
    __syncwarp();
}

// Requests the 128-byte lines of [p, p + bytes) into L2, the lines dealt round-robin to `nt` threads.
__device__ __forceinline__ void prefetch_l2_range(const char* p, size_t bytes, int ctid, int nt) {
    if (bytes == 0) return;
    const char* first = reinterpret_cast<const char*>(reinterpret_cast<uintptr_t>(p) & ~(uintptr_t)127);
    const char* end = p + bytes;
    for (const char* l = first + (size_t)ctid * 128; l < end; l += (size_t)nt * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(l));
}

// mbarrier wait that also gives up as soon as another wait of this CTA has failed.
__device__ __forceinline__ bool mbar_wait_step(uint64_t* bar, uint32_t parity, volatile int* err) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = wait_clock();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*err || wait_expired(t0)) return false;
    }
}

// This CTA's share of group g: its problem and its range of work units, or nothing.
struct Share {
    uint32_t pi;
    uint32_t r0, r1;      // work units tile * kg + granule: 32 bits (the host refuses problems beyond that)
    bool any;
};
__device__ __forceinline__ Share step_share(const StepArgs& a, uint32_t g, uint32_t cta) {
    Share s;
    s.pi = 0; s.r0 = s.r1 = 0; s.any = false;
    for (uint32_t i = a.group_begin[g]; i < a.group_begin[g + 1]; ++i) {
        const StepProblem& q = a.p[i];
        if (cta >= q.cta_begin && cta < q.cta_begin + q.cta_count) {
            s.pi = i;
            s.r0 = step_share_begin_t<uint32_t>(cta - q.cta_begin, q.tiles, q.kg, q.charge, q.cta_count);
            s.r1 = step_share_begin_t<uint32_t>(cta - q.cta_begin + 1, q.tiles, q.kg, q.charge, q.cta_count);
            s.any = s.r1 > s.r0;
            break;
        }
    }
    return s;
}

// Activation limbs from mailbox entries.  An L2 round trip costs about a microsecond while the weight stream is
// running, and a thread's loads only overlap if they are issued before the first result is used: a sweep issues
// the loads of KB octets (4 x 16 bytes each) back to back, then looks at the tags; entries that are not there yet
// repeat the sweep.  Warp-uniform (the conversion uses quad shuffles), bounded, with a pause between sweeps.
template <int NT, int KB, bool GATED>
__device__ __forceinline__ void prologue_from_mailbox(const StepArgs& a, uint8_t* xs, float2* sx, const unsigned long long* xm,
                                                      const unsigned long long* um, uint32_t a0, uint32_t na, uint32_t b0,
                                                      uint32_t noct, int ctid, uint32_t stag, volatile int* s_err) {
    for (uint32_t o0 = 0; o0 < noct; o0 += KB * NT) {
        float v[KB][8];
        {
            const uint32_t i = o0 + (uint32_t)(ctid & ~31);      // the first octet this warp reads in this sweep
            if (i < noct) mbox_probe_wait(xm + (size_t)(i < na ? a0 + i : b0 + (i - na)) * 8, stag, s_err);
        }
        const long long t0 = wait_clock();
        for (;;) {
            bool ready = true;
            unsigned long long ex[KB][8], eu[GATED ? KB : 1][8];
#pragma unroll
            for (int u = 0; u < KB; ++u) {
                const uint32_t i = o0 + u * NT + ctid;
                if (i < noct) {
                    const size_t o = (size_t)(i < na ? a0 + i : b0 + (i - na)) * 8;
                    mbox_load8_raw(xm + o, ex[u]);
                    if (GATED) mbox_load8_raw(um + o, eu[GATED ? u : 0]);
                }
            }
#pragma unroll
            for (int u = 0; u < KB; ++u) {
                const uint32_t i = o0 + u * NT + ctid;
#pragma unroll
                for (int e = 0; e < 8; ++e) v[u][e] = 0.0f;
                if (i < noct) {
                    ready = mbox_unpack8(ex[u], stag, v[u]) && ready;
                    if (GATED) {
                        float up[8];
                        ready = mbox_unpack8(eu[GATED ? u : 0], stag, up) && ready;
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[u][e] = silu_mul(v[u][e], up[e]);
                    }
                }
            }
            if (__all_sync(kFull, ready)) break;
            if (__any_sync(kFull, *s_err != 0 || wait_expired(t0))) {
                if ((ctid & 31) == 0) atomicOr(a.status, kDevErrGridWaitTimeout);
                *s_err = 1;
                break;
            }
            __nanosleep(256);
        }
#pragma unroll
        for (int u = 0; u < KB; ++u) {
            const uint32_t i = o0 + u * NT + ctid;
            store_limbs(xs, sx, 1, 0, i, i < noct, v[u]);      // the buffer is indexed from the start of the range
        }
    }
}

// The last CTA that works on `tile`, for the CTA that owns the tile's first granule: walks on from this CTA
// (the next one or two, as a rule).  Runs once per finished tile.  Measured: as a call it keeps its divisions out
// of the stage loop's register allocation (1 us per step on the plain-input instantiation); the mailbox-fed
// instantiation, which spills either way, is quicker with it inlined.
__device__ __forceinline__ uint32_t tile_last_cta_inline(const StepProblem& q, uint32_t tile) {
    return q.cta_begin + step_share_last_t<uint32_t>(blockIdx.x - q.cta_begin, (tile + 1) * q.kg - 1, q.tiles, q.kg, q.charge, q.cta_count);
}
__device__ __noinline__ uint32_t tile_last_cta_call(const StepProblem& q, uint32_t tile) { return tile_last_cta_inline(q, tile); }

// First block and octet ranges of the k range(s) a share [r0, r1) of work units touches: the whole row when the
// share spans a tile, else up to two pieces (the share may wrap from the end of one tile into the next).
struct XRange {
    uint32_t a0, na, b0, noct;     // octets: piece a = [a0, a0 + na), piece b = [b0, b0 + noct - na)
    uint32_t base_blk;             // first block of piece a: the limb buffer is indexed from here, wrapping at k / 32
};
__device__ __forceinline__ XRange step_xrange(const StepProblem& q, uint32_t r0, uint32_t r1) {
    const uint32_t opg = kGemvGranuleBlocks * 4;              // octets (8 activations) per granule
    uint32_t a0 = 0, a1 = q.k / 8, b0 = 0, b1 = 0;
    if (r1 - r0 < q.kg) {
        const uint32_t g0 = (uint32_t)(r0 % q.kg), len = (uint32_t)(r1 - r0);
        if (g0 + len <= q.kg) { a0 = g0 * opg; a1 = (g0 + len) * opg; }
        else { a0 = g0 * opg; a1 = q.kg * opg; b0 = 0; b1 = (g0 + len - q.kg) * opg; }
    }
    XRange x;
    x.a0 = a0; x.na = a1 - a0; x.b0 = b0; x.noct = x.na + (b1 - b0); x.base_blk = a0 / 4;
    return x;
}

// One thread builds the limbs of a whole Q4 block (32 activations): no exchange between lanes.  The converter
// warps use this form: their quad shuffles, issued beside the consumers' shared-memory loads, took up to four
// times as long as alone (measured with device time stamps), and a conversion that is late stops the consumers.
// Same arithmetic and the same order of additions as store_limbs, so both give the same bytes.
__device__ __forceinline__ void store_limbs_block(uint8_t* xs, float2* sx, uint32_t blk, const float (&v)[32]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    float so[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float* w = v + 8 * j;
        so[j] = ((w[0] + w[1]) + (w[2] + w[3])) + ((w[4] + w[5]) + (w[6] + w[7]));
    }
    const float sum = (so[0] + so[1]) + (so[2] + so[3]);
    uint32_t l0[8], l1[8];
    float scale = 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = v[8 * j + e];
        const Limbs8 l = make_limbs8(w, amax);
        l0[2 * j] = l.l0a; l0[2 * j + 1] = l.l0b;
        l1[2 * j] = l.l1a; l1[2 * j + 1] = l.l1b;
        scale = l.scale;
    }
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)blk * 64);
    dst[0] = make_uint4(l0[0], l0[1], l0[2], l0[3]);
    dst[1] = make_uint4(l0[4], l0[5], l0[6], l0[7]);
    dst[2] = make_uint4(l1[0], l1[1], l1[2], l1[3]);
    dst[3] = make_uint4(l1[4], l1[5], l1[6], l1[7]);
    sx[blk] = make_float2(scale, sum);
}

// The converter warps' conversion of a share's k range(s) from plain memory, a block per thread and turn.  The
// loop is kept small on purpose (one block's arithmetic, the next block's loads issued before it): these warps
// share their schedulers' instruction caches with the consumers' stage loop.
template <int NT>
__device__ __forceinline__ void convert_blocks_plain(const StepProblem& q, uint8_t* xs, float2* sx, int ctid, const XRange& xr) {
    const uint32_t nblk = xr.noct / 4, nba = xr.na / 4, a0b = xr.a0 / 4, b0b = xr.b0 / 4;      // ranges are whole granules
    auto load_block = [&](uint32_t i, float (&v)[32]) {
        const uint32_t o = i < nba ? a0b + i : b0b + (i - nba);
#pragma unroll
        for (int j = 0; j < 4; ++j) load8(q.x, q.x_dtype, (size_t)o * 32 + 8 * j, *reinterpret_cast<float(*)[8]>(&v[8 * j]));
        if (q.x_mul) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float up[8];
                load8(q.x_mul, LQ4_DTYPE_F32, (size_t)o * 32 + 8 * j, up);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[8 * j + e] = silu_mul(v[8 * j + e], up[e]);
            }
        }
    };
    float cur[32];
    uint32_t i = ctid;
    if (i < nblk) load_block(i, cur);
#pragma unroll 1
    for (; i < nblk; i += NT) {
        float nxt[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) nxt[e] = 0.0f;
        if (i + NT < nblk) load_block(i + NT, nxt);
        store_limbs_block(xs, sx, i, cur);
#pragma unroll
        for (int e = 0; e < 32; ++e) cur[e] = nxt[e];
    }
}

// NT threads turn the k range(s) of a share into two int8 limbs per activation, into the limb buffer (xs, sx).
// MAILBOX: the input comes from the step's mailbox (polled); else from plain memory.
template <bool MAILBOX, int NT>
__device__ __forceinline__ void convert_activations(const StepArgs& a, const StepProblem& q, uint8_t* xs, float2* sx, int ctid,
                                                    const XRange& xr, const unsigned long long* mb, uint32_t stag,
                                                    volatile int* s_err) {
    const uint32_t a0 = xr.a0, na = xr.na, b0 = xr.b0, noct = xr.noct;
    if constexpr (!MAILBOX) {
        // plain memory: several octets per thread and pass, all loads issued before the first use
        constexpr int kBatch = 8;
        for (uint32_t o0 = 0; o0 < noct; o0 += kBatch * NT) {
            float v[kBatch][8];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint32_t i = o0 + u * NT + ctid;
                const uint32_t o = i < na ? a0 + i : b0 + (i - na);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[u][e] = 0.0f;
                if (i < noct) load8(q.x, q.x_dtype, (size_t)o * 8, v[u]);
            }
            if (q.x_mul) {
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const uint32_t i = o0 + u * NT + ctid;
                    const uint32_t o = i < na ? a0 + i : b0 + (i - na);
                    if (i < noct) {
                        float up[8];
                        load8(q.x_mul, LQ4_DTYPE_F32, (size_t)o * 8, up);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[u][e] = silu_mul(v[u][e], up[e]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint32_t i = o0 + u * NT + ctid;
                store_limbs(xs, sx, 1, 0, i, i < noct, v[u]);      // the buffer is indexed from the start of the range
            }
        }
    } else {
        // Octets per thread and sweep: 2 (1 with a gating row).  Larger sweeps save L2 round trips but their
        // registers spill, and the spill code lands in the consumers' stage loop: with 4 (2) the whole
        // instantiation ran 26 % slower on plain inputs and the chained bench step took 144 us instead of 112.
        const unsigned long long* xm = mb + q.x_slot;
        if (q.xmul_slot != kNoSlot) prologue_from_mailbox<NT, 1, true>(a, xs, sx, xm, mb + q.xmul_slot, a0, na, b0, noct, ctid, stag, s_err);
        else prologue_from_mailbox<NT, 2, false>(a, xs, sx, xm, nullptr, a0, na, b0, noct, ctid, stag, s_err);
    }
}

// The projection warp (one per CTA): the adapters' t = A x for every group, published as tagged messages.
// Work item e of group g = (problem, rank row j, k piece): item e belongs to CTA e mod grid.  Items of a later
// group wait (inside the dot product) for their inputs' mailbox entries.
template <bool MB>
__device__ __forceinline__ void step_projections(const StepArgs& a, volatile int* s_err) {
    const int lane = threadIdx.x & 31;
            // Work item e of group g = (problem, rank row j, k piece): item e belongs to CTA e mod grid.  Items
            // of a later group wait (inside the dot product) for their inputs' mailbox entries.
            if (a.use_pdl) pdl_wait_prior_grids();
            const uint32_t tag = launch_tag(a.tsync);
            const uint32_t stag = launch_tag(a.step_counter);
            const unsigned long long* mb = a.mbox + (size_t)(stag & 1u) * a.mbox_half;
            for (uint32_t g = 0; g < a.ngroups; ++g) {
                const uint32_t nitems = a.group_items[g];
                uint32_t pj = a.group_begin[g];
                const uint32_t pend = a.group_begin[g + 1];
                if (lane == 0) TL_STAMP(g, 4);
                for (uint32_t e = blockIdx.x; e < nitems; e += gridDim.x) {
                    while (pj + 1 < pend && e >= a.p[pj + 1].dot_begin) ++pj;
                    const StepProblem& q = a.p[pj];
                    const uint32_t local = e - q.dot_begin;
                    const uint32_t j = local / q.tsplit, sp = local - j * q.tsplit;
                    const uint32_t k4 = q.k / 4;
                    const uint32_t chunk4 = ((k4 + q.tsplit - 1) / q.tsplit + 31u) & ~31u;
                    const uint32_t i0 = sp * chunk4, i1 = min(k4, i0 + chunk4);
                    const float* arow = q.la + (size_t)j * q.k;
                    const float4* a4 = reinterpret_cast<const float4*>(arow);
                    float s = 0.0f;
                    if (MB && q.x_slot != kNoSlot) {
                        const unsigned long long* xm = mb + q.x_slot;
                        const unsigned long long* um = q.xmul_slot != kNoSlot ? mb + q.xmul_slot : nullptr;
                        if (i0 < i1) mbox_probe_wait(xm + (size_t)(i1 - 1) * 4, stag, s_err);
                        // The host cuts the dot products of mailbox-fed problems into pieces of at most
                        // kStepMailboxPiece4 float4 per lane stride x 32 lanes, so a lane has at most UB strides: all
                        // its loads are in flight together and an attempt costs one L2 round trip per row.
                        constexpr int UB = kStepMailboxStrides;
                        const long long t0 = wait_clock();
                        for (;;) {
                            bool ready = true;
                            s = 0.0f;
                            for (uint32_t ib = i0 + lane; ib < i1; ib += 32 * UB) {
                                unsigned long long ex[UB][4];
                                float4 av[UB];
                                float xv[UB][4];
                                unsigned long long eu[UB][4];
#pragma unroll
                                for (int b = 0; b < UB; ++b) {
                                    const uint32_t i = ib + 32 * b;
                                    if (i < i1) {
                                        av[b] = __ldg(a4 + i);
                                        mbox_load2(xm + (size_t)i * 4, ex[b][0], ex[b][1]);
                                        mbox_load2(xm + (size_t)i * 4 + 2, ex[b][2], ex[b][3]);
                                        if (um) {
                                            mbox_load2(um + (size_t)i * 4, eu[b][0], eu[b][1]);
                                            mbox_load2(um + (size_t)i * 4 + 2, eu[b][2], eu[b][3]);
                                        }
                                    }
                                }
#pragma unroll
                                for (int b = 0; b < UB; ++b) {
                                    const uint32_t i = ib + 32 * b;
                                    if (i < i1) {
#pragma unroll
                                        for (int c = 0; c < 4; ++c) {
                                            ready = ready && (uint32_t)(ex[b][c] >> 32) == stag;
                                            xv[b][c] = __uint_as_float((uint32_t)ex[b][c]);
                                            if (um) {
                                                ready = ready && (uint32_t)(eu[b][c] >> 32) == stag;
                                                xv[b][c] = silu_mul(xv[b][c], __uint_as_float((uint32_t)eu[b][c]));
                                            }
                                        }
                                    }
                                }
#pragma unroll
                                for (int b = 0; b < UB; ++b) {
                                    const uint32_t i = ib + 32 * b;
                                    if (i < i1) {
                                        s = fmaf(av[b].x, xv[b][0], s); s = fmaf(av[b].y, xv[b][1], s);
                                        s = fmaf(av[b].z, xv[b][2], s); s = fmaf(av[b].w, xv[b][3], s);
                                    }
                                }
                            }
                            if (__all_sync(kFull, ready)) break;
                            if (__any_sync(kFull, *s_err != 0 || wait_expired(t0))) {
                                if (lane == 0) atomicOr(a.status, kDevErrGridWaitTimeout);
                                *s_err = 1;
                                break;
                            }
                            __nanosleep(512);
                        }
                    } else if (q.x_mul) {
                        const float4* g4 = reinterpret_cast<const float4*>(q.x);
                        const float4* u4 = reinterpret_cast<const float4*>(q.x_mul);
    #pragma unroll 8
                        for (uint32_t i = i0 + lane; i < i1; i += 32) {
                            const float4 av = __ldg(a4 + i), gv = g4[i], uv = u4[i];
                            s = fmaf(av.x, silu_mul(gv.x, uv.x), s); s = fmaf(av.y, silu_mul(gv.y, uv.y), s);
                            s = fmaf(av.z, silu_mul(gv.z, uv.z), s); s = fmaf(av.w, silu_mul(gv.w, uv.w), s);
                        }
                    } else if (q.x_dtype == LQ4_DTYPE_F32) {
                        const float4* x4 = reinterpret_cast<const float4*>(q.x);
    #pragma unroll 8
                        for (uint32_t i = i0 + lane; i < i1; i += 32) {
                            const float4 av = __ldg(a4 + i), b = x4[i];
                            s = fmaf(av.x, b.x, s); s = fmaf(av.y, b.y, s); s = fmaf(av.z, b.z, s); s = fmaf(av.w, b.w, s);
                        }
                    } else {
    #pragma unroll 8
                        for (uint32_t i = i0 * 4 + lane; i < i1 * 4; i += 32)
                            s = fmaf(__ldg(arow + i), load_act(q.x, q.x_dtype, i), s);
                    }
    #pragma unroll
                    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
                    if (lane == 0) msg_store(q.tmsg + local, s, tag);
                }
                if (lane == 0) TL_STAMP(g, 5);
            }
}

// MB: some projection of the launch takes its input from the mailbox.  Launches without such inputs run the
// instantiation that holds none of the polling code (the kernel sits at the register limit of a 12-warp CTA).
template <bool MB>
__global__ void __launch_bounds__(kStepThreads, 1) decode_step_kernel(const __grid_constant__ StepArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    __shared__ int s_err_mem;
    volatile int* s_err = &s_err_mem;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t NST = a.nstages;
    uint64_t* xready = reinterpret_cast<uint64_t*>(smem + kXBarOffset);     // limb buffer b holds the group's limbs
    uint64_t* xfree = xready + 2;                                           // the consumers are done with limb buffer b
    uint64_t* tready = xfree + 2;                                           // t = A x of the group is in t buffer b
    uint64_t* tfree = tready + 2;                                           // the consumers are done with t buffer b
    if (tid == 0) {
        for (uint32_t s = 0; s < NST; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 8);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&xready[b], kConvWarps);
            mbar_init(&xfree[b], 8);
            mbar_init(&tready[b], kConvWarps);
            mbar_init(&tfree[b], 8);
        }
        s_err_mem = 0;
        for (int i = 0; i < 8; ++i) reinterpret_cast<uint32_t*>(smem + kZeroOffset)[i] = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (a.use_pdl) pdl_launch_dependents();
    uint32_t issued = 0;

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        // Walks the CTA's shares of ALL groups back to back: weights do not depend on anything, so the ring
        // keeps filling with the next group's tiles while the consumers finish the current group.
        const uint64_t pol = l2_policy_evict_first();
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t g = 0; g < a.ngroups && ok; ++g) {
            const Share sh = step_share(a, g, blockIdx.x);
            if (!sh.any) continue;
            const StepProblem& q = a.p[sh.pi];
            for (uint32_t pos = sh.r0; pos < sh.r1 && ok;) {
                const uint32_t tile = pos / q.kg;
                const uint32_t g0 = pos - tile * q.kg;
                const uint32_t left = sh.r1 - pos;
                const uint32_t g1 = q.kg - g0 < left ? q.kg : g0 + left;
                for (uint32_t gs = g0; gs < g1; ++it) {
                    const uint32_t ngr = stage_granules(g1 - gs);
                    const uint32_t s = it % NST;
                    bool got = true;
                    if (lane == 0) got = mbar_wait_step(&empty[s], ((it / NST) & 1u) ^ 1u, s_err);
                    if (!__shfl_sync(kFull, got, 0)) { ok = false; break; }
                    if (lane == 0) {
                        uint8_t* st = smem + a.off_stage + (size_t)s * kSlotBytes;
                        mbar_arrive_expect_tx(&full[s], ngr * kSmallBytes);
                        tma_load_2d(st, &a.maps[sh.pi][ngr == 5 ? 0 : (ngr == 3 ? 1 : 2)], (int32_t)(gs * kGemvGranuleBlocks * 5),
                                    (int32_t)(tile * kGemvTileRows), &full[s], pol);
                    }
                    gs += ngr;
                }
                pos += g1 - g0;
            }
        }
        issued = it;
        if (!ok && lane == 0) {
            atomicOr(a.status, kDevErrBarrierTimeout);
            *s_err = 1;
        }
    } else if (warp == 9) {
        step_projections<MB>(a, s_err);
    } else if (warp >= 10) {
        // ------------------------------ activation converters ------------------------------
        // Build the limbs of the CTA's NEXT shares while the consumers work: with two limb buffers they run a
        // whole group ahead, so the consumers never stop to convert (during a conversion by the consumers the
        // ring stays full and the SM requests nothing from memory: about 2 us per group).  Inputs that come from
        // the mailbox are converted by the consumers themselves, who have four times the threads for the sweeps.
        const int ctid = tid - 320;
        if (a.use_pdl) pdl_wait_prior_grids();
        const uint32_t tag = launch_tag(a.tsync);
        float* cstage = reinterpret_cast<float*>(smem + a.off_cstage);
        uint32_t gcount = 0;
        for (uint32_t g = 0; g < a.ngroups; ++g) {
            const Share sh = step_share(a, g, blockIdx.x);
            if (!sh.any) continue;
            const StepProblem& q = a.p[sh.pi];
            const uint32_t b = gcount % a.nxbuf, use = gcount / a.nxbuf;
            ++gcount;
            const bool convert_here = MB ? q.x_slot == kNoSlot : gcount != 1;
            const XRange xr = step_xrange(q, sh.r0, sh.r1);
            if (convert_here) {
                // Pull the share's activations towards L2 while waiting for the limb buffer: a load that has to go
                // to memory queues behind the weight stream (several microseconds per pass when the ring is being
                // refilled), and the passes of the conversion run one after the other.
                const uint32_t ob = q.x_dtype == LQ4_DTYPE_BF16 ? 16u : 32u;      // bytes per octet
                prefetch_l2_range(static_cast<const char*>(q.x) + (size_t)xr.a0 * ob, (size_t)xr.na * ob, ctid, kConvThreads);
                prefetch_l2_range(static_cast<const char*>(q.x) + (size_t)xr.b0 * ob, (size_t)(xr.noct - xr.na) * ob, ctid, kConvThreads);
                if (q.x_mul) {
                    prefetch_l2_range(reinterpret_cast<const char*>(q.x_mul) + (size_t)xr.a0 * 32, (size_t)xr.na * 32, ctid, kConvThreads);
                    prefetch_l2_range(reinterpret_cast<const char*>(q.x_mul) + (size_t)xr.b0 * 32, (size_t)(xr.noct - xr.na) * 32, ctid, kConvThreads);
                }
            }
            if (lane == 0 && !mbar_wait_step(&xfree[b], (use & 1u) ^ 1u, s_err)) {
                atomicOr(a.status, kDevErrBarrierTimeout);
                *s_err = 1;
            }
            __syncwarp();
            if (ctid == 0) TL_STAMP(g, 7);
            // the first share's limbs are on the critical path of the launch: the consumers build them themselves
            // (four times the threads) while these warps start on the second share
            if (convert_here) {                                // (only in the instantiation that has the registers for it)
                uint8_t* xs = smem + a.off_xbuf + (size_t)b * a.xbuf_stride;
                float2* sx = reinterpret_cast<float2*>(xs + a.xbuf_sx);
                convert_blocks_plain<kConvThreads>(q, xs, sx, ctid, xr);
            }
            __syncwarp();
            if (ctid == 0) TL_STAMP(g, 8);
            if (lane == 0) mbar_arrive(&xready[b]);
            // ... and gather the adapter projection t = A x of the same share's problem (published by the
            // projection warps of all CTAs in the first microseconds when the input is plain), so that the
            // consumers find it in shared memory at their first epilogue instead of fetching it themselves
            if (lane == 0 && !mbar_wait_step(&tfree[b], (use & 1u) ^ 1u, s_err)) {
                atomicOr(a.status, kDevErrBarrierTimeout);
                *s_err = 1;
            }
            __syncwarp();
            if (q.rank && (!MB || q.x_slot == kNoSlot)) {
                float* tb = reinterpret_cast<float*>(smem + a.off_t + (size_t)b * a.t_stride);
                const uint32_t nmsg = q.rank * q.tsplit;
                bool good = true;
                for (uint32_t idx = ctid; idx < nmsg; idx += kConvThreads) {
                    uint2 msg = msg_load(q.tmsg + idx);
                    if (msg.y != tag) {
                        const long long t0 = wait_clock();
                        unsigned ns = 128;
                        for (;;) {
                            __nanosleep(ns);
                            ns = ns < 1024 ? ns * 2 : 1024;
                            msg = msg_load(q.tmsg + idx);
                            if (msg.y == tag) break;
                            if (*s_err != 0 || wait_expired(t0)) { good = false; break; }
                        }
                    }
                    cstage[idx] = __uint_as_float(msg.x);
                }
                if (!good) { atomicOr(a.status, kDevErrGridWaitTimeout); *s_err = 1; }
                named_bar_sync(kBarConverters, kConvThreads);
                for (uint32_t j = ctid; j < q.rank; j += kConvThreads) {
                    float sum = 0.0f;
                    for (uint32_t sp = 0; sp < q.tsplit; ++sp) sum += cstage[j * q.tsplit + sp];      // piece order: fixed sum
                    tb[j] = sum;
                }
                named_bar_sync(kBarConverters, kConvThreads);      // the staging area is free for the next group
            }
            __syncwarp();
            if (ctid == 0) TL_STAMP(g, 9);
            if (lane == 0) mbar_arrive(&tready[b]);
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int gq = lane >> 2, t = lane & 3;
        if (a.use_pdl) pdl_wait_prior_grids();
        const uint32_t tag = launch_tag(a.tsync);
        const uint32_t stag = launch_tag(a.step_counter);
        unsigned long long* mb = a.mbox + (size_t)(stag & 1u) * a.mbox_half;

        const bool has_b = (gq >> 1) == t;
        const uint8_t* zeros = smem + kZeroOffset;
        uint32_t gcount = 0;

        // A failed wait (its time limit, or another wait of this CTA failed before) never changes the control
        // flow: every warp keeps walking the same groups, tiles and stages, so the named barriers below always
        // see all eight warps; once s_err is set every later wait returns at once and the walk is short.
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t g = 0; g < a.ngroups; ++g) {
            const Share sh = step_share(a, g, blockIdx.x);
            if (!sh.any) continue;                                 // the same for every thread of the CTA
            const StepProblem& q = a.p[sh.pi];
            // everyone is done with the previous group's limbs and projection before they are replaced
            named_bar_sync(kBarConsumers, kConsumerThreads);
            if (tid == 0) TL_STAMP(g, 0);
            // this group's limb buffer: filled by the converter warps (plain inputs) or, below, by the consumers
            const uint32_t xb_i = gcount % a.nxbuf, xb_use = gcount / a.nxbuf;
            ++gcount;
            uint8_t* xs_buf = smem + a.off_xbuf + (size_t)xb_i * a.xbuf_stride;
            const float2* sx_all = reinterpret_cast<const float2*>(xs_buf + a.xbuf_sx);
            const uint8_t* xs_lane = xs_buf + (size_t)(gq & 1) * 32;
            const XRange xr = step_xrange(q, sh.r0, sh.r1);
            float* t_sm = reinterpret_cast<float*>(smem + a.off_t + (size_t)xb_i * a.t_stride);
            const bool helper_t = !MB || q.x_slot == kNoSlot;      // the converter warps gather t for plain inputs
            if (!mbar_wait_step(&xready[xb_i], xb_use & 1u, s_err)) { ok = false; *s_err = 1; }
            if constexpr (MB) {
                if (q.x_slot != kNoSlot) {
                    convert_activations<true, kConsumerThreads>(a, q, xs_buf, reinterpret_cast<float2*>(xs_buf + a.xbuf_sx), tid, xr,
                                                                mb, stag, s_err);
                    named_bar_sync(kBarConsumers, kConsumerThreads);
                }
            }
            if constexpr (!MB) {
                if (gcount == 1) {      // the first share (gcount was just advanced)
                    convert_activations<false, kConsumerThreads>(a, q, xs_buf, reinterpret_cast<float2*>(xs_buf + a.xbuf_sx), tid,
                                                                 xr, nullptr, 0, s_err);
                    named_bar_sync(kBarConsumers, kConsumerThreads);
                }
            }
            if (tid == 0) TL_STAMP(g, 1);
            bool t_loaded = false;
            // Gathers t = A x of this problem from the projection warps' messages into shared memory, adding
            // the k pieces of every dot product in order.  All consumer warps call it at the same point.
            auto gather_t = [&]() {
                // one message per thread and sweep (all in flight together), staged in shared memory, then every
                // dot product's pieces are added in piece order by one thread: the sum does not depend on timing
                float* stage = reinterpret_cast<float*>(smem + a.off_tstage);
                const uint32_t nmsg = q.rank * q.tsplit;
                bool good = true;
                for (uint32_t idx = tid; idx < nmsg; idx += kConsumerThreads) {
                    uint2 msg = msg_load(q.tmsg + idx);
                    if (msg.y != tag) {
                        const long long t0 = wait_clock();
                        for (;;) {
                            __nanosleep(128);
                            msg = msg_load(q.tmsg + idx);
                            if (msg.y == tag) break;
                            if (*s_err != 0 || wait_expired(t0)) { good = false; break; }
                        }
                    }
                    stage[idx] = __uint_as_float(msg.x);
                }
                if (!good) { atomicOr(a.status, kDevErrGridWaitTimeout); *s_err = 1; }
                named_bar_sync(kBarConsumers, kConsumerThreads);
                for (uint32_t j = tid; j < q.rank; j += kConsumerThreads) {
                    float sum = 0.0f;
                    for (uint32_t sp = 0; sp < q.tsplit; ++sp) sum += stage[j * q.tsplit + sp];
                    t_sm[j] = sum;
                }
                named_bar_sync(kBarConsumers, kConsumerThreads);
                t_loaded = true;
            };
            uint32_t git = 0;                                      // stages of this group consumed so far
            for (uint32_t pos = sh.r0; pos < sh.r1;) {
                const uint32_t tile = pos / q.kg;
                const uint32_t g0 = pos - tile * q.kg;
                const uint32_t left = sh.r1 - pos;
                const uint32_t g1 = q.kg - g0 < left ? q.kg : g0 + left;
                pos += g1 - g0;

                float acc0 = 0.0f, acc1 = 0.0f;
                if (q.rank && g0 == 0) {
                    // this CTA will finish the tile: pull the warp's 16 rows of LoRA B towards L2 now
                    const uint32_t rfirst = tile * kGemvTileRows + warp * 16;
                    const uint32_t rows = rfirst < q.n ? min(16u, q.n - rfirst) : 0u;
                    const char* bb = reinterpret_cast<const char*>(q.lb + (size_t)rfirst * q.rank);
                    for (uint32_t off = lane * 128; off < rows * q.rank * 4; off += 32 * 128)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(bb + off));
                }
                for (uint32_t gs = g0; gs < g1; ++it, ++git) {
                    const uint32_t ngr = stage_granules(g1 - gs);
                    const uint32_t rs = ngr * (kGemvGranuleBlocks * kBlockBytes);
                    const uint32_t s = it % NST;
                    if (!mbar_wait_step(&full[s], (it / NST) & 1u, s_err)) { ok = false; *s_err = 1; }
                    const uint8_t* st = smem + a.off_stage + (size_t)s * kSlotBytes;
                    const uint8_t* row0 = st + (warp * 16 + gq) * rs + t * kBlockBytes;
                    const uint8_t* row1 = row0 + 8 * rs;
#pragma unroll 1
                    for (uint32_t gi = 0; gi < ngr; ++gi) {
                        const uint32_t blk_abs = (gs + gi) * kGemvGranuleBlocks + t;     // this thread's block of the row
                        const uint32_t blk = blk_abs >= xr.base_blk ? blk_abs - xr.base_blk : blk_abs + q.kb - xr.base_blk;
                        const uint32_t* q0 = reinterpret_cast<const uint32_t*>(row0 + gi * (4 * kBlockBytes));
                        const uint32_t* q1 = reinterpret_cast<const uint32_t*>(row1 + gi * (4 * kBlockBytes));
                        const uint32_t meta0 = q0[0], meta1 = q1[0];
                        uint32_t w0[4], w1[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) { w0[j] = q0[1 + j]; w1[j] = q1[1 + j]; }
                        const uint8_t* xb = has_b ? xs_lane + (size_t)blk * 64 : zeros;
                        const uint4 bq0 = *reinterpret_cast<const uint4*>(xb);
                        const uint4 bq1 = *reinterpret_cast<const uint4*>(xb + 16);
                        const float2 info = sx_all[blk];
                        int c[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t av[4];
                            av[0] = w0[j] & 0x0F0F0F0Fu;
                            av[1] = w1[j] & 0x0F0F0F0Fu;
                            av[2] = (w0[j] >> 4) & 0x0F0F0F0Fu;
                            av[3] = (w1[j] >> 4) & 0x0F0F0F0Fu;
                            const uint4 bq = (j >> 1) ? bq1 : bq0;
                            imma_16832(c, av, (j & 1) ? bq.z : bq.x, (j & 1) ? bq.w : bq.y);
                        }
                        const float d0 = h2f_bits(meta0 & 0xffffu), bb0 = h2f_bits(meta0 >> 16);
                        const float d1 = h2f_bits(meta1 & 0xffffu), bb1 = h2f_bits(meta1 >> 16);
                        const float dot0 = fmaf((float)c[1], 1.0f / kLimb1Ratio, (float)c[0]);
                        const float dot1 = fmaf((float)c[3], 1.0f / kLimb1Ratio, (float)c[2]);
                        acc0 = fmaf(d0 * info.x, dot0, fmaf(bb0, info.y, acc0));
                        acc1 = fmaf(d1 * info.x, dot1, fmaf(bb1, info.y, acc1));
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]);
                    gs += ngr;
                    if (tid == 0 && git == 0) TL_STAMP(g, 6);
                }
                if (tid == 0) TL_STAMP(g, 2);
                if (pos >= sh.r1) {
                    // the share's last stage is consumed: the limb buffer may be refilled for a later group while
                    // this tile is finished (the fix-up waits for the other CTAs' partial sums)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&xfree[xb_i]);
                }

                // each thread of a quad covered blocks = t (mod 4): add the four
                float v0 = acc0, v1 = acc1;
                v0 += __shfl_xor_sync(kFull, v0, 1);
                v0 += __shfl_xor_sync(kFull, v0, 2);
                v1 += __shfl_xor_sync(kFull, v1, 1);
                v1 += __shfl_xor_sync(kFull, v1, 2);
                const bool complete = (g0 == 0 && g1 == q.kg);
                const uint32_t rowa = tile * kGemvTileRows + warp * 16 + gq, rowb = rowa + 8;
                const float* bra = q.lb + (size_t)(rowa < q.n ? rowa : 0) * q.rank;
                const float* brb = q.lb + (size_t)(rowb < q.n ? rowb : 0) * q.rank;
                float ba0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, bb0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (q.rank && (complete || g0 == 0)) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t j = t + 4 * u;
                        if (j < q.rank) { ba0[u] = __ldg(bra + j); bb0[u] = __ldg(brb + j); }
                    }
                }
                uint2* part = reinterpret_cast<uint2*>(a.partials) + (size_t)g * gridDim.x * kGemvTileRows;
                if (!complete && g0 != 0) {
                    // contributor: publish the partial sums as tagged messages and go on
                    uint2* dst = part + (size_t)blockIdx.x * kGemvTileRows + warp * 16;
                    if (t == 0) {
                        msg_store(dst + gq, v0, tag);
                        msg_store(dst + gq + 8, v1, tag);
                    }
                    continue;
                }
                if (!complete) {
                    // finisher: add the contributors' messages in CTA order (warp-uniform loop, bounded)
                    // the tile's last CTA: walk on from this CTA (the next one or two, as a rule)
                    const uint32_t c_last = MB ? tile_last_cta_inline(q, tile) : tile_last_cta_call(q, tile);
                    constexpr int CB = 4;
                    bool good = true;
                    for (uint32_t c0 = blockIdx.x + 1; c0 <= c_last && good; c0 += CB) {
                        uint2 msg[CB][2];
                        const long long t0 = wait_clock();
                        for (;;) {
                            bool all = true;
#pragma unroll
                            for (int cb = 0; cb < CB; ++cb) {
                                if (c0 + cb > c_last) continue;
                                const uint2* src = part + (size_t)(c0 + cb) * kGemvTileRows + warp * 16;
                                msg[cb][0] = msg_load(src + gq);
                                msg[cb][1] = msg_load(src + gq + 8);
                            }
#pragma unroll
                            for (int cb = 0; cb < CB; ++cb) {
                                if (c0 + cb > c_last) continue;
                                all = all && msg[cb][0].y == tag && msg[cb][1].y == tag;
                            }
                            if (__all_sync(kFull, all)) break;
                            if (__any_sync(kFull, *s_err != 0 || wait_expired(t0))) { good = false; break; }
                        }
#pragma unroll
                        for (int cb = 0; cb < CB; ++cb) {
                            if (c0 + cb > c_last) continue;
                            v0 += __uint_as_float(msg[cb][0].x);
                            v1 += __uint_as_float(msg[cb][1].x);
                        }
                    }
                    if (!good) {
                        if (lane == 0) atomicOr(a.status, kDevErrGridWaitTimeout);
                        *s_err = 1;
                    }
                }

                // epilogue: LoRA term (the quad splits the rank), then quad thread 0 stores
                if (q.rank) {
                    if (!t_loaded) {
                        if (helper_t) {
                            if (!mbar_wait_step(&tready[xb_i], xb_use & 1u, s_err)) { ok = false; *s_err = 1; }
                            t_loaded = true;
                        } else {
                            gather_t();      // mailbox-fed: the projection starts late, fetch it where it is needed
                        }
                    }
                    float la = 0.0f, lb2 = 0.0f;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t j = t + 4 * u;
                        const float tv = j < q.rank ? t_sm[j] : 0.0f;
                        la = fmaf(ba0[u], tv, la);
                        lb2 = fmaf(bb0[u], tv, lb2);
                    }
#pragma unroll 4
                    for (uint32_t j = t + 16; j < q.rank; j += 4) {
                        const float tv = t_sm[j];
                        la = fmaf(__ldg(bra + j), tv, la);
                        lb2 = fmaf(__ldg(brb + j), tv, lb2);
                    }
                    la += __shfl_xor_sync(kFull, la, 1);
                    la += __shfl_xor_sync(kFull, la, 2);
                    lb2 += __shfl_xor_sync(kFull, lb2, 1);
                    lb2 += __shfl_xor_sync(kFull, lb2, 2);
                    v0 += q.lscale * la;
                    v1 += q.lscale * lb2;
                }
                // Results: plain f32 for whoever reads after the launch, a tagged mailbox entry on every rank for the
                // later groups of this launch (and for the final gather).
                auto publish = [&](uint32_t row, float val) {
                    q.y[row] = val;
                    if (q.y_slot != kNoSlot) {
                        const unsigned long long e = mbox_pack(val, stag);
                        char* own = reinterpret_cast<char*>(mb + q.y_slot + row);
                        for (uint32_t r = 0; r < a.world; ++r) mbox_store(reinterpret_cast<unsigned long long*>(own + a.peer_mbox_off[r]), e);
                    }
                };
                if constexpr (!MB) {
                    // every lane of a quad holds both sums: lane 0 stores the first row, lane 1 the second, so one
                    // store instruction of the warp writes the warp's 16 consecutive rows (64 bytes of y, whole
                    // packets when y is host memory behind PCIe); 0.7 % of the step on the plain-input instantiation
                    const uint32_t row = t == 0 ? rowa : rowb;
                    if (t < 2 && row < q.n) publish(row, t == 0 ? v0 : v1);
                } else if (t == 0) {
                    if (rowa < q.n) publish(rowa, v0);
                    if (rowb < q.n) publish(rowb, v1);
                }
                if (tid == 0) TL_STAMP(g, 3);
            }
            // the projection buffer may be refilled for a later group
            __syncwarp();
            if (lane == 0) mbar_arrive(&tfree[xb_i]);
        }
        if (!ok) {
            if (lane == 0) atomicOr(a.status, kDevErrBarrierTimeout);
            *s_err = 1;
        }
        // Gather: every entry of the listed ranges, whoever wrote it, becomes plain f32 in this GPU's payload.
        // A thread polls its own entries (no shuffles follow, so the warp may split); bounded.
        for (uint32_t u = 0; u < a.n_ranges; ++u) {
            const unsigned long long* src = mb + a.range_begin[u];
            float* dst = a.payload + a.range_begin[u];
            const uint32_t cnt = a.range_count[u];
            for (uint32_t i = blockIdx.x * kConsumerThreads + tid; i < cnt; i += gridDim.x * kConsumerThreads) {
                unsigned long long e = mbox_load(src + i);
                if ((uint32_t)(e >> 32) != stag) {
                    const long long t0 = wait_clock();
                    unsigned ns = 128;
                    for (;;) {
                        __nanosleep(ns);
                        ns = ns < 1024 ? ns * 2 : 1024;
                        e = mbox_load(src + i);
                        if ((uint32_t)(e >> 32) == stag) break;
                        if (*s_err != 0 || wait_expired(t0)) {
                            atomicOr(a.status, kDevErrGridWaitTimeout);
                            *s_err = 1;
                            break;
                        }
                    }
                }
                dst[i] = __uint_as_float((uint32_t)e);
            }
        }
    }

    __syncthreads();
    if (tid == 0) {
        launch_done(a.tsync, blockIdx.x, gridDim.x);
        if (a.step_counter != a.tsync) launch_done(a.step_counter, blockIdx.x, gridDim.x);
    }
    // After a failed wait some TMA loads may still be in flight towards this CTA's shared memory: wait
    // (bounded) for the stages that were issued before leaving.
    if (*s_err && warp == 8 && lane == 0) {
        const uint32_t first = issued > NST ? issued - NST : 0;
        for (uint32_t j = first; j < issued; ++j) mbar_wait(&full[j % NST], (j / NST) & 1u);
    }
}

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

}  // namespace

#ifdef LQ4_STEP_TIMELINE
extern "C" int lq4_debug_step_timeline(unsigned long long* host_out, size_t count) {
    return (int)cudaMemcpyFromSymbol(host_out, g_step_timeline, count * sizeof(unsigned long long));
}
#endif

size_t step_plan_smem(StepArgs& a, uint32_t cap_blocks, uint32_t max_rank, uint32_t max_items) {
    if (cap_blocks == 0) return 0;
    uint32_t off = 2 * kMaxStages * 8 + 128;      // ring barriers, the block of zeros, the limb-buffer barriers
    a.off_t = off;                                // two t buffers (one per limb buffer)
    a.t_stride = align_up(max_rank * 4, 128);
    off += 2 * a.t_stride;
    a.off_tstage = off;                           // the pieces of t = A x before they are added: rank x pieces floats
    off += align_up(max_items * 4, 128);
    a.off_cstage = off;                           // the same for the converter warps
    off += align_up(max_items * 4, 128);
    // one limb buffer: limbs (64 B per block), then {scale, sum} (8 B per block)
    a.xbuf_sx = align_up(cap_blocks * 64, 128);
    a.xbuf_stride = a.xbuf_sx + align_up(cap_blocks * 8, 128);
    a.off_xbuf = off;
    const uint32_t budget = (uint32_t)kMaxSmem - 1024;    // static shared memory and driver reserve
    // two limb buffers (conversion runs a group ahead of consumption) when that costs no ring stage
    auto stages_with = [&](uint32_t nbuf) -> uint32_t {
        const uint32_t o = off + nbuf * a.xbuf_stride;
        if (o + 2 * kSlotBytes > budget) return 0;
        const uint32_t n = (budget - o) / kSlotBytes;
        return n > 4 ? 4 : n;
    };
    const uint32_t st1 = stages_with(1), st2 = stages_with(2);
    if (st1 == 0) return 0;
    a.nxbuf = (st2 >= st1 || st2 >= 3) ? 2 : 1;
    a.nstages = a.nxbuf == 2 ? st2 : st1;
    a.off_stage = off + a.nxbuf * a.xbuf_stride;
    return (size_t)a.off_stage + (size_t)a.nstages * kSlotBytes;
}

template <bool MB>
static cudaError_t launch_step_t(const StepArgs& a, size_t smem, int grid, cudaStream_t s) {
    static DeviceOnce once;            // the shared-memory opt-in is per device and per instantiation
    cudaError_t e = opt_in_smem(reinterpret_cast<const void*>(decode_step_kernel<MB>), kMaxSmem - 1024, once);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kStepThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (a.use_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, decode_step_kernel<MB>, a);
}

cudaError_t launch_decode_step(const StepArgs& a, size_t smem, int grid, cudaStream_t s) {
    bool mailbox_inputs = false;
    for (uint32_t i = 0; i < a.group_begin[a.ngroups]; ++i) mailbox_inputs = mailbox_inputs || a.p[i].x_slot != kNoSlot;
    // LQ4_STEP_FORCE_MB: run the mailbox-fed instantiation on plain inputs too (to compare the two builds' stage loops)
    static const bool force_mb = getenv("LQ4_STEP_FORCE_MB") != nullptr;
    return (mailbox_inputs || force_mb) ? launch_step_t<true>(a, smem, grid, s) : launch_step_t<false>(a, smem, grid, s);
}

}  // namespace lq4
