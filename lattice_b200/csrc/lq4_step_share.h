// How the work units of one projection of a decode step are cut into the shares of its CTAs (lq4_step.cu).
// Plain C++ (no CUDA headers): the host plans with the same functions the kernel walks with.
#pragma once

#include <cstdint>

#ifdef __CUDACC__
#define LQ4_HD __host__ __device__
#else
#define LQ4_HD
#endif

namespace lq4 {

// First work unit (position = tile * kg + granule) of CTA c's share of a problem, c in [0, count]: CTA c works
// on [begin(c), begin(c + 1)).  The CTA that owns a tile's first granule also finishes the tile (fix-up of the
// other CTAs' partial sums, adapter term, stores: time in which it streams nothing), so the split is equal in
// units PLUS `charge` units per tile start: every tile is stretched by `charge` virtual units in front of its
// first granule, the stretched range is cut evenly, and the cuts are mapped back.
template <typename U>
LQ4_HD inline U step_share_begin_t(U c, U tiles, U kg, U charge, U count) {
    const U kv = kg + charge;
    const U v = c * (tiles * kv) / count;
    const U tile = v / kv, off = v - tile * kv;
    return tile * kg + (off > charge ? off - charge : 0);
}
// Last CTA of [first, count) whose share begins at or before `pos` (first's share is known to).
template <typename U>
LQ4_HD inline U step_share_last_t(U first, U pos, U tiles, U kg, U charge, U count) {
    U c = first;
    while (c + 1 < count && step_share_begin_t<U>(c + 1, tiles, kg, charge, count) <= pos) ++c;
    return c;
}
// True if every product in the two functions above fits 32 bits.  The kernel divides in 32 bits (a 64-bit
// division costs about a hundred instructions, and the CTA that finishes a tile looks up the tile's last CTA),
// and the host refuses a problem for which this is false: 28 million work units, more than 280 GB of payload.
LQ4_HD inline bool step_share_fits32(uint32_t tiles, uint32_t kg, uint32_t charge, uint32_t count) {
    const uint64_t kv = (uint64_t)kg + charge;
    return (uint64_t)tiles * kv * ((uint64_t)count + 1) < (1ull << 32);
}

LQ4_HD inline uint64_t step_share_begin(uint64_t c, uint32_t tiles, uint32_t kg, uint32_t charge, uint32_t count) {
    return step_share_begin_t<uint64_t>(c, tiles, kg, charge, count);
}
// CTA whose share contains position `pos`.
LQ4_HD inline uint32_t step_share_owner(uint64_t pos, uint32_t tiles, uint32_t kg, uint32_t charge, uint32_t count) {
    const uint64_t kv = (uint64_t)kg + charge;
    const uint64_t tile = pos / kg, v = tile * kv + charge + (pos - tile * kg);
    uint64_t c = v * count / ((uint64_t)tiles * kv);
    if (c >= count) c = count - 1;
    while (c + 1 < count && step_share_begin(c + 1, tiles, kg, charge, count) <= pos) ++c;
    while (c > 0 && step_share_begin(c, tiles, kg, charge, count) > pos) --c;
    return (uint32_t)c;
}

}  // namespace lq4
