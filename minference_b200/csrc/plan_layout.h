// Layout of the compact attention plan in device memory (shared by host and device code).
//
// Per (batch*heads + head) slot, `head_bytes` apart:
//   int32  rng_cnt[rows]              number of merged [start,end) token ranges of row block m
//   uint32 col_bits[rows][words_v]    bit i of word w set <=> vertical_indexes[32*w+i] is a
//                                     gathered column of row block m
//   int2   rng[...]                   ranges of row block m start at rng_offset(m); row block
//                                     m can hold min(cap_s, m+2) ranges: its ranges are
//                                     disjoint, at least 64 tokens long and end at or before
//                                     64*(m+2), and every slash entry starts at most one.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define MINF_HD __host__ __device__ __forceinline__
#else
#define MINF_HD inline
#endif

namespace minf {

struct PlanLayout {
    int rows;
    int cap_s;
    int words_v;
    long long bits_off;    // bytes from slot start
    long long rng_off;     // bytes from slot start
    long long head_bytes;  // slot size
};

MINF_HD long long plan_rng_index(int m, int cap_s) {
    long long k = m < cap_s - 1 ? m : (cap_s - 1 > 0 ? cap_s - 1 : 0);
    return k * (k - 1) / 2 + 2 * k + (static_cast<long long>(m) - k) * cap_s;
}

MINF_HD long long align_up(long long x, long long a) { return (x + a - 1) / a * a; }

MINF_HD PlanLayout make_plan_layout(int context_size, int cap_v, int cap_s) {
    PlanLayout L;
    L.rows = (context_size + 63) / 64;
    L.cap_s = cap_s < 1 ? 1 : cap_s;
    L.words_v = (cap_v + 31) / 32;
    L.bits_off = align_up(static_cast<long long>(L.rows) * 4, 16);
    L.rng_off = align_up(L.bits_off + static_cast<long long>(L.rows) * L.words_v * 4, 16);
    L.head_bytes = align_up(L.rng_off + plan_rng_index(L.rows, L.cap_s) * 8, 256);
    return L;
}

}  // namespace minf
