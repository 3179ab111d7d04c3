// Layout of the compact attention plan in device memory (shared by host and device code).
//
// A plan covers `rows` consecutive 64-row query blocks starting at block `rb_base` of the
// sequence (rb_base = 0 and rows = ceil(N/64) for a whole sequence; a sequence-sharded caller
// builds one plan per local query chunk).  Per (batch*heads + head) slot, `head_bytes` apart:
//   int32  rng_cnt[rows]              number of merged [start,end) token ranges of row block m
//   uint32 col_bits[rows][words_v]    bit i of word w set <=> vertical_indexes[32*w+i] is a
//                                     gathered column of row block m
//   int2   rng[...]                   ranges of local row block ml start at plan_rng_offset(ml).
//                                     Row block m (global index) can hold min(cap_s, m+2)
//                                     ranges: its ranges are disjoint, at least 64 tokens long
//                                     and end at or before 64*(m+2), and every slash entry
//                                     starts at most one.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define MINF_HD __host__ __device__ __forceinline__
#else
#define MINF_HD inline
#endif

namespace minf {

struct PlanLayout {
    int rb_base;
    int rows;
    int cap_s;
    int words_v;
    long long bits_off;    // bytes from slot start
    long long rng_off;     // bytes from slot start
    long long head_bytes;  // slot size
};

// sum over m' < m of min(cap_s, m' + 2)
MINF_HD long long plan_rng_index(int m, int cap_s) {
    long long k = m < cap_s - 1 ? m : (cap_s - 1 > 0 ? cap_s - 1 : 0);
    return k * (k - 1) / 2 + 2 * k + (static_cast<long long>(m) - k) * cap_s;
}

MINF_HD long long plan_rng_offset(const PlanLayout& L, int local_row_block) {
    return plan_rng_index(L.rb_base + local_row_block, L.cap_s) - plan_rng_index(L.rb_base, L.cap_s);
}

MINF_HD long long align_up(long long x, long long a) { return (x + a - 1) / a * a; }

MINF_HD PlanLayout make_plan_layout_window(int rb_base, int rows, int cap_v, int cap_s) {
    PlanLayout L;
    L.rb_base = rb_base;
    L.rows = rows;
    L.cap_s = cap_s < 1 ? 1 : cap_s;
    L.words_v = (cap_v + 31) / 32;
    L.bits_off = align_up(static_cast<long long>(L.rows) * 4, 16);
    L.rng_off = align_up(L.bits_off + static_cast<long long>(L.rows) * L.words_v * 4, 16);
    L.head_bytes = align_up(L.rng_off + plan_rng_offset(L, L.rows) * 8, 256);
    return L;
}

MINF_HD PlanLayout make_plan_layout(int context_size, int cap_v, int cap_s) {
    return make_plan_layout_window(0, (context_size + 63) / 64, cap_v, cap_s);
}

}  // namespace minf
