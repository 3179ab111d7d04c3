// Vertical/slash index conversion, one warp per 64-row query block.
//
// Replaces convert_vertical_slash_indexes_kernel (csrc/vertical_slash_index.cu:27-99 of the
// reference), which walks the two sorted lists with one thread per row block.  The
// sequential merge there has a closed form that a warp can evaluate 32 entries at a time:
//
//   * Slash offset o maps to the end token e = max(end_m - o, 64) of a 64-wide tile; with
//     offsets sorted descending, e is non-decreasing.
//   * While a range that started at e0 keeps growing, its end after seeing e is
//     e0 + 64*ceil((e - e0)/64) (the reference grows it by exactly 64 whenever e passes the
//     current end).  A new range starts at entry j iff e_j > end(e_{j-1}) + 64.
//   * Hence only entries with e_j - e_{j-1} > 64 can start a range; a ballot finds them and
//     the warp resolves them in order, everything else needs no work.
//   * A vertical column is gathered iff it lies below the start of the last range and in
//     none of the ranges; since both lists are sorted this is a forward scan, done 32
//     columns per step with ballots.
//
// Two kernels share that walk:
//   vs_convert_kernel -- the reference's dense tables (block_count/block_offset/column_count/
//           column_index), bit-exact including zero tails; one warp per row block scans the list.
//   vs_plan_kernel -- merged [start,end) ranges + a bit mask over the vertical list
//           (plan_layout.h).  The gaps of the slash list do not depend on the row block, so a
//           CTA compacts the positions whose gap exceeds 64 once and each of its 32 row blocks
//           walks only those, writing its ranges; the bit mask is then built in shared memory in
//           one sweep over the written ranges, 32 ranges and 32 columns at a time.
#include <climits>

#include "common.h"
#include "plan_layout.h"

namespace minf {

constexpr int kConvertWarps = 8;
constexpr int kPlanRowsPerWarp = 4;    // a plan CTA covers 32 row blocks of one head

struct ConvertArgs {
    const int32_t* seqlens;
    const int32_t* v_idx;
    const int32_t* s_idx;
    const int32_t* nnz_v_per_head;
    const int32_t* nnz_s_per_head;
    int heads, rows, cap_v, cap_s;
    int rb_base;                      // first row block covered (0 for a whole sequence)
    // reference-format outputs
    int32_t* block_count;
    int32_t* block_offset;
    int32_t* column_count;
    int32_t* column_index;
    // plan output
    unsigned char* plan;
    PlanLayout layout;
    int32_t* status;
};

// first slash entry below end_m (list is descending): lower bound, uniform across lanes
__device__ __forceinline__ int first_slash_below(const int32_t* s_list, int nnz_s, int end_m) {
    int lo = 0, hi = nnz_s;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_list[mid] >= end_m) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(kConvertWarps * 32) vs_convert_kernel(const ConvertArgs a) {
    extern __shared__ int32_t lists[];
    int32_t* s_list = lists;
    int32_t* v_list = lists + a.cap_s;

    const int b = blockIdx.z, h = blockIdx.y;
    const int bh = b * a.heads + h;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nnz_s = a.cap_s, nnz_v = a.cap_v;

    for (int i = threadIdx.x; i < nnz_s; i += blockDim.x) s_list[i] = a.s_idx[(size_t)bh * a.cap_s + i];
    for (int i = threadIdx.x; i < nnz_v; i += blockDim.x) v_list[i] = a.v_idx[(size_t)bh * a.cap_v + i];
    __syncthreads();

    const int m = blockIdx.x * kConvertWarps + warp;          // row block
    if (m >= a.rows) return;
    const int seqlen = a.seqlens[b];
    const int start_m = m * 64, end_m = start_m + 64;
    const size_t row = (size_t)bh * a.rows + m;
    int32_t* bo = a.block_offset + row * a.cap_s;
    int32_t* ci = a.column_index + row * a.cap_v;

    int nblk = 0, ncol = 0, vp = 0;
    int i0 = nnz_s;
    if (start_m < seqlen) {
        i0 = first_slash_below(s_list, nnz_s, end_m);
        if (i0 == nnz_s && lane == 0) atomicAdd(a.status + MINF_ST_NO_SLASH, 1);
    }

    if (i0 < nnz_s) {
        // close range [rs, re): emit its tiles, then advance through the verticals
        auto close_range = [&](int rs, int re) {
            for (int t = rs + 64 * lane; t < re; t += 64 * 32)
                if (MINF_IN_BOUNDS(a.status, nblk + ((t - rs) >> 6) < a.cap_s)) bo[nblk + ((t - rs) >> 6)] = t;
            nblk += (re - rs) >> 6;
            for (;;) {
                const int i = vp + lane;
                const int val = i < nnz_v ? v_list[i] : INT_MAX;
                const int n_below = __popc(__ballot_sync(0xffffffffu, val < rs));
                if (lane < n_below && MINF_IN_BOUNDS(a.status, ncol + lane < a.cap_v)) ci[ncol + lane] = val;
                ncol += n_below;
                const int n_inside = __popc(__ballot_sync(0xffffffffu, val < re));
                vp += n_inside;
                if (n_inside < 32) break;
            }
        };

        int e_first = max(end_m - s_list[i0], 64);
        int carry = e_first;
        for (int base = i0; base < nnz_s; base += 32) {
            const int i = base + lane;
            const bool valid = i < nnz_s;
            const int e = valid ? max(end_m - s_list[i], 64) : INT_MAX;
            int prev = __shfl_up_sync(0xffffffffu, e, 1);
            if (lane == 0) prev = carry;
            unsigned cand = __ballot_sync(0xffffffffu, valid && (e - prev > 64));
            while (cand) {
                const int j = __ffs(cand) - 1;
                cand &= cand - 1;
                const int ej = __shfl_sync(0xffffffffu, e, j);
                const int pj = __shfl_sync(0xffffffffu, prev, j);
                const int re = e_first + ((pj - e_first + 63) & ~63);
                if (ej > re + 64) {
                    close_range(e_first - 64, re);
                    e_first = ej;
                }
            }
            const int last = min(31, nnz_s - 1 - base);
            carry = __shfl_sync(0xffffffffu, e, last);
        }
        close_range(e_first - 64, e_first + ((carry - e_first + 63) & ~63));
    }

    if (lane == 0) {
        a.block_count[row] = nblk;
        a.column_count[row] = ncol;
    }
    for (int j = nblk + lane; j < a.cap_s; j += 32) bo[j] = 0;
    for (int j = ncol + lane; j < a.cap_v; j += 32) ci[j] = 0;
}

__global__ void __launch_bounds__(kConvertWarps * 32) vs_plan_kernel(const ConvertArgs a) {
    extern __shared__ int32_t lists[];
    int32_t* s_list = lists;
    int32_t* v_list = lists + a.cap_s;
    int32_t* cand = v_list + a.cap_v;                      // positions j with s[j-1] - s[j] > 64, ascending
    uint32_t* wbits = reinterpret_cast<uint32_t*>(cand + a.cap_s);   // [warp][words_v]
    __shared__ int warp_count[kConvertWarps];
    __shared__ int sh_ncand;

    const int b = blockIdx.z, h = blockIdx.y;
    const int bh = b * a.heads + h;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (a.nnz_s_per_head && a.nnz_s_per_head[bh] < 0) return;   // head owned by another pattern
    const int nnz_s = a.nnz_s_per_head ? min(a.nnz_s_per_head[bh], a.cap_s) : a.cap_s;
    const int nnz_v = a.nnz_v_per_head ? min(max(a.nnz_v_per_head[bh], 0), a.cap_v) : a.cap_v;
    const int words_v = a.layout.words_v;

    for (int i = threadIdx.x; i < nnz_s; i += blockDim.x) s_list[i] = a.s_idx[(size_t)bh * a.cap_s + i];
    for (int i = threadIdx.x; i < nnz_v; i += blockDim.x) v_list[i] = a.v_idx[(size_t)bh * a.cap_v + i];
    if (threadIdx.x == 0) sh_ncand = 0;
    __syncthreads();
    // ordered compaction of the gap positions, one block-wide round per 256 entries
    for (int base = 1; base < nnz_s; base += kConvertWarps * 32) {
        const int j = base + threadIdx.x;
        const bool is_gap = j < nnz_s && s_list[j - 1] - s_list[j] > 64;
        const unsigned bal = __ballot_sync(0xffffffffu, is_gap);
        if (lane == 0) warp_count[warp] = __popc(bal);
        __syncthreads();
        int dst = sh_ncand + __popc(bal & ((1u << lane) - 1u));
        int total = 0;
#pragma unroll
        for (int w = 0; w < kConvertWarps; ++w) {
            if (w < warp) dst += warp_count[w];
            total += warp_count[w];
        }
        if (is_gap) cand[dst] = j;
        __syncthreads();
        if (threadIdx.x == 0) sh_ncand += total;
    }
    __syncthreads();
    const int n_cand = sh_ncand;
    uint32_t* wb = wbits + warp * words_v;
    unsigned char* slot = a.plan + (size_t)bh * a.layout.head_bytes;

    for (int rr = 0; rr < kPlanRowsPerWarp; ++rr) {
        const int m = (blockIdx.x * kPlanRowsPerWarp + rr) * kConvertWarps + warp;    // row block inside the output
        if (m >= a.rows) break;
        const int seqlen = a.seqlens[b];
        const int start_m = (a.rb_base + m) * 64, end_m = start_m + 64;   // its rows in the sequence
        int2* rng = reinterpret_cast<int2*>(slot + a.layout.rng_off) + plan_rng_offset(a.layout, m);
        for (int w = lane; w < words_v; w += 32) wb[w] = 0u;
        __syncwarp();

        int nrng = 0, vp = 0;
        int i0 = nnz_s;
        if (start_m < seqlen) {
            i0 = first_slash_below(s_list, nnz_s, end_m);
            if (i0 == nnz_s && lane == 0) atomicAdd(a.status + MINF_ST_NO_SLASH, 1);
        }
        if (i0 < nnz_s) {
            // The ranges depend on the slash list only: they are written first, and the columns are marked afterwards
            // in one sweep over the written ranges, 32 at a time (see below).  (Marking while walking -- a scan of the
            // vertical list per range -- and two binary searches per range were both measured: slower.)
            auto close_range = [&](int rs, int re) {
                // row block m of the sequence holds at most min(cap_s, m + 2) ranges (plan_layout.h)
                if (lane == 0 && MINF_IN_BOUNDS(a.status, nrng < min(a.cap_s, a.rb_base + m + 2) && rs >= 0 && re > rs))
                    rng[nrng] = make_int2(rs, re);
                ++nrng;
            };
            // first gap position after i0
            int lo = 0, hi = n_cand;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (cand[mid] <= i0) lo = mid + 1; else hi = mid;
            }
            int e_first = max(end_m - s_list[i0], 64);
            for (int base = lo; base < n_cand; base += 32) {
                const bool valid = base + lane < n_cand;
                const int j = valid ? cand[base + lane] : 1;
                const int e = max(end_m - s_list[j], 64), prev = max(end_m - s_list[j - 1], 64);
                // Under a given range start every lane can test its own entry; the first lane whose entry opens a
                // new range is the next start, and only the lanes after it are tested again: one ballot per range
                // instead of one shuffle pair per candidate.
                unsigned todo = __ballot_sync(0xffffffffu, valid && (e - prev > 64));
                // Scattered lists: every candidate of the batch opens a range of its own.  Lane l then knows the
                // range it closes without waiting for the others -- it starts at the previous candidate's tile --
                // so the whole batch is written with one store per lane.
                const unsigned all_valid = __ballot_sync(0xffffffffu, valid);    // lanes 0..cnt-1
                const int cnt = __popc(all_valid);
                if (todo == all_valid && cnt > 1) {
                    int ef = __shfl_up_sync(0xffffffffu, e, 1);
                    if (lane == 0) ef = e_first;
                    const int re_l = ef + ((prev - ef + 63) & ~63);
                    if (__ballot_sync(0xffffffffu, valid && e > re_l + 64) == all_valid) {
                        const int rs_l = ef - 64;
                        if (valid && MINF_IN_BOUNDS(a.status, nrng + lane < min(a.cap_s, a.rb_base + m + 2) && rs_l >= 0 && re_l > rs_l))
                            rng[nrng + lane] = make_int2(rs_l, re_l);
                        nrng += cnt;
                        e_first = __shfl_sync(0xffffffffu, e, cnt - 1);
                        todo = 0u;
                    }
                }
                while (todo) {
                    const int re_mine = e_first + ((prev - e_first + 63) & ~63);
                    const unsigned opens = __ballot_sync(0xffffffffu, ((todo >> lane) & 1u) && e > re_mine + 64);
                    if (opens == 0u) break;
                    const int l = __ffs(opens) - 1;
                    const int pj = __shfl_sync(0xffffffffu, prev, l);
                    close_range(e_first - 64, e_first + ((pj - e_first + 63) & ~63));
                    e_first = __shfl_sync(0xffffffffu, e, l);
                    todo &= ~((2u << l) - 1u);          // entries up to and including l are settled
                }
            }
            const int e_last = max(end_m - s_list[nnz_s - 1], 64);
            close_range(e_first - 64, e_first + ((e_last - e_first + 63) & ~63));
            // Columns: a vertical index is gathered iff it lies below the end of the last range and in none of the
            // ranges.  Both lists ascend, so the ranges are taken 32 at a time (one per lane) and the verticals up to
            // the end of the group 32 at a time: each finds the range that starts at or below it by a binary search
            // over the lanes.
            __syncwarp();                     // the ranges written above are read back here
            const int n_read = min(nrng, min(a.cap_s, a.rb_base + m + 2));
            if (n_read <= 8) {
                // few ranges (dense index sets): two warp-uniform binary searches per range, then every lane fills
                // one word of the bit mask
                int settled = 0;                    // vertical entries below it are done
                for (int g = 0; g < n_read; ++g) {
                    const int2 rg = rng[g];
                    int lo = settled, hi = nnz_v;
                    while (lo < hi) { const int mid = (lo + hi) >> 1; if (v_list[mid] < rg.x) lo = mid + 1; else hi = mid; }
                    const int below = lo;           // entries [settled, below) lie under the range: gathered
                    hi = nnz_v;
                    while (lo < hi) { const int mid = (lo + hi) >> 1; if (v_list[mid] < rg.y) lo = mid + 1; else hi = mid; }
                    if (settled < below) {
                        for (int w = (settled >> 5) + lane; w <= ((below - 1) >> 5); w += 32) {
                            if (!MINF_IN_BOUNDS(a.status, w < words_v)) break;
                            const int l = max(settled - 32 * w, 0), h = min(below - 32 * w, 32);
                            wb[w] |= (h == 32 ? 0xffffffffu : ((1u << h) - 1u)) & ~((1u << l) - 1u);
                        }
                    }
                    __syncwarp();
                    settled = lo;                   // entries inside the range are skipped
                }
                vp = settled;
            }
            for (int g = 0; n_read > 8 && g < n_read; g += 32) {
                const int cnt = min(32, n_read - g);
                const int2 mine = lane < cnt ? rng[g + lane] : make_int2(INT_MAX, INT_MAX);
                const int re_last = __shfl_sync(0xffffffffu, mine.y, cnt - 1);
                for (;;) {
                    const int i = vp + lane;
                    const int val = i < nnz_v ? v_list[i] : INT_MAX;
                    const bool in_group = val < re_last;
                    int blo = 0, bhi = cnt;         // number of ranges of the group starting at or below val
#pragma unroll
                    for (int it = 0; it < 6; ++it) {
                        const int mid = (blo + bhi) >> 1;
                        const int rs_mid = __shfl_sync(0xffffffffu, mine.x, mid & 31);
                        if (blo < bhi) { if (rs_mid <= val) blo = mid + 1; else bhi = mid; }
                    }
                    const int re_before = __shfl_sync(0xffffffffu, mine.y, max(blo - 1, 0));
                    const bool covered = blo > 0 && val < re_before;
                    const unsigned marks = __ballot_sync(0xffffffffu, in_group && !covered);
                    const int n_in = __popc(__ballot_sync(0xffffffffu, in_group));
                    if (marks && lane == 0) {
                        const int w0 = vp >> 5, sh = vp & 31;
                        if (MINF_IN_BOUNDS(a.status, w0 < words_v)) wb[w0] |= marks << sh;
                        if (sh && (marks >> (32 - sh)) && MINF_IN_BOUNDS(a.status, w0 + 1 < words_v)) wb[w0 + 1] |= marks >> (32 - sh);
                    }
                    vp += n_in;
                    if (n_in < 32) break;
                }
            }
        }
        __syncwarp();
        if (lane == 0) reinterpret_cast<int32_t*>(slot)[m] = nrng;
        uint32_t* out = reinterpret_cast<uint32_t*>(slot + a.layout.bits_off) + (size_t)m * words_v;
        for (int w = lane; w < words_v; w += 32) out[w] = wb[w];
        __syncwarp();
    }
}

__global__ void plan_count_tiles_kernel(const unsigned char* plan, PlanLayout L, int total_rows,
                                        unsigned long long* out) {
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long tiles = 0;
    if (gid < total_rows) {
        const int bh = (int)(gid / L.rows), m = (int)(gid % L.rows);
        const unsigned char* slot = plan + (size_t)bh * L.head_bytes;
        const int n = reinterpret_cast<const int32_t*>(slot)[m];
        const int2* rng = reinterpret_cast<const int2*>(slot + L.rng_off) + plan_rng_offset(L, m);
        for (int i = 0; i < n; ++i) tiles += (rng[i].y - rng[i].x) >> 6;
        const uint32_t* wb = reinterpret_cast<const uint32_t*>(slot + L.bits_off) + (size_t)m * L.words_v;
        int cols = 0;
        for (int w = 0; w < L.words_v; ++w) cols += __popc(wb[w]);
        tiles += (cols + 63) >> 6;
    }
    // warp reduce then one atomic per warp
    for (int o = 16; o; o >>= 1) tiles += __shfl_down_sync(0xffffffffu, tiles, o);
    if ((threadIdx.x & 31) == 0 && tiles) atomicAdd(out, tiles);
}

static int launch_convert(const ConvertArgs& a, int batch, cudaStream_t st) {
    const size_t smem = (size_t)(a.cap_s + a.cap_v) * sizeof(int32_t);
    if (smem > 200 * 1024) return fail(MINF_E_UNSUPPORTED, "index lists too long for shared memory (%zu bytes)", smem);
    dim3 grid((a.rows + kConvertWarps - 1) / kConvertWarps, a.heads, batch);
    MINF_CUDA_OK(cudaFuncSetAttribute(vs_convert_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    vs_convert_kernel<<<grid, kConvertWarps * 32, smem, st>>>(a);
    MINF_LAUNCH_OK("vs_convert_kernel");
    return MINF_OK;
}

static int launch_plan(const ConvertArgs& a, int batch, cudaStream_t st) {
    const size_t smem = ((size_t)2 * a.cap_s + a.cap_v + (size_t)kConvertWarps * a.layout.words_v) * sizeof(int32_t);
    if (smem > 200 * 1024) return fail(MINF_E_UNSUPPORTED, "index lists too long for shared memory (%zu bytes)", smem);
    const int per_cta = kConvertWarps * kPlanRowsPerWarp;
    dim3 grid((a.rows + per_cta - 1) / per_cta, a.heads, batch);
    MINF_CUDA_OK(cudaFuncSetAttribute(vs_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    vs_plan_kernel<<<grid, kConvertWarps * 32, smem, st>>>(a);
    MINF_LAUNCH_OK("vs_plan_kernel");
    return MINF_OK;
}

}  // namespace minf

using namespace minf;

extern "C" int minf_convert_vertical_slash_indexes(
    const int32_t* seqlens, const int32_t* vertical_indexes, const int32_t* slash_indexes,
    int batch, int heads, int context_size, int nnz_v, int nnz_s,
    int32_t* block_count, int32_t* block_offset, int32_t* column_count, int32_t* column_index,
    int32_t* status, void* stream) {
    if (!seqlens || !vertical_indexes || !slash_indexes || !block_count || !block_offset || !column_count ||
        !column_index || !status)
        return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || heads < 1 || context_size < 1 || nnz_v < 1 || nnz_s < 1 || heads > 65535 || batch > 65535)
        return fail(MINF_E_ARG, "bad sizes: batch=%d heads=%d context=%d nnz_v=%d nnz_s=%d", batch, heads,
                    context_size, nnz_v, nnz_s);
    ConvertArgs a{};
    a.seqlens = seqlens; a.v_idx = vertical_indexes; a.s_idx = slash_indexes;
    a.heads = heads; a.rows = (context_size + 63) / 64; a.cap_v = nnz_v; a.cap_s = nnz_s;
    a.block_count = block_count; a.block_offset = block_offset;
    a.column_count = column_count; a.column_index = column_index;
    a.status = status;
    return launch_convert(a, batch, static_cast<cudaStream_t>(stream));
}

extern "C" size_t minf_plan_bytes(int batch, int heads, int context_size, int cap_v, int cap_s) {
    if (batch < 1 || heads < 1 || context_size < 1 || cap_v < 0 || cap_s < 1) return 0;
    return (size_t)make_plan_layout(context_size, cap_v, cap_s).head_bytes * batch * heads;
}

extern "C" size_t minf_plan_bytes_window(int batch, int heads, int q_pos0, int n_q, int cap_v, int cap_s) {
    if (batch < 1 || heads < 1 || q_pos0 < 0 || (q_pos0 % 64) || n_q < 1 || cap_v < 0 || cap_s < 1) return 0;
    return (size_t)make_plan_layout_window(q_pos0 / 64, (n_q + 63) / 64, cap_v, cap_s).head_bytes * batch * heads;
}

extern "C" int minf_vs_build_plan_window(
    const int32_t* seqlens, const int32_t* vertical_indexes, const int32_t* slash_indexes,
    const int32_t* nnz_v_per_head, const int32_t* nnz_s_per_head,
    int batch, int heads, int q_pos0, int n_q, int cap_v, int cap_s,
    void* plan, int32_t* status, void* stream) {
    if (!seqlens || !vertical_indexes || !slash_indexes || !plan || !status)
        return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || heads < 1 || n_q < 1 || q_pos0 < 0 || (q_pos0 % 64) || cap_v < 1 || cap_s < 1 || heads > 65535 || batch > 65535)
        return fail(MINF_E_ARG, "bad sizes: batch=%d heads=%d q_pos0=%d n_q=%d cap_v=%d cap_s=%d", batch, heads,
                    q_pos0, n_q, cap_v, cap_s);
    ConvertArgs a{};
    a.seqlens = seqlens; a.v_idx = vertical_indexes; a.s_idx = slash_indexes;
    a.nnz_v_per_head = nnz_v_per_head; a.nnz_s_per_head = nnz_s_per_head;
    a.heads = heads; a.rows = (n_q + 63) / 64; a.cap_v = cap_v; a.cap_s = cap_s;
    a.rb_base = q_pos0 / 64;
    a.plan = static_cast<unsigned char*>(plan);
    a.layout = make_plan_layout_window(a.rb_base, a.rows, cap_v, cap_s);
    a.status = status;
    return launch_plan(a, batch, static_cast<cudaStream_t>(stream));
}

extern "C" int minf_vs_build_plan(
    const int32_t* seqlens, const int32_t* vertical_indexes, const int32_t* slash_indexes,
    const int32_t* nnz_v_per_head, const int32_t* nnz_s_per_head,
    int batch, int heads, int context_size, int cap_v, int cap_s,
    void* plan, int32_t* status, void* stream) {
    return minf_vs_build_plan_window(seqlens, vertical_indexes, slash_indexes, nnz_v_per_head, nnz_s_per_head,
                                     batch, heads, 0, context_size, cap_v, cap_s, plan, status, stream);
}

extern "C" int minf_plan_count_tiles_window(const void* plan, int batch, int heads, int q_pos0, int n_q,
                                            int cap_v, int cap_s, unsigned long long* tiles_out, void* stream);

extern "C" int minf_plan_count_tiles(const void* plan, int batch, int heads, int context_size,
                                     int cap_v, int cap_s, unsigned long long* tiles_out, void* stream) {
    return minf_plan_count_tiles_window(plan, batch, heads, 0, context_size, cap_v, cap_s, tiles_out, stream);
}

extern "C" int minf_plan_count_tiles_window(const void* plan, int batch, int heads, int q_pos0, int n_q,
                                            int cap_v, int cap_s, unsigned long long* tiles_out, void* stream) {
    if (!plan || !tiles_out) return fail(MINF_E_ARG, "null pointer argument");
    if (q_pos0 < 0 || (q_pos0 % 64) || n_q < 1) return fail(MINF_E_ARG, "bad query window");
    PlanLayout L = make_plan_layout_window(q_pos0 / 64, (n_q + 63) / 64, cap_v, cap_s);
    const long long total = (long long)L.rows * batch * heads;
    if (total > INT_MAX) return fail(MINF_E_UNSUPPORTED, "too many row blocks");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    MINF_CUDA_OK(cudaMemsetAsync(tiles_out, 0, sizeof(unsigned long long), st));
    plan_count_tiles_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        static_cast<const unsigned char*>(plan), L, (int)total, tiles_out);
    MINF_LAUNCH_OK("plan_count_tiles_kernel");
    return MINF_OK;
}
