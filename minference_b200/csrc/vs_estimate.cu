// Online vertical/slash index estimation for every head of a layer.
//
// Replaces the torch ops of vertical_and_slash_kernel (modules/minference_forward.py:599-614
// of the reference) and sum_all_diagonal_matrix (:110-116), which run once per head from a
// Python loop: a skinny GEMM, a [64, N] fp32 softmax, a zero-padded strided view for the
// diagonal sums and two full top-k sorts.
//
// Here: two passes of one tcgen05 kernel over K, a small combine step, then a radix select
// spread over many CTAs.
//   scores kernel   CTA = (block of 2048 keys, pair of query heads sharing a KV head, batch);
//                   128 keys per tile by TMA, 128x128 fp32 logits in TMEM (double buffered),
//                   eight softmax warps.  Logits are rounded to bf16 twice like the
//                   reference's bf16 einsum followed by the bf16 division by sqrt(d).
//     pass 1        S = Q_last K^T (TMEM lane = query row): running (max, sum exp) per row,
//                   written per block of 2048 keys.  Blocks sit on a fixed grid of the key
//                   positions and are combined in ascending order (vs_stats_combine_kernel),
//                   so the row statistics do not depend on how a caller shards the keys.
//     pass 2        S^T = K Q_last^T (TMEM lane = key): every thread owns one key of one head,
//                   so the vertical score is a sum in registers, and the diagonal sums travel
//                   along the warp as a systolic chain of shuffles (the value for i - j = const
//                   moves up one lane per query row).  A diagonal is 64 long: it touches at
//                   most two 128-key tiles, whose partial sums are added in a fixed order
//                   inside a CTA and with two commuting atomics across CTAs, so the scores
//                   are the same bits however the keys are split over CTAs, calls or ranks.
//   select kernels  three histogram levels (11 + 10 + 10 bits of the non-negative fp32 score)
//                   over 8192-element segments, the last CTA of a level picks the bin of the
//                   k-th largest; then per-segment counts and an ordered compaction.  +inf
//                   forcing of the first 30 keys / the 100 nearest diagonals as the reference.
//                   Output is already sorted the way the index conversion wants (vertical
//                   ascending, slash offsets descending).  Equal scores at the threshold:
//                   lowest key index first / smallest offset first (torch.topk leaves this
//                   unspecified).
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.h"
#include "sm100_ptx.cuh"

namespace minf {

constexpr int kEstTileN = 128;
constexpr int kEstBlockTiles = 16;                       // statistics block = 2048 keys
constexpr int kEstBlockKeys = kEstTileN * kEstBlockTiles;
constexpr int kEstThreads = 64 + 256;                    // producer warp, MMA warp, 8 softmax warps
constexpr uint32_t kEstQBytes = 128 * 256;
constexpr uint32_t kEstKBytes = 128 * 256;
constexpr uint32_t kEstAuxOff = kEstQBytes + 2 * kEstKBytes;         // 98304
constexpr int kDiagSlots = 96;                           // partial diagonal sums of one warp and head (95 used)
constexpr uint32_t kEstAuxBytes = 2 * 4 * 2 * kDiagSlots * 4;        // [buffer][warp quarter][head][slot] floats
constexpr uint32_t kEstCtlOff = kEstAuxOff + kEstAuxBytes;

struct EstControl {
    unsigned long long q_full;
    unsigned long long k_full[2], k_empty[2], s_full[2], s_empty[2];
    uint32_t tmem_base;
    int abort;
    float cst[2][64];                // pass 2: -(M*log2(e) + log2(L)) per head and query row
    float2 half_stat[128];           // pass 1: statistics of the second half of each row's columns
};

struct EstArgs {
    int batch, hq, hkv, n_ctx, last_q;
    int n_k, col_base;               // local keys and the position of the first one
    int group, pairs_per_group;      // hq / hkv, ceil(group / 2)
    int tiles;                       // 128-key tiles over the local keys
    int block_offset, blocks_total;  // where this call's statistics blocks sit among those of the sequence
    float2* stats;                   // pass 1 out: [batch*hq][64][blocks_total] (max, sum)
    const float2* row_stats;         // pass 2 in:  [batch*hq][64] (max, sum) over the whole sequence
    float* vertical;                 // [batch*hq][n_ctx]
    float* slash;                    // [batch*hq][n_ctx], indexed by diagonal offset
    float sqrt_d;                    // logits are divided by it
    float rcp_sqrt_d;                // its reciprocal, for the refined multiply that replaces the division
    int32_t* status;
};

// x / d correctly rounded from a reciprocal and one Newton step on the exact remainder (no MUFU,
// three FMA-pipe instructions instead of the division sequence).
__device__ __forceinline__ float div_refined(float x, float d, float rcp) {
    const float q = x * rcp;
    return fmaf(fmaf(-q, d, x), rcp, q);
}
// The reference's logits: the bf16 GEMM output divided by sqrt(d) in fp32 and rounded to bf16 again.
// MUL: one multiply by the reciprocal instead of the refined division.  For the two divisors the callers use,
// sqrt(128) and 1, the bf16 result is the same for every one of the 65536 bf16 inputs (checked exhaustively on
// the host: the quotient of an 8-bit significand never lies within an fp32 rounding error of a bf16 tie).
template <bool MUL>
__device__ __forceinline__ void logits_pair(uint32_t a0, uint32_t a1, float d, float rcp, float& v0, float& v1) {
    const uint32_t g = pack_bf16x2(__uint_as_float(a0), __uint_as_float(a1));
    const float x0 = __uint_as_float(g << 16), x1 = __uint_as_float(g & 0xffff0000u);
    const uint32_t r = MUL ? pack_bf16x2(x0 * rcp, x1 * rcp) : pack_bf16x2(div_refined(x0, d, rcp), div_refined(x1, d, rcp));
    v0 = __uint_as_float(r << 16);
    v1 = __uint_as_float(r & 0xffff0000u);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

constexpr float kLog2e = 1.4426950408889634f;

template <int PASS, bool MUL>
__global__ void __launch_bounds__(kEstThreads, 2)
vs_scores_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const EstArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    EstControl* ctl = reinterpret_cast<EstControl*>(smem + kEstCtlOff);
    float* part = reinterpret_cast<float*>(smem + kEstAuxOff);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int blk = blockIdx.x;                        // statistics block = chunk of 16 tiles
    const int pair = blockIdx.y;                       // over hkv * pairs_per_group
    const int b = blockIdx.z;
    const int hk = pair / a.pairs_per_group;
    const int h0 = hk * a.group + 2 * (pair % a.pairs_per_group);
    const bool has_h1 = (2 * (pair % a.pairs_per_group) + 1) < a.group;
    const int tile_lo = blk * kEstBlockTiles;
    const int ntiles = min(kEstBlockTiles, a.tiles - tile_lo);
    const int q_pos0 = a.n_ctx - a.last_q;          // position of the first of the last_q queries

    if (__syncthreads_or(threadIdx.x == 0 && *(volatile int32_t*)(a.status + MINF_ST_ERROR) != 0)) return;
    if ((smem_base & 1023u) != 0u) {
        if (threadIdx.x == 0) atomicOr(a.status + MINF_ST_ERROR, 2);
        return;
    }
    auto bar = [&](const unsigned long long* p) { return smem_u32(p); };
    volatile int* abort_flag = &ctl->abort;
    if (threadIdx.x == 0) {
        mbar_init(bar(&ctl->q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(&ctl->k_full[s]), 1);
            mbar_init(bar(&ctl->k_empty[s]), 1);
            mbar_init(bar(&ctl->s_full[s]), 1);
            mbar_init(bar(&ctl->s_empty[s]), 8);       // one arrival per softmax warp
        }
        ctl->abort = 0;
        fence_mbar_init();
    }
    if (PASS == 2 && threadIdx.x >= 64 && threadIdx.x < 192) {
        // exponent offset of every (head, query row): p = 2^(x*log2(e) + cst) is the normalised probability
        const int r = threadIdx.x - 64, hs = r >> 6, i = r & 63;
        float c = -INFINITY;
        if ((hs == 0 || has_h1) && i < a.last_q) {
            const float2 st = a.row_stats[((size_t)b * a.hq + h0 + hs) * 64 + i];
            if (st.y > 0.f) c = -(st.x * kLog2e + log2f(st.y));
        }
        ctl->cst[hs][i] = c;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&ctl->tmem_base), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    if (warp == 0) {
        if (lane == 0 && ntiles > 0) {
            tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k);
            // rows 0-63: head h0, rows 64-127: head h0+1 (zero-filled when absent: head coordinate out of range)
            mbar_arrive_expect_tx(bar(&ctl->q_full), kEstQBytes);
            const int h1 = has_h1 ? h0 + 1 : a.hq;   // a.hq is out of range -> zero fill
            tma_load_4d(smem_base, &tm_q, bar(&ctl->q_full), 0, 0, h0, b);
            tma_load_4d(smem_base + 8192, &tm_q, bar(&ctl->q_full), 0, 0, h1, b);
            tma_load_4d(smem_base + 16384, &tm_q, bar(&ctl->q_full), 64, 0, h0, b);
            tma_load_4d(smem_base + 16384 + 8192, &tm_q, bar(&ctl->q_full), 64, 0, h1, b);
            for (int i = 0; i < ntiles; ++i) {
                const int s = i & 1, use = i >> 1;
                if (use > 0 && !mbar_wait(bar(&ctl->k_empty[s]), (use - 1) & 1, abort_flag)) break;
                const uint32_t dst = smem_base + kEstQBytes + s * kEstKBytes;
                mbar_arrive_expect_tx(bar(&ctl->k_full[s]), kEstKBytes);
                tma_load_4d(dst, &tm_k, bar(&ctl->k_full[s]), 0, (tile_lo + i) * kEstTileN, hk, b);
                tma_load_4d(dst + 16384, &tm_k, bar(&ctl->k_full[s]), 64, (tile_lo + i) * kEstTileN, hk, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && ntiles > 0) {
            constexpr uint32_t idesc = umma_idesc(128, 128, true, false, false);
            bool ok = mbar_wait(bar(&ctl->q_full), 0, abort_flag);
            for (int i = 0; i < ntiles && ok; ++i) {
                const int s = i & 1, use = i >> 1;
                ok = mbar_wait(bar(&ctl->k_full[s]), use & 1, abort_flag);
                if (ok && use > 0) ok = mbar_wait(bar(&ctl->s_empty[s]), (use - 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t kb = smem_base + kEstQBytes + s * kEstKBytes;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t qd = umma_desc_sw128(smem_base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    const uint64_t kd = umma_desc_sw128(kb + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    // pass 1: rows = queries, columns = keys; pass 2: rows = keys, columns = queries
                    if (PASS == 1) umma_ss(tmem + s * 128, qd, kd, idesc, kk > 0);
                    else umma_ss(tmem + s * 128, kd, qd, idesc, kk > 0);
                }
                umma_commit(bar(&ctl->s_full[s]));
                umma_commit(bar(&ctl->k_empty[s]));
            }
        }
    } else {
        const int quarter = warp & 3;                  // TMEM lane quarter this warp may access
        const int half = (warp - 2) >> 2;              // which 64 of the 128 columns
        const int tl = 32 * quarter + lane;            // TMEM lane
        const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
        const int tid = threadIdx.x - 64;              // 0..255

        if (PASS == 1) {
            // ---- lane = query row (two heads x 64), this thread's columns = keys [64*half, +64) of a tile
            const int hs = tl >> 6, i = tl & 63;
            const bool row_ok = (hs == 0 || has_h1) && i < a.last_q;
            const int qpos = q_pos0 + i;               // key c is visible iff c <= qpos
            float row_m = -INFINITY, row_l = 0.f;
            bool ok = true;
            for (int it = 0; it < ntiles && ok; ++it) {
                const int s = it & 1, use = it >> 1;
                const int l0 = (tile_lo + it) * kEstTileN + 64 * half;   // first of this thread's keys inside the local keys
                const int c0 = a.col_base + l0;                          // and its position in the sequence
                ok = mbar_wait(bar(&ctl->s_full[s]), use & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                // only the tiles that reach the last queries' diagonal or the end of the keys need masks
                const bool plain = row_ok && c0 + 63 <= q_pos0 && l0 + 64 <= a.n_k;
#pragma unroll 1
                for (int q2 = 0; q2 < 2; ++q2) {
                    uint32_t xr[32];
                    tmem_ld32(tmem + s * 128 + half * 64 + q2 * 32 + lane_base, xr);
                    tmem_wait_ld();
                    float x[32];
                    float mx = -INFINITY;
                    if (plain) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            logits_pair<MUL>(xr[j], xr[j + 1], a.sqrt_d, a.rcp_sqrt_d, x[j], x[j + 1]);
                            mx = max3(mx, x[j], x[j + 1]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            float v0, v1;
                            logits_pair<MUL>(xr[j], xr[j + 1], a.sqrt_d, a.rcp_sqrt_d, v0, v1);
                            const int c = c0 + q2 * 32 + j;
                            x[j] = (row_ok && c <= qpos && l0 + q2 * 32 + j < a.n_k) ? v0 : -INFINITY;
                            x[j + 1] = (row_ok && c + 1 <= qpos && l0 + q2 * 32 + j + 1 < a.n_k) ? v1 : -INFINITY;
                            mx = max3(mx, x[j], x[j + 1]);
                        }
                    }
                    if (mx > row_m) {
                        row_l *= fast_exp2((row_m - mx) * kLog2e);   // 0 * 2^(-inf) = 0 on the first hit
                        row_m = mx;
                    }
                    if (row_m > -INFINITY) {
                        const float neg = -row_m * kLog2e;
                        float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int j = 0; j < 32; ++j) ps[j & 3] += fast_exp2(fmaf(x[j], kLog2e, neg));
                        row_l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(&ctl->s_empty[s]));
            }
            // the two halves of a row meet in shared memory; the first half's thread writes the block's entry
            if (half == 1) ctl->half_stat[tl] = make_float2(row_m, row_l);
            named_bar_sync(1, 256);
            if (half == 0 && ok && (hs == 0 || has_h1) && ntiles > 0) {
                const float2 o = ctl->half_stat[tl];
                const float m = fmaxf(row_m, o.x);
                float l = 0.f;
                if (row_l > 0.f) l += row_l * fast_exp2((row_m - m) * kLog2e);
                if (o.y > 0.f) l += o.y * fast_exp2((o.x - m) * kLog2e);
                a.stats[(((size_t)b * a.hq + h0 + hs) * 64 + i) * a.blocks_total + a.block_offset + blk] = make_float2(m, l);
            }
        } else {
            // ---- lane = key of the tile, this thread's columns = the 64 query rows of head h0 + half
            const int hh = half;
            const bool head_ok = hh == 0 || has_h1;
            const size_t bh = (size_t)b * a.hq + h0 + hh;
            const int ct = tid & 127;                  // this thread's place in the combination step
            float carry = 0.f;                         // partial sum of an offset that the next tile completes
            bool ok = true;
            // every warp runs every iteration and meets the others at the named barrier even after a
            // wait was abandoned (its results are then reported as invalid through the status word)
            for (int it = 0; it < ntiles; ++it) {
                const int s = it & 1, use = it >> 1;
                const int l0 = (tile_lo + it) * kEstTileN;   // first key of the tile inside the local keys
                const int c0 = a.col_base + l0;              // and its position in the sequence
                float* pbuf = part + (size_t)(it & 1) * (4 * 2 * kDiagSlots);
                if (ok) ok = mbar_wait(bar(&ctl->s_full[s]), use & 1, abort_flag);
                tc_fence_after();
                if (head_ok && ok) {
                    const int kloc = l0 + tl;                // this thread's key
                    const int c = c0 + tl;
                    const bool key_ok = kloc < a.n_k;
                    const bool plain = c0 + kEstTileN - 1 <= q_pos0 && l0 + kEstTileN <= a.n_k;
                    float* my_part = pbuf + (quarter * 2 + hh) * kDiagSlots;
                    float vsum = 0.f, acc = 0.f;
#pragma unroll 1
                    for (int q2 = 0; q2 < 2; ++q2) {
                        uint32_t xr[32];
                        tmem_ld32(tmem + s * 128 + hh * 64 + q2 * 32 + lane_base, xr);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            float v0, v1;
                            logits_pair<MUL>(xr[j], xr[j + 1], a.sqrt_d, a.rcp_sqrt_d, v0, v1);
                            const int i0 = q2 * 32 + j;
                            const float2 cc = *reinterpret_cast<const float2*>(&ctl->cst[hh][i0]);
                            float p0 = fast_exp2(fmaf(v0, kLog2e, cc.x));
                            float p1 = fast_exp2(fmaf(v1, kLog2e, cc.y));
                            if (!plain) {
                                p0 = (key_ok && c <= q_pos0 + i0) ? p0 : 0.f;
                                p1 = (key_ok && c <= q_pos0 + i0 + 1) ? p1 : 0.f;
                            }
                            // the sum for i - key = const moves up one lane per query row; what leaves
                            // lane 31 is complete as far as this warp's 32 keys go
                            vsum += p0;
                            acc = __shfl_up_sync(0xffffffffu, acc, 1);
                            if (lane == 0) acc = 0.f;
                            acc += p0;
                            if (lane == 31) my_part[i0] = acc;
                            vsum += p1;
                            acc = __shfl_up_sync(0xffffffffu, acc, 1);
                            if (lane == 0) acc = 0.f;
                            acc += p1;
                            if (lane == 31 && i0 + 1 < 63) my_part[i0 + 1] = acc;
                        }
                    }
                    my_part[94 - lane] = acc;           // slot s holds i - key = s - 32*quarter - 31
                    if (key_ok) a.vertical[bh * a.n_ctx + c] = vsum;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(bar(&ctl->s_empty[s]));
                named_bar_sync(1, 256);
                // ---- combination: thread ct of a head sums the tile's partials for i - key = ct - 127 and ct + 1
                if (head_ok) {
                    const float* hp = pbuf + hh * kDiagSlots;
                    auto tile_sum = [&](int d) {
                        float sum = 0.f;
#pragma unroll
                        for (int wq = 0; wq < 4; ++wq) {
                            const int sl = d + 32 * wq + 31;
                            if (sl >= 0 && sl <= 94) sum += hp[wq * 2 * kDiagSlots + sl];
                        }
                        return sum;
                    };
                    float* sl_out = a.slash + bh * a.n_ctx;
                    const int off1 = q_pos0 - c0 + (ct - 127);
                    const float v1 = tile_sum(ct - 127);
                    if (ct <= 62) {
                        // offsets shared with the previous tile: its part was carried in a register
                        const int off2 = q_pos0 - c0 + (ct + 1);
                        const float v2 = tile_sum(ct + 1);
                        if (off2 >= 0 && off2 < a.n_ctx) {
                            if (it > 0) sl_out[off2] = carry + v2;
                            else if (v2 != 0.f) atomicAdd(sl_out + off2, v2);      // the other part comes from another CTA
                        }
                        carry = v1;                      // completed by the next tile
                        if (it == ntiles - 1 && off1 >= 0 && off1 < a.n_ctx && v1 != 0.f) atomicAdd(sl_out + off1, v1);
                    } else if (off1 >= 0 && off1 < a.n_ctx) {
                        sl_out[off1] = v1;               // offsets only this tile touches
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && ctl->abort) atomicOr(a.status + MINF_ST_ERROR, 1);
    if (warp == 1) tmem_dealloc(tmem, 256);
}

// Row statistics of the whole sequence from the per-block ones: one warp per (head, query row),
// blocks taken in ascending order with a fixed reduction tree, so the result depends on the
// block grid only.
__global__ void __launch_bounds__(256) vs_stats_combine_kernel(const float2* stats, int rows, int blocks_total, float2* row_stats) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float2* st = stats + (size_t)row * blocks_total;
    float m = -INFINITY;
    for (int c = lane; c < blocks_total; c += 32) m = fmaxf(m, st[c].x);
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
    for (int c = lane; c < blocks_total; c += 32) {
        const float2 e = st[c];
        if (e.y > 0.f) l += e.y * exp2f((e.x - m) * kLog2e);
    }
    for (int o = 16; o; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) row_stats[row] = make_float2(m, l);
}

// ------------------------------------------------------------------------------------ top-k
constexpr int kSelThreads = 1024;
constexpr int kSelItems = 8;
constexpr int kSelSegment = kSelThreads * kSelItems;     // elements of one list handled by one CTA
constexpr int kSelBins = 2048;
constexpr int kSelStateWords = 8;                         // prefix, remaining, done[3], ties_total, spare

struct SelectArgs {
    int lists, n_ctx, segments;
    const float* vertical;
    const float* slash;
    const int32_t* vertical_size;   // per head budgets before clamping
    const int32_t* slash_size;
    int cap_v, cap_s;
    int force_columns, force_diagonals;   // the first columns / nearest diagonals that are always taken
    int min_vertical, min_slash;          // budgets are raised to these
    int32_t* v_idx;
    int32_t* s_idx;
    int32_t* nnz_v;
    int32_t* nnz_s;
    uint32_t* hist;                 // [3][lists][kSelBins]
    uint32_t* state;                // [lists][kSelStateWords]
    uint32_t* seg_counts;           // [lists][segments][2]: keys above the threshold, keys equal to it
};

// value of element `pos` in iteration order, with the forced +inf entries applied
//   vertical: pos = key index, first 30 forced          (minference_forward.py:608)
//   slash:    pos = N-1-offset (the reference's order), offsets < 100 forced (:612; 30 in the static
//             variant :433 and in the offline search :145)
__device__ __forceinline__ uint32_t sel_key(const SelectArgs& a, const float* src, int pos, int n, bool is_slash) {
    if (is_slash) {
        const int off = n - 1 - pos;
        return off < a.force_diagonals ? 0x7f800000u : __float_as_uint(src[off]);
    }
    return pos < a.force_columns ? 0x7f800000u : __float_as_uint(src[pos]);
}

// list = 2 * (batch*heads index) + (0 vertical | 1 slash); returns k (or -1 when the head is skipped)
__device__ __forceinline__ int sel_list_k(const SelectArgs& a, int list) {
    const int bh = list >> 1;
    const bool is_slash = list & 1;
    const int budget = is_slash ? a.slash_size[bh] : a.vertical_size[bh];
    if (budget < 0) return -1;
    const int k = min(a.n_ctx, max(budget, is_slash ? a.min_slash : a.min_vertical));    // minference_forward.py:600
    return min(k, is_slash ? a.cap_s : a.cap_v);
}

// One radix level: histogram of this CTA's segment among the keys that match the prefix found so
// far; the CTA that finishes last walks the list's histogram from the top and fixes the next bits.
//   level 0: bits 30-20 (the sign bit is clear: scores are >= 0), level 1: bits 19-10, level 2: bits 9-0
template <int LEVEL>
__global__ void __launch_bounds__(kSelThreads) vs_select_hist_kernel(const SelectArgs a) {
    constexpr int kShift = LEVEL == 0 ? 20 : (LEVEL == 1 ? 10 : 0);
    constexpr int kBins = LEVEL == 0 ? 2048 : 1024;
    constexpr uint32_t kPrefixMask = LEVEL == 0 ? 0u : (LEVEL == 1 ? 0x7ff00000u : 0x7ffffc00u);
    __shared__ uint32_t hist[kSelBins];
    __shared__ int sh_last;
    const int list = blockIdx.y, seg = blockIdx.x;
    const int k = sel_list_k(a, list);
    const bool is_slash = list & 1;
    if (LEVEL == 0 && seg == 0 && threadIdx.x == 0) (is_slash ? a.nnz_s : a.nnz_v)[list >> 1] = k;
    if (k < 0) return;
    const int n = a.n_ctx;
    const float* src = (is_slash ? a.slash : a.vertical) + (size_t)(list >> 1) * n;
    uint32_t* st = a.state + (size_t)list * kSelStateWords;
    const uint32_t prefix = LEVEL == 0 ? 0u : st[0];
    for (int i = threadIdx.x; i < kBins; i += kSelThreads) hist[i] = 0;
    __syncthreads();
    const int p0 = seg * kSelSegment;
#pragma unroll
    for (int j = 0; j < kSelItems; ++j) {
        const int pos = p0 + j * kSelThreads + threadIdx.x;
        if (pos < n) {
            const uint32_t key = sel_key(a, src, pos, n, is_slash);
            if ((key & kPrefixMask) == prefix) atomicAdd(&hist[(key >> kShift) & (kBins - 1)], 1u);
        }
    }
    __syncthreads();
    uint32_t* gh = a.hist + ((size_t)LEVEL * a.lists + list) * kSelBins;
    for (int i = threadIdx.x; i < kBins; i += kSelThreads)
        if (hist[i]) atomicAdd(&gh[i], hist[i]);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) sh_last = atomicAdd(&st[2 + LEVEL], 1u) == (uint32_t)(a.segments - 1);
    __syncthreads();
    if (!sh_last) return;
    // ---- last CTA of this list and level: find the bin that holds the k-th largest key
    __threadfence();
    const uint32_t remaining = LEVEL == 0 ? (uint32_t)k : st[1];
    // inclusive suffix sums over the bins (descending bin order), two bins per thread at level 0
    __shared__ uint32_t wsum[32];
    constexpr int kPer = kBins / kSelThreads;                  // 2 or 1
    uint32_t cnt[kPer];
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        // thread t owns bins (kBins - 1 - t*kPer - j): highest bins first
        cnt[j] = ((volatile uint32_t*)gh)[kBins - 1 - (threadIdx.x * kPer + j)];
        mine += cnt[j];
    }
    uint32_t incl = mine;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = wsum[lane];
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        wsum[lane] = w;
    }
    __syncthreads();
    uint32_t before = (warp ? wsum[warp - 1] : 0u) + incl - mine;   // keys in higher bins than this thread's
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        if (before < remaining && before + cnt[j] >= remaining) {
            const uint32_t bin = (uint32_t)(kBins - 1 - (threadIdx.x * kPer + j));
            st[0] = prefix | (bin << kShift);
            st[1] = remaining - before;          // how many keys of this bin are still wanted
            if (LEVEL == 2) st[5] = cnt[j];      // keys equal to the threshold
        }
        before += cnt[j];
    }
}

// keys above the threshold / equal to it, per segment
__global__ void __launch_bounds__(kSelThreads) vs_select_count_kernel(const SelectArgs a) {
    const int list = blockIdx.y, seg = blockIdx.x;
    if (sel_list_k(a, list) < 0) return;
    const bool is_slash = list & 1;
    const int n = a.n_ctx;
    const float* src = (is_slash ? a.slash : a.vertical) + (size_t)(list >> 1) * n;
    const uint32_t thr = a.state[(size_t)list * kSelStateWords];
    int gt = 0, eq = 0;
    const int p0 = seg * kSelSegment;
#pragma unroll
    for (int j = 0; j < kSelItems; ++j) {
        const int pos = p0 + j * kSelThreads + threadIdx.x;
        if (pos < n) {
            const uint32_t key = sel_key(a, src, pos, n, is_slash);
            gt += key > thr;
            eq += key == thr;
        }
    }
    __shared__ int sh[2];
    if (threadIdx.x < 2) sh[threadIdx.x] = 0;
    __syncthreads();
    for (int o = 16; o; o >>= 1) {
        gt += __shfl_down_sync(0xffffffffu, gt, o);
        eq += __shfl_down_sync(0xffffffffu, eq, o);
    }
    if ((threadIdx.x & 31) == 0) {
        if (gt) atomicAdd(&sh[0], gt);
        if (eq) atomicAdd(&sh[1], eq);
    }
    __syncthreads();
    if (threadIdx.x < 2) a.seg_counts[((size_t)list * a.segments + seg) * 2 + threadIdx.x] = (uint32_t)sh[threadIdx.x];
}

// ordered compaction: every thread owns kSelItems consecutive positions of its segment
__global__ void __launch_bounds__(kSelThreads) vs_select_write_kernel(const SelectArgs a) {
    const int list = blockIdx.y, seg = blockIdx.x;
    const int k = sel_list_k(a, list);
    if (k < 0) return;
    const bool is_slash = list & 1;
    const int n = a.n_ctx;
    const int cap = is_slash ? a.cap_s : a.cap_v;
    const float* src = (is_slash ? a.slash : a.vertical) + (size_t)(list >> 1) * n;
    int32_t* out = (is_slash ? a.s_idx : a.v_idx) + (size_t)(list >> 1) * cap;
    const uint32_t* st = a.state + (size_t)list * kSelStateWords;
    const uint32_t thr = st[0];
    const int ties_needed = (int)st[1], ties_total = (int)st[5];
    // vertical: ties taken from the lowest key index: the first `ties_needed` in order.
    // slash: order is ascending N-1-offset, i.e. descending offset; smallest offsets win, so the
    //        first (ties_total - ties_needed) ties in this order are skipped.
    const int ties_skip = is_slash ? ties_total - ties_needed : 0;
    if (seg == 0)
        for (int i = k + threadIdx.x; i < cap; i += kSelThreads) out[i] = 0;

    __shared__ int sh_base[2];
    __shared__ int wsum[2][32];
    if (threadIdx.x < 2) {      // keys above / equal in the segments before this one
        int sum = 0;
        for (int s = 0; s < seg; ++s) sum += (int)a.seg_counts[((size_t)list * a.segments + s) * 2 + threadIdx.x];
        sh_base[threadIdx.x] = sum;
    }
    uint32_t key[kSelItems];
    int gt = 0, eq = 0;
    const int p0 = seg * kSelSegment + threadIdx.x * kSelItems;
#pragma unroll
    for (int j = 0; j < kSelItems; ++j) {
        key[j] = p0 + j < n ? sel_key(a, src, p0 + j, n, is_slash) : 0u;
        gt += p0 + j < n && key[j] > thr;
        eq += p0 + j < n && key[j] == thr;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int gi = gt, ei = eq;
    for (int o = 1; o < 32; o <<= 1) {
        const int ug = __shfl_up_sync(0xffffffffu, gi, o), ue = __shfl_up_sync(0xffffffffu, ei, o);
        if (lane >= o) { gi += ug; ei += ue; }
    }
    if (lane == 31) { wsum[0][warp] = gi; wsum[1][warp] = ei; }
    __syncthreads();
    if (warp < 2) {
        int w = wsum[warp][lane];
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        wsum[warp][lane] = w;
    }
    __syncthreads();
    int gt_before = sh_base[0] + (warp ? wsum[0][warp - 1] : 0) + gi - gt;
    int eq_before = sh_base[1] + (warp ? wsum[1][warp - 1] : 0) + ei - eq;
#pragma unroll
    for (int j = 0; j < kSelItems; ++j) {
        if (p0 + j >= n) break;
        const bool is_gt = key[j] > thr, is_eq = key[j] == thr;
        const int ties_taken_before = min(max(eq_before - ties_skip, 0), ties_needed);
        const bool take = is_gt || (is_eq && eq_before >= ties_skip && eq_before < ties_skip + ties_needed);
        const int dst = gt_before + ties_taken_before;
        if (take && dst < cap) out[dst] = is_slash ? (n - 1 - (p0 + j)) : (p0 + j);
        gt_before += is_gt;
        eq_before += is_eq;
    }
}

// ------------------------------------------------------------------------------------ host
int make_tmap_bhnd(CUtensorMap* tm, const void* base, int batch, int heads, int tokens, const int64_t st[3],
                   int box_rows, const char* what);   // defined in sparse_attn_fwd.cu

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace minf

using namespace minf;

extern "C" int minf_vs_scores_blocks(int n_k) { return n_k < 1 ? 0 : (n_k + kEstBlockKeys - 1) / kEstBlockKeys; }

extern "C" int minf_vs_scores_pass(
    int pass, const void* q_last, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int n_k, int col_base, int head_dim,
    void* stats, int block_offset, int blocks_total, const void* row_stats,
    float* vertical_scores, float* slash_scores, int32_t* status, void* stream) {
    return minf_vs_scores_pass_divisor(pass, q_last, k, q_strides, k_strides, batch, hq, hkv, context_size, n_k, col_base,
                                       head_dim, sqrtf((float)head_dim), stats, block_offset, blocks_total, row_stats,
                                       vertical_scores, slash_scores, status, stream);
}

extern "C" int minf_vs_scores_pass_divisor(
    int pass, const void* q_last, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int n_k, int col_base, int head_dim, float logit_divisor,
    void* stats, int block_offset, int blocks_total, const void* row_stats,
    float* vertical_scores, float* slash_scores, int32_t* status, void* stream) {
    if (!(logit_divisor > 0.f)) return fail(MINF_E_ARG, "logit_divisor must be positive");
    if (!q_last || !k || !status) return fail(MINF_E_ARG, "null pointer argument");
    if (pass != 1 && pass != 2) return fail(MINF_E_ARG, "pass must be 1 or 2");
    if (pass == 1 && !stats) return fail(MINF_E_ARG, "pass 1 needs the statistics array");
    if (pass == 2 && (!row_stats || !vertical_scores || !slash_scores))
        return fail(MINF_E_ARG, "pass 2 needs the row statistics and both score arrays");
    if (head_dim != 128) return fail(MINF_E_UNSUPPORTED, "head_dim must be 128 (got %d)", head_dim);
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || context_size < 1 || batch > 65535 || n_k < 1 ||
        col_base < 0 || col_base + n_k > context_size)
        return fail(MINF_E_ARG, "bad sizes");
    if (col_base % kEstTileN) return fail(MINF_E_ARG, "col_base must be a multiple of %d", kEstTileN);
    EstArgs a{};
    a.batch = batch; a.hq = hq; a.hkv = hkv; a.n_ctx = context_size;
    a.last_q = context_size < 64 ? context_size : 64;
    a.n_k = n_k; a.col_base = col_base;
    a.group = hq / hkv;
    a.pairs_per_group = (a.group + 1) / 2;
    a.tiles = (n_k + kEstTileN - 1) / kEstTileN;
    const int blocks = minf_vs_scores_blocks(n_k);
    if (pass == 1 && (block_offset < 0 || block_offset + blocks > blocks_total))
        return fail(MINF_E_ARG, "block window outside the statistics array");
    a.block_offset = block_offset; a.blocks_total = blocks_total;
    a.stats = static_cast<float2*>(stats);
    a.row_stats = static_cast<const float2*>(row_stats);
    a.vertical = vertical_scores; a.slash = slash_scores;
    a.sqrt_d = logit_divisor;
    a.rcp_sqrt_d = 1.0f / a.sqrt_d;
    a.status = status;
    CUtensorMap tq, tk;
    int rc;
    if ((rc = make_tmap_bhnd(&tq, q_last, batch, hq, a.last_q, q_strides, 64, "q_last"))) return rc;
    if ((rc = make_tmap_bhnd(&tk, k, batch, hkv, n_k, k_strides, 128, "k"))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = kEstCtlOff + sizeof(EstControl);
    dim3 grid(blocks, hkv * a.pairs_per_group, batch);
    // the reciprocal multiply is exact for these two divisors (see logits_pair); any other one takes the division
    const bool mul = logit_divisor == 1.0f || logit_divisor == sqrtf(128.0f);
    auto launch = [&](auto kernel) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        kernel<<<grid, kEstThreads, smem, st>>>(tq, tk, a);
        return cudaSuccess;
    };
    if (pass == 1) {
        MINF_CUDA_OK(mul ? launch(vs_scores_kernel<1, true>) : launch(vs_scores_kernel<1, false>));
    } else {
        MINF_CUDA_OK(mul ? launch(vs_scores_kernel<2, true>) : launch(vs_scores_kernel<2, false>));
    }
    MINF_LAUNCH_OK("vs_scores_kernel");
    return MINF_OK;
}

extern "C" int minf_vs_scores_combine(const void* stats, int batch, int hq, int blocks_total, void* row_stats, void* stream) {
    if (!stats || !row_stats) return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || hq < 1 || blocks_total < 1) return fail(MINF_E_ARG, "bad sizes");
    const int rows = batch * hq * 64;
    vs_stats_combine_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float2*>(stats), rows, blocks_total, static_cast<float2*>(row_stats));
    MINF_LAUNCH_OK("vs_stats_combine_kernel");
    return MINF_OK;
}

extern "C" size_t minf_vs_select_scratch_bytes(int batch, int hq, int context_size) {
    if (batch < 1 || hq < 1 || context_size < 1) return 0;
    const size_t lists = 2 * (size_t)batch * hq;
    const size_t segments = ((size_t)context_size + kSelSegment - 1) / kSelSegment;
    return align256(lists * (3 * kSelBins + kSelStateWords) * sizeof(uint32_t)) + align256(lists * segments * 2 * sizeof(uint32_t));
}

extern "C" int minf_vs_select(
    const float* vertical_scores, const float* slash_scores, int batch, int hq, int context_size,
    const int32_t* vertical_size, const int32_t* slash_size, int cap_v, int cap_s,
    int32_t* v_idx_out, int32_t* s_idx_out, int32_t* nnz_v_out, int32_t* nnz_s_out,
    int force_columns, int force_diagonals, int min_vertical, int min_slash, void* scratch, void* stream) {
    if (!vertical_scores || !slash_scores || !vertical_size || !slash_size || !v_idx_out || !s_idx_out || !nnz_v_out ||
        !nnz_s_out || !scratch)
        return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || hq < 1 || context_size < 1 || cap_v < 1 || cap_s < 1) return fail(MINF_E_ARG, "bad sizes");
    if (force_columns < 0 || force_diagonals < 0 || min_vertical < 0 || min_slash < 0) return fail(MINF_E_ARG, "bad selection rules");
    SelectArgs s{};
    s.force_columns = force_columns; s.force_diagonals = force_diagonals;
    s.min_vertical = min_vertical; s.min_slash = min_slash;
    s.lists = 2 * batch * hq; s.n_ctx = context_size;
    s.segments = (context_size + kSelSegment - 1) / kSelSegment;
    if (s.lists > 65535) return fail(MINF_E_UNSUPPORTED, "too many heads");
    s.vertical = vertical_scores; s.slash = slash_scores;
    s.vertical_size = vertical_size; s.slash_size = slash_size;
    s.cap_v = cap_v; s.cap_s = cap_s;
    s.v_idx = v_idx_out; s.s_idx = s_idx_out; s.nnz_v = nnz_v_out; s.nnz_s = nnz_s_out;
    const size_t head = (size_t)s.lists * (3 * kSelBins + kSelStateWords) * sizeof(uint32_t);
    s.hist = static_cast<uint32_t*>(scratch);
    s.state = s.hist + (size_t)3 * s.lists * kSelBins;
    s.seg_counts = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(scratch) + align256(head));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    MINF_CUDA_OK(cudaMemsetAsync(scratch, 0, head, st));       // histograms, prefixes and completion counters
    const dim3 grid(s.segments, s.lists);
    vs_select_hist_kernel<0><<<grid, kSelThreads, 0, st>>>(s);
    vs_select_hist_kernel<1><<<grid, kSelThreads, 0, st>>>(s);
    vs_select_hist_kernel<2><<<grid, kSelThreads, 0, st>>>(s);
    vs_select_count_kernel<<<grid, kSelThreads, 0, st>>>(s);
    vs_select_write_kernel<<<grid, kSelThreads, 0, st>>>(s);
    MINF_LAUNCH_OK("vs_select kernels");
    return MINF_OK;
}

// scratch layout of minf_vs_estimate: per-block statistics | row statistics | score arrays | select scratch
extern "C" size_t minf_vs_estimate_scratch_bytes(int batch, int hq, int context_size) {
    if (batch < 1 || hq < 1 || context_size < 1) return 0;
    const size_t blocks = (size_t)minf_vs_scores_blocks(context_size);
    size_t bytes = align256((size_t)batch * hq * 64 * blocks * sizeof(float2));
    bytes += align256((size_t)batch * hq * 64 * sizeof(float2));
    bytes += align256(2 * (size_t)batch * hq * context_size * sizeof(float));   // score arrays when the caller passes none
    bytes += minf_vs_select_scratch_bytes(batch, hq, context_size);
    return bytes + 256;
}

extern "C" int minf_vs_estimate(
    const void* q, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim,
    const int32_t* vertical_size, const int32_t* slash_size, int cap_v, int cap_s,
    int32_t* v_idx_out, int32_t* s_idx_out, int32_t* nnz_v_out, int32_t* nnz_s_out,
    float* vertical_scores_out, float* slash_scores_out,
    void* scratch, int32_t* status, void* stream) {
    if (!q || !k || !vertical_size || !slash_size || !v_idx_out || !s_idx_out || !nnz_v_out || !nnz_s_out || !scratch || !status)
        return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || context_size < 1 || cap_v < 1 || cap_s < 1 || batch > 65535)
        return fail(MINF_E_ARG, "bad sizes");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int blocks = minf_vs_scores_blocks(context_size);
    unsigned char* sc = static_cast<unsigned char*>(scratch);
    sc = reinterpret_cast<unsigned char*>(align256(reinterpret_cast<size_t>(sc)));
    void* stats = sc;
    sc += align256((size_t)batch * hq * 64 * blocks * sizeof(float2));
    void* row_stats = sc;
    sc += align256((size_t)batch * hq * 64 * sizeof(float2));
    float* vertical = vertical_scores_out ? vertical_scores_out : reinterpret_cast<float*>(sc);
    float* slash = slash_scores_out ? slash_scores_out : reinterpret_cast<float*>(sc) + (size_t)batch * hq * context_size;
    sc += align256(2 * (size_t)batch * hq * context_size * sizeof(float));
    void* sel_scratch = sc;
    // the last min(64, N) queries, viewed in place
    const int last_q = context_size < 64 ? context_size : 64;
    const void* q_last = static_cast<const __nv_bfloat16*>(q) + (size_t)(context_size - last_q) * q_strides[2];
    MINF_CUDA_OK(cudaMemsetAsync(slash, 0, (size_t)batch * hq * context_size * sizeof(float), st));
    int rc;
    if ((rc = minf_vs_scores_pass(1, q_last, k, q_strides, k_strides, batch, hq, hkv, context_size, context_size, 0, head_dim,
                                  stats, 0, blocks, nullptr, nullptr, nullptr, status, stream)))
        return rc;
    if ((rc = minf_vs_scores_combine(stats, batch, hq, blocks, row_stats, stream))) return rc;
    if ((rc = minf_vs_scores_pass(2, q_last, k, q_strides, k_strides, batch, hq, hkv, context_size, context_size, 0, head_dim,
                                  nullptr, 0, blocks, row_stats, vertical, slash, status, stream)))
        return rc;
    return minf_vs_select(vertical, slash, batch, hq, context_size, vertical_size, slash_size, cap_v, cap_s,
                          v_idx_out, s_idx_out, nnz_v_out, nnz_s_out, 30, 100, 30, 50, sel_scratch, stream);
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant of the estimator.
//
// Some hosts of this library cannot hand it scratch memory: an attention plugin loaded into
// a serving process whose device memory is one arena carved up at start-up (the plugin has no
// handle to that allocator and the process may have no free device memory left to cudaMalloc
// from), or a caller on a latency-critical path that is not allowed to touch an allocator at
// all.  For them the scratch of the estimator lives in the library image: a fixed array in
// device global memory that exists once per GPU that has loaded the library, from the moment
// the module is loaded until the process ends.
//
// The array's name is only meaningful to device code.  Host code must ask the runtime where the
// array lives on the current device (cudaGetSymbolAddress); handing the bare symbol to a kernel
// would pass a host-side placeholder, not a device address.  The lookup is done once per device,
// on the first call made with that device current, and cached.
namespace minf {

constexpr size_t kStaticScratchBytes = 16u << 20;    // 16 MiB per GPU, stated in the header as the limit
static __device__ __align__(256) unsigned char g_estimate_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_estimate_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the static scratch on the current device (looked up on first use).
static int static_scratch_for_current_device(void** out) {
    int dev = -1;
    MINF_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(MINF_E_UNSUPPORTED, "device ordinal %d out of range", dev);
    void* p = __atomic_load_n(&g_estimate_scratch_addr[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        MINF_CUDA_OK(cudaGetSymbolAddress(&p, g_estimate_scratch));
        if (!p) return fail(MINF_E_CUDA, "cudaGetSymbolAddress returned a null address");
        __atomic_store_n(&g_estimate_scratch_addr[dev], p, __ATOMIC_RELEASE);   // same value from every thread
    }
    *out = p;
    return MINF_OK;
}

}  // namespace minf

extern "C" size_t minf_vs_estimate_static_scratch_limit(void) { return minf::kStaticScratchBytes; }

// Same computation and outputs as minf_vs_estimate, without a caller-provided scratch buffer and
// without any allocation (no cudaMalloc/cudaFree, no allocating library call): the scratch is the
// static array above.  Problems larger than the array are refused.  The array is shared by every
// call on the GPU and still holds what the previous call left there; the parts that must start
// at zero (the diagonal-score accumulators, the select histograms and counters) are cleared on the
// stream before the kernels run, as in the buffer-taking entry point.  Two calls whose kernels may
// overlap on the same GPU (different streams, or different host threads) would use the same
// scratch at once: that is a data race the caller must exclude.  The first call on a device
// performs the one-time address lookup and should therefore be made outside any stream capture.
extern "C" int minf_vs_estimate_static(
    const void* q, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim,
    const int32_t* vertical_size, const int32_t* slash_size, int cap_v, int cap_s,
    int32_t* v_idx_out, int32_t* s_idx_out, int32_t* nnz_v_out, int32_t* nnz_s_out,
    int32_t* status, void* stream) {
    const size_t need = minf_vs_estimate_scratch_bytes(batch, hq, context_size);
    if (need == 0) return minf::fail(MINF_E_ARG, "bad sizes");
    if (need > minf::kStaticScratchBytes)
        return minf::fail(MINF_E_UNSUPPORTED,
                          "problem needs %zu bytes of scratch, the built-in scratch holds %zu "
                          "(batch*heads*tokens of about one million); use minf_vs_estimate with a caller buffer",
                          need, minf::kStaticScratchBytes);
    void* scratch = nullptr;
    int rc = minf::static_scratch_for_current_device(&scratch);
    if (rc) return rc;
    return minf_vs_estimate(q, k, q_strides, k_strides, batch, hq, hkv, context_size, head_dim,
                            vertical_size, slash_size, cap_v, cap_s, v_idx_out, s_idx_out, nnz_v_out, nnz_s_out,
                            nullptr, nullptr, scratch, status, stream);
}
