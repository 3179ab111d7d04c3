// Online vertical/slash index estimation for every head of a layer.
//
// Replaces the torch ops of vertical_and_slash_kernel (modules/minference_forward.py:599-614
// of the reference) and sum_all_diagonal_matrix (:110-116), which run once per head from a
// Python loop: a skinny GEMM, a [64, N] fp32 softmax, a zero-padded strided view for the
// diagonal sums and two full top-k sorts.
//
// Here: two passes of one tcgen05 kernel over K, then one select kernel.
//   scores kernel   CTA = (column chunk, pair of query heads sharing a KV head, batch).
//                   A = the last 64 queries of both heads (128 rows), B = 128 keys per tile by
//                   TMA, D = 128x128 fp32 logits in TMEM (double buffered); one thread per
//                   query row reads its logits.  Logits are rounded to bf16 twice like the
//                   reference's bf16 einsum followed by the bf16 division by sqrt(d).
//     pass 1        running (max, sum exp) per row and chunk -> scratch
//     pass 2        p = exp(x - M) / L staged in shared memory; column sums give the vertical
//                   score of every key, sums along i - j = const give the slash score of
//                   every diagonal offset (a diagonal is 64 long, so it touches at most two
//                   128-key tiles: the two float atomics commute, results are deterministic)
//   select kernel   CTA = (head, vertical | slash): +inf forcing of the first 30 keys / the
//                   100 nearest diagonals, radix select of the k-th largest score, ordered
//                   compaction.  Output is already sorted the way the index conversion wants
//                   (vertical ascending, slash offsets descending).  Equal scores at the
//                   threshold: lowest key index first / smallest offset first (torch.topk
//                   leaves this unspecified).
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.h"
#include "sm100_ptx.cuh"

namespace minf {

constexpr int kEstTileN = 128;
constexpr int kEstPitch = 129;
constexpr uint32_t kEstQBytes = 128 * 256;
constexpr uint32_t kEstKBytes = 128 * 256;
constexpr uint32_t kEstPOff = kEstQBytes + 2 * kEstKBytes;           // 98304
constexpr uint32_t kEstPBytes = 128 * kEstPitch * 4;                 // 66048
// pass 1 keeps no probability tile, so two of its CTAs fit one SM
template <int PASS> constexpr uint32_t est_ctl_off() { return PASS == 1 ? kEstPOff : kEstPOff + kEstPBytes; }

struct EstControl {
    unsigned long long q_full;
    unsigned long long k_full[2], k_empty[2], s_full[2], s_empty[2];
    uint32_t tmem_base;
    int abort;
};

struct EstArgs {
    int batch, hq, hkv, n_ctx, last_q;
    int n_k, col_base;               // local keys and the position of the first one
    int group, pairs_per_group;      // hq / hkv, ceil(group / 2)
    int tiles, chunks, tiles_per_chunk;   // geometry of this call over its local keys
    int chunk_offset, chunks_total;  // where this call's chunks sit among all chunks of the sequence
    float2* stats;                   // [batch*hq][64][chunks_total]
    float* vertical;                 // [batch*hq][n_ctx]
    float* slash;                    // [batch*hq][n_ctx], indexed by diagonal offset
    float inv_sqrt_d_div;            // sqrt(d): logits are divided by it
    float rcp_sqrt_d;                // its reciprocal, for the refined multiply that replaces the division
    int32_t* status;
};

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// x / d correctly rounded from a reciprocal and one Newton step on the exact remainder (no MUFU,
// three FMA-pipe instructions instead of the division sequence).
__device__ __forceinline__ float div_refined(float x, float d, float rcp) {
    const float q = x * rcp;
    return fmaf(fmaf(-q, d, x), rcp, q);
}
// The reference's logits: the bf16 GEMM output divided by sqrt(d) in fp32 and rounded to bf16 again.
__device__ __forceinline__ void logits_pair(uint32_t a0, uint32_t a1, float d, float rcp, float& v0, float& v1) {
    const uint32_t g = pack_bf16x2(__uint_as_float(a0), __uint_as_float(a1));
    const uint32_t r = pack_bf16x2(div_refined(__uint_as_float(g << 16), d, rcp),
                                   div_refined(__uint_as_float(g & 0xffff0000u), d, rcp));
    v0 = __uint_as_float(r << 16);
    v1 = __uint_as_float(r & 0xffff0000u);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int PASS>
__global__ void __launch_bounds__(192, PASS == 1 ? 2 : 1)
vs_scores_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const EstArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    EstControl* ctl = reinterpret_cast<EstControl*>(smem + est_ctl_off<PASS>());
    float* ptile = reinterpret_cast<float*>(smem + kEstPOff);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int chunk = blockIdx.x;
    const int pair = blockIdx.y;                       // over hkv * pairs_per_group
    const int b = blockIdx.z;
    const int hk = pair / a.pairs_per_group;
    const int h0 = hk * a.group + 2 * (pair % a.pairs_per_group);
    const bool has_h1 = (2 * (pair % a.pairs_per_group) + 1) < a.group;
    const int tile_lo = chunk * a.tiles_per_chunk;
    const int tile_hi = min(tile_lo + a.tiles_per_chunk, a.tiles);
    const int ntiles = tile_hi - tile_lo;
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
            mbar_init(bar(&ctl->s_empty[s]), 128);
        }
        ctl->abort = 0;
        fence_mbar_init();
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
                    const uint64_t ad = umma_desc_sw128(smem_base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    const uint64_t bd = umma_desc_sw128(kb + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    umma_ss(tmem + s * 128, ad, bd, idesc, kk > 0);
                }
                umma_commit(bar(&ctl->s_full[s]));
                umma_commit(bar(&ctl->k_empty[s]));
            }
        }
    } else {
        const int sub = warp & 3;
        const int r = 32 * sub + lane;               // row of the 128-row tile
        const int hs = r >> 6, i = r & 63;
        const int h = h0 + hs;
        const bool row_ok = (hs == 0 || has_h1) && i < a.last_q;
        const int qpos = q_pos0 + i;                 // key c is visible iff c <= qpos
        const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
        const int tid = threadIdx.x - 64;            // 0..127
        const size_t bh = (size_t)b * a.hq + h;
        constexpr float kLog2e = 1.4426950408889634f;

        float row_m = -INFINITY, row_l = 0.f;
        if (PASS == 2 && row_ok) {
            // combine the per-chunk statistics of pass 1 in chunk order
            const float2* st = a.stats + (bh * 64 + i) * a.chunks_total;
            for (int c = 0; c < a.chunks_total; ++c) row_m = fmaxf(row_m, st[c].x);
            for (int c = 0; c < a.chunks_total; ++c)
                if (st[c].y > 0.f) row_l += st[c].y * exp2f((st[c].x - row_m) * kLog2e);
        }
        const float inv_l = (PASS == 2 && row_l > 0.f) ? 1.f / row_l : 0.f;

        bool ok = true;
        for (int it = 0; it < ntiles && ok; ++it) {
            const int s = it & 1, use = it >> 1;
            const int l0 = (tile_lo + it) * kEstTileN;   // first key of the tile inside the local keys
            const int c0 = a.col_base + l0;              // and its position in the sequence
            ok = mbar_wait(bar(&ctl->s_full[s]), use & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            // only the tiles that reach the last queries' diagonal or the end of the keys need masks
            const bool plain = row_ok && c0 + kEstTileN - 1 <= q_pos0 && l0 + kEstTileN <= a.n_k;
#pragma unroll 1
            for (int q4 = 0; q4 < 4; ++q4) {
                uint32_t xr[32];
                tmem_ld32(tmem + s * 128 + q4 * 32 + lane_base, xr);
                tmem_wait_ld();
                float x[32];
                float mx = -INFINITY;
                if (plain) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        logits_pair(xr[j], xr[j + 1], a.inv_sqrt_d_div, a.rcp_sqrt_d, x[j], x[j + 1]);
                        mx = max3(mx, x[j], x[j + 1]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float v0, v1;
                        logits_pair(xr[j], xr[j + 1], a.inv_sqrt_d_div, a.rcp_sqrt_d, v0, v1);
                        const int c = c0 + q4 * 32 + j;
                        x[j] = (row_ok && c <= qpos && l0 + q4 * 32 + j < a.n_k) ? v0 : -INFINITY;
                        x[j + 1] = (row_ok && c + 1 <= qpos && l0 + q4 * 32 + j + 1 < a.n_k) ? v1 : -INFINITY;
                        mx = max3(mx, x[j], x[j + 1]);
                    }
                }
                if (PASS == 1) {
                    if (mx > row_m) {
                        row_l *= exp2f((row_m - mx) * kLog2e);   // 0 * exp2(-inf) = 0 on the first hit
                        row_m = mx;
                    }
                    if (row_m > -INFINITY) {
                        const float neg = -row_m * kLog2e;
                        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int j = 0; j < 32; ++j) part[j & 3] += exp2f(fmaf(x[j], kLog2e, neg));
                        row_l += (part[0] + part[1]) + (part[2] + part[3]);
                    }
                } else {
                    const float neg = -row_m * kLog2e;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        ptile[r * kEstPitch + q4 * 32 + j] = row_ok ? exp2f(fmaf(x[j], kLog2e, neg)) * inv_l : 0.f;
                }
            }
            tc_fence_before();
            mbar_arrive(bar(&ctl->s_empty[s]));
            if (PASS == 2) {
                named_bar_sync(1, 128);
                // vertical: column sums over the 64 rows of each head, fixed order
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    if (hh == 1 && !has_h1) break;
                    const int c = c0 + tid;
                    if (l0 + tid < a.n_k) {
                        float sum = 0.f;
                        for (int ii = 0; ii < 64; ++ii) sum += ptile[(hh * 64 + ii) * kEstPitch + tid];
                        a.vertical[((size_t)b * a.hq + h0 + hh) * a.n_ctx + c] = sum;
                    }
                    // slash: d = i - j in [-127, 63]; offset = q_start - c0 + d
                    for (int d = tid - 127; d <= 63; d += 128) {
                        const int off = q_pos0 - c0 + d;
                        if (off < 0 || off >= a.n_ctx) continue;
                        float sum = 0.f;
                        const int i_lo = max(0, d), i_hi = min(63, 127 + d);
                        for (int ii = i_lo; ii <= i_hi; ++ii) sum += ptile[(hh * 64 + ii) * kEstPitch + (ii - d)];
                        if (sum != 0.f) atomicAdd(a.slash + ((size_t)b * a.hq + h0 + hh) * a.n_ctx + off, sum);
                    }
                }
                named_bar_sync(1, 128);
            }
        }
        if (PASS == 1 && ok && row_ok && ntiles > 0)
            a.stats[(bh * 64 + i) * a.chunks_total + a.chunk_offset + chunk] = make_float2(row_m, row_l);
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && ctl->abort) atomicOr(a.status + MINF_ST_ERROR, 1);
    if (warp == 1) tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------ top-k
struct SelectArgs {
    int batch_heads, n_ctx;
    const float* vertical;
    const float* slash;
    const int32_t* vertical_size;   // per head budgets before clamping
    const int32_t* slash_size;
    int cap_v, cap_s;
    int32_t* v_idx;
    int32_t* s_idx;
    int32_t* nnz_v;
    int32_t* nnz_s;
};

constexpr int kSelThreads = 1024;

// value of element `pos` in iteration order, with the forced +inf entries applied
//   vertical: pos = key index, first 30 forced          (minference_forward.py:608)
//   slash:    pos = N-1-offset (the reference's order), offsets < 100 forced (:612)
__device__ __forceinline__ uint32_t sel_key(const float* src, int pos, int n, bool is_slash) {
    if (is_slash) {
        const int off = n - 1 - pos;
        return off < 100 ? 0x7f800000u : __float_as_uint(src[off]);
    }
    return pos < 30 ? 0x7f800000u : __float_as_uint(src[pos]);
}

__global__ void __launch_bounds__(kSelThreads) vs_select_kernel(const SelectArgs a) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t sh_prefix, sh_remaining;
    __shared__ int scan_tmp[32];
    __shared__ int sh_base;

    const int bh = blockIdx.x;
    const bool is_slash = blockIdx.y == 1;
    const int n = a.n_ctx;
    const float* src = (is_slash ? a.slash : a.vertical) + (size_t)bh * n;
    const int budget = is_slash ? a.slash_size[bh] : a.vertical_size[bh];
    const int cap = is_slash ? a.cap_s : a.cap_v;
    if (budget < 0) {   // head not estimated (another pattern owns it)
        if (threadIdx.x == 0) (is_slash ? a.nnz_s : a.nnz_v)[bh] = -1;
        return;
    }
    int k = min(n, max(budget, is_slash ? 50 : 30));    // minference_forward.py:600
    k = min(k, cap);
    int32_t* out = (is_slash ? a.s_idx : a.v_idx) + (size_t)bh * cap;
    if (threadIdx.x == 0) (is_slash ? a.nnz_s : a.nnz_v)[bh] = k;

    // ---- radix select of the k-th largest key (scores are >= 0, so uint order == float order)
    uint32_t prefix = 0, prefix_mask = 0;
    uint32_t remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int pos = threadIdx.x; pos < n; pos += blockDim.x) {
            const uint32_t key = sel_key(src, pos, n, is_slash);
            if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t rem = remaining;
            int d = 255;
            for (; d > 0; --d) {
                if (hist[d] >= rem) break;
                rem -= hist[d];
            }
            sh_prefix = prefix | ((uint32_t)d << shift);
            sh_remaining = rem;
        }
        __syncthreads();
        prefix = sh_prefix;
        remaining = sh_remaining;
        prefix_mask |= 255u << shift;
        __syncthreads();
    }
    const uint32_t thr = prefix;         // k-th largest key
    const int ties_needed = (int)remaining;  // how many keys equal to thr are taken

    // number of keys equal to thr (to apply the tie rule in iteration order)
    __shared__ int sh_ties_total;
    if (threadIdx.x == 0) sh_ties_total = 0;
    __syncthreads();
    {
        int local = 0;
        for (int pos = threadIdx.x; pos < n; pos += blockDim.x) local += sel_key(src, pos, n, is_slash) == thr;
        for (int o = 16; o; o >>= 1) local += __shfl_down_sync(0xffffffffu, local, o);
        if ((threadIdx.x & 31) == 0 && local) atomicAdd(&sh_ties_total, local);
    }
    __syncthreads();
    // vertical: ties taken from the lowest key index: the first `ties_needed` in order.
    // slash: order is ascending N-1-offset, i.e. descending offset; smallest offsets win, so the
    //        first (ties_total - ties_needed) ties in this order are skipped.
    const int ties_skip = is_slash ? sh_ties_total - ties_needed : 0;

    // ---- ordered compaction
    if (threadIdx.x == 0) sh_base = 0;
    int ties_seen_base = 0;   // ties before the current block of positions (uniform)
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int start = 0; start < n; start += kSelThreads) {
        const int pos = start + threadIdx.x;
        const uint32_t key = pos < n ? sel_key(src, pos, n, is_slash) : 0u;
        const int is_tie = pos < n && key == thr;
        // rank of this tie among all ties in order
        const unsigned tb = __ballot_sync(0xffffffffu, is_tie);
        if (lane == 0) scan_tmp[warp] = __popc(tb);
        __syncthreads();
        int tie_rank = ties_seen_base + __popc(tb & ((1u << lane) - 1u));
        int block_ties = 0;
        for (int w = 0; w < kSelThreads / 32; ++w) {
            const int c = scan_tmp[w];
            if (w < warp) tie_rank += c;
            block_ties += c;
        }
        __syncthreads();
        const int take = pos < n && (key > thr || (is_tie && tie_rank >= ties_skip && tie_rank < ties_skip + ties_needed));
        const unsigned kb = __ballot_sync(0xffffffffu, take);
        if (lane == 0) scan_tmp[warp] = __popc(kb);
        __syncthreads();
        int dst = sh_base + __popc(kb & ((1u << lane) - 1u));
        int block_take = 0;
        for (int w = 0; w < kSelThreads / 32; ++w) {
            const int c = scan_tmp[w];
            if (w < warp) dst += c;
            block_take += c;
        }
        if (take && dst < cap) out[dst] = is_slash ? (n - 1 - pos) : pos;
        __syncthreads();
        if (threadIdx.x == 0) sh_base += block_take;
        ties_seen_base += block_ties;
        __syncthreads();
    }
    for (int i = k + threadIdx.x; i < cap; i += blockDim.x) out[i] = 0;
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_tmap_bhnd(CUtensorMap* tm, const void* base, int batch, int heads, int tokens, const int64_t st[3],
                   int box_rows, const char* what);   // defined in sparse_attn_fwd.cu

static void est_geometry(int n_ctx, int* tiles, int* chunks, int* tiles_per_chunk, int pair_ctas) {
    *tiles = (n_ctx + kEstTileN - 1) / kEstTileN;
    // about four waves of CTAs over 148 SMs, at least 4 tiles per CTA
    int want = (4 * 148 + pair_ctas - 1) / pair_ctas;
    if (want < 1) want = 1;
    int tpc = (*tiles + want - 1) / want;
    if (tpc < 4) tpc = 4;
    *tiles_per_chunk = tpc;
    *chunks = (*tiles + tpc - 1) / tpc;
}

}  // namespace minf

using namespace minf;

extern "C" int minf_vs_scores_chunks(int batch, int hq, int hkv, int n_k) {
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || n_k < 1) return 0;
    int tiles, chunks, tpc;
    est_geometry(n_k, &tiles, &chunks, &tpc, hkv * ((hq / hkv + 1) / 2) * batch);
    return chunks;
}

extern "C" int minf_vs_scores_pass(
    int pass, const void* q_last, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int n_k, int col_base, int head_dim,
    void* stats, int chunk_offset, int chunks_total, float* vertical_scores, float* slash_scores,
    int32_t* status, void* stream) {
    if (!q_last || !k || !stats || !status || (pass == 2 && (!vertical_scores || !slash_scores)))
        return fail(MINF_E_ARG, "null pointer argument");
    if (pass != 1 && pass != 2) return fail(MINF_E_ARG, "pass must be 1 or 2");
    if (head_dim != 128) return fail(MINF_E_UNSUPPORTED, "head_dim must be 128 (got %d)", head_dim);
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || context_size < 1 || batch > 65535 || n_k < 1 ||
        col_base < 0 || col_base + n_k > context_size)
        return fail(MINF_E_ARG, "bad sizes");
    EstArgs a{};
    a.batch = batch; a.hq = hq; a.hkv = hkv; a.n_ctx = context_size;
    a.last_q = context_size < 64 ? context_size : 64;
    a.n_k = n_k; a.col_base = col_base;
    a.group = hq / hkv;
    a.pairs_per_group = (a.group + 1) / 2;
    est_geometry(n_k, &a.tiles, &a.chunks, &a.tiles_per_chunk, hkv * a.pairs_per_group * batch);
    if (chunk_offset < 0 || chunk_offset + a.chunks > chunks_total) return fail(MINF_E_ARG, "chunk window outside the statistics array");
    a.chunk_offset = chunk_offset; a.chunks_total = chunks_total;
    a.stats = static_cast<float2*>(stats);
    a.vertical = vertical_scores; a.slash = slash_scores;
    a.inv_sqrt_d_div = sqrtf((float)head_dim);
    a.rcp_sqrt_d = 1.0f / a.inv_sqrt_d_div;
    a.status = status;
    CUtensorMap tq, tk;
    int rc;
    if ((rc = make_tmap_bhnd(&tq, q_last, batch, hq, a.last_q, q_strides, 64, "q_last"))) return rc;
    if ((rc = make_tmap_bhnd(&tk, k, batch, hkv, n_k, k_strides, 128, "k"))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = (pass == 1 ? est_ctl_off<1>() : est_ctl_off<2>()) + sizeof(EstControl);
    dim3 grid(a.chunks, hkv * a.pairs_per_group, batch);
    if (pass == 1) {
        MINF_CUDA_OK(cudaFuncSetAttribute(vs_scores_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        vs_scores_kernel<1><<<grid, 192, smem, st>>>(tq, tk, a);
    } else {
        MINF_CUDA_OK(cudaFuncSetAttribute(vs_scores_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        vs_scores_kernel<2><<<grid, 192, smem, st>>>(tq, tk, a);
    }
    MINF_LAUNCH_OK("vs_scores_kernel");
    return MINF_OK;
}

extern "C" int minf_vs_select(
    const float* vertical_scores, const float* slash_scores, int batch, int hq, int context_size,
    const int32_t* vertical_size, const int32_t* slash_size, int cap_v, int cap_s,
    int32_t* v_idx_out, int32_t* s_idx_out, int32_t* nnz_v_out, int32_t* nnz_s_out, void* stream) {
    if (!vertical_scores || !slash_scores || !vertical_size || !slash_size || !v_idx_out || !s_idx_out || !nnz_v_out || !nnz_s_out)
        return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || hq < 1 || context_size < 1 || cap_v < 1 || cap_s < 1) return fail(MINF_E_ARG, "bad sizes");
    SelectArgs s{};
    s.batch_heads = batch * hq; s.n_ctx = context_size;
    s.vertical = vertical_scores; s.slash = slash_scores;
    s.vertical_size = vertical_size; s.slash_size = slash_size;
    s.cap_v = cap_v; s.cap_s = cap_s;
    s.v_idx = v_idx_out; s.s_idx = s_idx_out; s.nnz_v = nnz_v_out; s.nnz_s = nnz_s_out;
    vs_select_kernel<<<dim3(batch * hq, 2), kSelThreads, 0, static_cast<cudaStream_t>(stream)>>>(s);
    MINF_LAUNCH_OK("vs_select_kernel");
    return MINF_OK;
}

extern "C" size_t minf_vs_estimate_scratch_bytes(int batch, int hq, int context_size) {
    if (batch < 1 || hq < 1 || context_size < 1) return 0;
    // chunk count is at most the number of tiles; use that bound so the size does not depend on hkv
    const size_t tiles = (size_t)(context_size + kEstTileN - 1) / kEstTileN;
    const size_t max_chunks = tiles < 4 * 148 ? tiles : 4 * 148;
    size_t bytes = (size_t)batch * hq * 64 * max_chunks * sizeof(float2);
    bytes = (bytes + 255) / 256 * 256;
    bytes += 2 * (size_t)batch * hq * context_size * sizeof(float);   // score arrays when the caller passes none
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
    const int chunks = minf_vs_scores_chunks(batch, hq, hkv, context_size);
    unsigned char* sc = static_cast<unsigned char*>(scratch);
    size_t off = (size_t)batch * hq * 64 * chunks * sizeof(float2);
    off = (off + 255) / 256 * 256;
    float* vertical = vertical_scores_out ? vertical_scores_out : reinterpret_cast<float*>(sc + off);
    float* slash = slash_scores_out ? slash_scores_out
                                    : reinterpret_cast<float*>(sc + off) + (size_t)batch * hq * context_size;
    // the last min(64, N) queries, viewed in place
    const int last_q = context_size < 64 ? context_size : 64;
    const void* q_last = static_cast<const __nv_bfloat16*>(q) + (size_t)(context_size - last_q) * q_strides[2];
    MINF_CUDA_OK(cudaMemsetAsync(slash, 0, (size_t)batch * hq * context_size * sizeof(float), st));
    int rc;
    for (int pass = 1; pass <= 2; ++pass)
        if ((rc = minf_vs_scores_pass(pass, q_last, k, q_strides, k_strides, batch, hq, hkv, context_size, context_size, 0,
                                      head_dim, sc, 0, chunks, vertical, slash, status, stream)))
            return rc;
    return minf_vs_select(vertical, slash, batch, hq, context_size, vertical_size, slash_size, cap_v, cap_s,
                          v_idx_out, s_idx_out, nnz_v_out, nnz_s_out, stream);
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
// at zero (the diagonal-score accumulators) are cleared on the stream before the kernels run, as in
// the buffer-taking entry point.  Two calls whose kernels may overlap on the same GPU (different
// streams, or different host threads) would use the same scratch at once: that is a data race the
// caller must exclude.  The first call on a device performs the one-time address lookup and
// should therefore be made outside any stream capture.
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
