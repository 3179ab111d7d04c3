// Block-sparse index estimation: top-k key blocks per 64-row query block from mean-pooled
// Q and K.  Replaces _build_block_index (ops/block_sparse_flash_attention.py:151-166 of the
// reference: reshape+mean, a [rows, rows] einsum, block-causal mask, torch.topk, sort) and the
// padding rule of its caller (:178: the sequence is padded by 64 - (N & 63) rows, a whole
// extra block of zeros when N is a multiple of 64).
//
//   pool kernel    one warp per (tensor, batch, head, block): fp32 mean of up to 64 rows,
//                  rounded to bf16 like the reference's bf16 mean.  HBM-bound: reads Q and K once.
//   select kernel  one CTA per (batch, head, four query blocks): scores of key blocks 0..m (fp32
//                  dot of the pooled bf16 vectors, rounded to bf16 like the reference's bf16
//                  einsum; every pooled key row is fetched once for the four query blocks) as
//                  16-bit keys in shared memory, then per query block a radix select of the
//                  k-th largest (two 8-bit passes) and an ordered compaction.  Equal scores at the threshold: lowest block index first
//                  (torch.topk leaves this unspecified).  Writes the reference-format sorted
//                  block ids and/or the merged token ranges of the attention plan.
#include <cuda_bf16.h>

#include "common.h"
#include "plan_layout.h"

namespace minf {

struct PoolArgs {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    long long q_sb, q_sh, q_sn, k_sb, k_sh, k_sn;
    int batch, hq, hkv, n_ctx, rows_pad;
    __nv_bfloat16* qpool;   // [batch, hq, rows_pad, 128]
    __nv_bfloat16* kpool;   // [batch, hkv, rows_pad, 128]
};

__global__ void __launch_bounds__(256) bs_pool_kernel(const PoolArgs a) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const long long nq = (long long)a.batch * a.hq * a.rows_pad;
    const long long nk = (long long)a.batch * a.hkv * a.rows_pad;
    if (warp >= nq + nk) return;
    const bool is_k = warp >= nq;
    const long long id = is_k ? warp - nq : warp;
    const int heads = is_k ? a.hkv : a.hq;
    const int m = (int)(id % a.rows_pad);
    const int h = (int)((id / a.rows_pad) % heads);
    const int b = (int)(id / ((long long)a.rows_pad * heads));
    const __nv_bfloat16* src = is_k ? a.k + b * a.k_sb + h * a.k_sh : a.q + b * a.q_sb + h * a.q_sh;
    const long long sn = is_k ? a.k_sn : a.q_sn;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int r_hi = min(64 * m + 64, a.n_ctx);
    for (int r = 64 * m; r < r_hi; ++r) {     // padded rows are zeros: they only count in the divisor
        const uint2 raw = *reinterpret_cast<const uint2*>(src + r * sn + 4 * lane);
        const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        acc[0] += __bfloat162float(p0.x); acc[1] += __bfloat162float(p0.y);
        acc[2] += __bfloat162float(p1.x); acc[3] += __bfloat162float(p1.y);
    }
    __nv_bfloat16* dst = (is_k ? a.kpool : a.qpool) + id * 128 + 4 * lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = __float2bfloat16_rn(acc[i] * (1.f / 64.f));
}

struct BsSelectArgs {
    const __nv_bfloat16* qpool;
    const __nv_bfloat16* kpool;
    int batch, hq, hkv, n_ctx, rows, rows_pad, top_k;   // top_k already clamped to rows_pad
    const int32_t* head_select;
    int32_t* block_index;    // optional [batch, hq, rows_pad, top_k]
    unsigned char* plan;     // optional
    PlanLayout layout;
    int m_base;              // query block of blockIdx.x = 0 (sequence-sharded callers plan a window of query blocks)
    int rows_q;              // query blocks held by qpool per head (rows_pad for a whole sequence)
    int rows_per_cta;        // 8, or 4 when eight rows of keys do not fit shared memory
};

constexpr int kBsRowsMax = 8;  // query blocks per CTA (4 or 8: what fits shared memory), one warp each in the select phase

// order-preserving map of a bf16 value (held in a float) to 16 bits: negative values have all bits flipped,
// the others the sign bit set, so unsigned comparison of the keys is comparison of the values
__device__ __forceinline__ uint32_t bf16_key(float x) {
    const uint32_t u = __float_as_uint(x) >> 16;
    return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
}

__global__ void __launch_bounds__(256) bs_select_kernel(const BsSelectArgs a) {
    extern __shared__ uint16_t keys16[];      // [rows_per_cta][rows_pad] score keys
    __shared__ float qv[4][128];
    __shared__ uint32_t hist[8][256];         // one histogram per warp

    const int h = blockIdx.y, b = blockIdx.z;
    if (a.head_select && a.head_select[h] == 0) return;
    const int hk = h / (a.hq / a.hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t bh = (size_t)b * a.hq + h;
    const int m_loc0 = blockIdx.x * a.rows_per_cta;           // first query block of this CTA (inside qpool / the plan)
    const int nr = min(a.rows_per_cta, a.rows_q - m_loc0);

    // ---- scores, four query blocks at a time: key blocks 0..m of the last of them against all four; four key blocks
    // per warp step, eight lanes (16 of the 128 dimensions each) per key block; fp32 dot products rounded to bf16 like
    // the reference's bf16 einsum.  Every pooled key row is fetched once per four query blocks.
    const __nv_bfloat16* kp = a.kpool + ((size_t)b * a.hkv + hk) * a.rows_pad * 128;
    for (int r0 = 0; r0 < nr; r0 += 4) {
        const int nq = min(4, nr - r0);
        __syncthreads();
        for (int i = threadIdx.x; i < 4 * 128; i += 256) {
            const int r = i >> 7;
            qv[r][i & 127] = r < nq ? __bfloat162float(a.qpool[(bh * a.rows_q + m_loc0 + r0 + r) * 128 + (i & 127)]) : 0.f;
        }
        __syncthreads();
        const int n_max = a.m_base + m_loc0 + r0 + nq;
        const int sub = lane >> 3, part = lane & 7;
        float q[4][16];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int i = 0; i < 16; ++i) q[r][i] = qv[r][16 * part + i];
#pragma unroll 2
        for (int n0 = warp * 4; n0 < n_max; n0 += 32) {      // two steps in flight: the loads of the second overlap the first
            const int n = n0 + sub;
            uint4 raw[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
            if (n < n_max) {
                const uint4* src = reinterpret_cast<const uint4*>(kp + (size_t)n * 128 + 16 * part);
                raw[0] = src[0];
                raw[1] = src[1];
            }
            const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(raw);
            float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 kf = __bfloat1622float2(k2[i]);
#pragma unroll
                for (int r = 0; r < 4; ++r) s[r] = fmaf(q[r][2 * i + 1], kf.y, fmaf(q[r][2 * i], kf.x, s[r]));
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                s[r] += __shfl_xor_sync(0xffffffffu, s[r], 4);
                s[r] += __shfl_xor_sync(0xffffffffu, s[r], 2);
                s[r] += __shfl_xor_sync(0xffffffffu, s[r], 1);
            }
            if (part == 0 && n < n_max) {
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (r < nq) keys16[(size_t)(r0 + r) * a.rows_pad + n] = (uint16_t)bf16_key(__bfloat162float(__float2bfloat16_rn(s[r])));
            }
        }
    }
    __syncthreads();

    // ---- selection: warp r takes query block r; nothing below synchronises across warps
    const int r = warp;
    if (r >= nr) return;
    const int m_loc = m_loc0 + r;
    const int m = a.m_base + m_loc;           // position of the query block in the sequence
    const int n_blocks = m + 1;               // causal key blocks 0..m
    const int k = min(a.top_k, n_blocks);     // blocks the attention kernel consumes (:81)
    const uint16_t* keys = keys16 + (size_t)r * a.rows_pad;
    uint32_t* myhist = hist[warp];
    const unsigned lt = (1u << lane) - 1u;

    uint32_t thr = 0;
    int ties_needed = 0;
    if (k < n_blocks) {                       // radix select of the k-th largest key, two 8-bit digits
        uint32_t prefix = 0, prefix_mask = 0, remaining = k;
        for (int shift = 8; shift >= 0; shift -= 8) {
#pragma unroll
            for (int i = 0; i < 8; ++i) myhist[8 * lane + i] = 0u;
            __syncwarp();
            // scores of one head lie close together, so most keys of a warp step share the digit: one
            // shared-memory atomic per distinct digit instead of one per key
            for (int base = 0; base < n_blocks; base += 32) {
                const int n = base + lane;
                const bool act = n < n_blocks && ((uint32_t)keys[n] & prefix_mask) == prefix;
                const uint32_t digit = act ? ((uint32_t)keys[n] >> shift) & 255u : 0xffffffffu;
                const unsigned peers = __match_any_sync(0xffffffffu, digit);
                if (act && lane == __ffs(peers) - 1) atomicAdd(&myhist[digit], (uint32_t)__popc(peers));
            }
            __syncwarp();
            // the highest digit at which the count from the top reaches `remaining`: lane l holds digits 8l..8l+7
            uint32_t c[8], mine = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { c[i] = myhist[8 * lane + i]; mine += c[i]; }
            uint32_t above = mine;            // inclusive suffix sum over lanes, then made exclusive
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_down_sync(0xffffffffu, above, o);
                if (lane + o < 32) above += t;
            }
            above -= mine;
            const bool here = above < remaining && remaining <= above + mine;
            const unsigned where = __ballot_sync(0xffffffffu, here);
            int d = 0;
            uint32_t rem = remaining;
            if (here) {
                uint32_t cum = above;
                d = 8 * lane;
                rem = remaining - above;
#pragma unroll
                for (int i = 7; i >= 0; --i) {
                    if (cum + c[i] >= remaining) { d = 8 * lane + i; rem = remaining - cum; break; }
                    cum += c[i];
                }
            }
            if (where) {
                const int src = __ffs(where) - 1;
                d = __shfl_sync(0xffffffffu, d, src);
                rem = __shfl_sync(0xffffffffu, rem, src);
            }                                 // (a lane always finds it: at least `remaining` keys match the prefix)
            prefix |= (uint32_t)d << shift;
            remaining = rem;
            prefix_mask |= 255u << shift;
            __syncwarp();
        }
        thr = prefix;
        ties_needed = (int)remaining;
    }

    // ordered compaction of the selected block ids (ascending), 32 candidates per step
    int32_t* bi = a.block_index ? a.block_index + (bh * a.rows_pad + m) * a.top_k : nullptr;
    int2* rng = nullptr;
    if (a.plan && m < a.rows)
        rng = reinterpret_cast<int2*>(a.plan + bh * a.layout.head_bytes + a.layout.rng_off) + plan_rng_offset(a.layout, m_loc);
    int taken = 0, ties_seen = 0, nrng = 0;
    int cur_lo = -1, cur_hi = -1;
    for (int base = 0; base < n_blocks; base += 32) {
        const int n = base + lane;
        const bool in = n < n_blocks;
        const uint32_t key = in ? keys[n] : 0u;
        const bool tie = in && k < n_blocks && key == thr;
        const unsigned tb = __ballot_sync(0xffffffffu, tie);
        const int tie_rank = ties_seen + __popc(tb & lt);
        const bool take = in && (k >= n_blocks || key > thr || (tie && tie_rank < ties_needed));
        unsigned word = __ballot_sync(0xffffffffu, take);
        if (take && bi) bi[taken + __popc(word & lt)] = n;
        taken += __popc(word);
        ties_seen += __popc(tb);
        if (rng) {
            while (word) {                    // runs of ones, cut out of the ballot word with bit scans (every lane alike)
                const int lo = __ffs(word) - 1;
                const unsigned inv = ~(word >> lo);
                const int len = inv ? __ffs(inv) - 1 : 32 - lo;
                const int first = (base + lo) * 64;
                if (first == cur_hi) cur_hi += 64 * len;
                else {
                    if (cur_lo >= 0) { if (lane == 0) rng[nrng] = make_int2(cur_lo, cur_hi); ++nrng; }
                    cur_lo = first; cur_hi = first + 64 * len;
                }
                word = lo + len >= 32 ? 0u : word & ~((1u << (lo + len)) - 1u);
            }
        }
    }
    if (rng) {
        if (cur_lo >= 0) { if (lane == 0) rng[nrng] = make_int2(cur_lo, cur_hi); ++nrng; }
        if (lane == 0) reinterpret_cast<int32_t*>(a.plan + bh * a.layout.head_bytes)[m_loc] = nrng;
    }
    if (a.plan && m < a.rows) {
        uint32_t* wb = reinterpret_cast<uint32_t*>(a.plan + bh * a.layout.head_bytes + a.layout.bits_off) + (size_t)m_loc * a.layout.words_v;
        for (int w = lane; w < a.layout.words_v; w += 32) wb[w] = 0u;
    }
    // tail of the reference-format row: the reference holds arbitrary masked block ids there
    // (ties among -inf scores); the first causally masked ids in ascending order are used here
    if (bi) {
        for (int j = k + lane; j < a.top_k; j += 32) bi[j] = min(n_blocks + (j - k), a.rows_pad - 1);
    }
}

}  // namespace minf

using namespace minf;

static int bs_rows_pad(int n) { return (n + (64 - (n & 63))) / 64; }

extern "C" size_t minf_block_sparse_scratch_bytes(int batch, int hq, int hkv, int context_size) {
    if (batch < 1 || hq < 1 || hkv < 1 || context_size < 1) return 0;
    return (size_t)batch * (hq + hkv) * bs_rows_pad(context_size) * 128 * sizeof(__nv_bfloat16) + 256;
}

extern "C" int minf_block_sparse_build_plan(
    const void* q, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim, int top_k,
    const int32_t* head_select, int cap_v, int cap_s, void* plan, int32_t* block_index_out,
    void* scratch, int32_t* status, void* stream) {
    (void)status;
    if (!q || !k || !scratch || (!plan && !block_index_out)) return fail(MINF_E_ARG, "null pointer argument");
    if (head_dim != 128) return fail(MINF_E_UNSUPPORTED, "head_dim must be 128 (got %d)", head_dim);
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || context_size < 1 || top_k < 1 || batch > 65535 || hq > 65535)
        return fail(MINF_E_ARG, "bad sizes");
    const int rows_pad = bs_rows_pad(context_size);
    const int k_eff = top_k < rows_pad ? top_k : rows_pad;
    if (plan && cap_s < k_eff) return fail(MINF_E_ARG, "cap_s=%d is smaller than top_k=%d", cap_s, k_eff);
    if ((size_t)rows_pad * 2 * 4 > 200 * 1024) return fail(MINF_E_UNSUPPORTED, "context too long for the block score buffer");
    for (int i = 0; i < 3; ++i)
        if (q_strides[i] % 4 || k_strides[i] % 4) return fail(MINF_E_ARG, "strides must be multiples of 4 elements");
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    PoolArgs p{};
    p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k);
    p.q_sb = q_strides[0]; p.q_sh = q_strides[1]; p.q_sn = q_strides[2];
    p.k_sb = k_strides[0]; p.k_sh = k_strides[1]; p.k_sn = k_strides[2];
    p.batch = batch; p.hq = hq; p.hkv = hkv; p.n_ctx = context_size; p.rows_pad = rows_pad;
    p.qpool = static_cast<__nv_bfloat16*>(scratch);
    p.kpool = p.qpool + (size_t)batch * hq * rows_pad * 128;
    const long long warps = (long long)batch * (hq + hkv) * rows_pad;
    bs_pool_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(p);
    MINF_LAUNCH_OK("bs_pool_kernel");

    BsSelectArgs s{};
    s.qpool = p.qpool; s.kpool = p.kpool;
    s.batch = batch; s.hq = hq; s.hkv = hkv; s.n_ctx = context_size;
    s.rows = (context_size + 63) / 64; s.rows_pad = rows_pad; s.top_k = k_eff;
    s.head_select = head_select;
    s.block_index = block_index_out;
    s.plan = static_cast<unsigned char*>(plan);
    s.layout = make_plan_layout(context_size, cap_v, cap_s);
    s.m_base = 0; s.rows_q = rows_pad;
    s.rows_per_cta = (size_t)rows_pad * 2 * kBsRowsMax <= 100 * 1024 ? kBsRowsMax : 4;
    const size_t smem = (size_t)rows_pad * s.rows_per_cta * sizeof(uint16_t);
    MINF_CUDA_OK(cudaFuncSetAttribute(bs_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    bs_select_kernel<<<dim3((rows_pad + s.rows_per_cta - 1) / s.rows_per_cta, hq, batch), 256, smem, st>>>(s);
    MINF_LAUNCH_OK("bs_select_kernel");
    return MINF_OK;
}

extern "C" int minf_block_sparse_pool(
    const void* x, const int64_t strides[3], int batch, int heads, int n_rows, void* pooled, void* stream) {
    if (!x || !strides || !pooled) return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || heads < 1 || n_rows < 1) return fail(MINF_E_ARG, "bad sizes");
    for (int i = 0; i < 3; ++i)
        if (strides[i] % 4) return fail(MINF_E_ARG, "strides must be multiples of 4 elements");
    PoolArgs p{};
    p.q = static_cast<const __nv_bfloat16*>(x); p.k = nullptr;
    p.q_sb = strides[0]; p.q_sh = strides[1]; p.q_sn = strides[2];
    p.batch = batch; p.hq = heads; p.hkv = 0; p.n_ctx = n_rows; p.rows_pad = (n_rows + 63) / 64;
    p.qpool = static_cast<__nv_bfloat16*>(pooled); p.kpool = nullptr;
    const long long warps = (long long)batch * heads * p.rows_pad;
    bs_pool_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    MINF_LAUNCH_OK("bs_pool_kernel");
    return MINF_OK;
}

extern "C" int minf_block_sparse_select_window(
    const void* q_pooled, const void* k_pooled, int batch, int hq, int hkv, int context_size,
    int q_pos0, int n_q, int top_k, const int32_t* head_select, int cap_v, int cap_s, void* plan, void* stream) {
    if (!q_pooled || !k_pooled || !plan) return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || context_size < 1 || top_k < 1 || batch > 65535 || hq > 65535)
        return fail(MINF_E_ARG, "bad sizes");
    if (q_pos0 < 0 || (q_pos0 % 64) || n_q < 1 || q_pos0 + n_q > context_size) return fail(MINF_E_ARG, "bad query window");
    const int rows_k = (context_size + 63) / 64;
    const int rows_loc = (n_q + 63) / 64;
    const int k_eff = top_k < bs_rows_pad(context_size) ? top_k : bs_rows_pad(context_size);
    if (cap_s < k_eff) return fail(MINF_E_ARG, "cap_s=%d is smaller than top_k=%d", cap_s, k_eff);
    if ((size_t)rows_k * 2 * 4 > 200 * 1024) return fail(MINF_E_UNSUPPORTED, "context too long for the block score buffer");
    BsSelectArgs s{};
    s.qpool = static_cast<const __nv_bfloat16*>(q_pooled); s.kpool = static_cast<const __nv_bfloat16*>(k_pooled);
    s.batch = batch; s.hq = hq; s.hkv = hkv; s.n_ctx = context_size;
    s.rows = rows_k; s.rows_pad = rows_k; s.top_k = k_eff;
    s.head_select = head_select;
    s.block_index = nullptr;
    s.plan = static_cast<unsigned char*>(plan);
    s.layout = make_plan_layout_window(q_pos0 / 64, rows_loc, cap_v, cap_s);
    s.m_base = q_pos0 / 64; s.rows_q = rows_loc;
    s.rows_per_cta = (size_t)rows_k * 2 * kBsRowsMax <= 100 * 1024 ? kBsRowsMax : 4;
    const size_t smem = (size_t)rows_k * s.rows_per_cta * sizeof(uint16_t);
    MINF_CUDA_OK(cudaFuncSetAttribute(bs_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    bs_select_kernel<<<dim3((rows_loc + s.rows_per_cta - 1) / s.rows_per_cta, hq, batch), 256, smem, static_cast<cudaStream_t>(stream)>>>(s);
    MINF_LAUNCH_OK("bs_select_kernel");
    return MINF_OK;
}
