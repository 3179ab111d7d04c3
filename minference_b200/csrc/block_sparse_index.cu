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
};

constexpr int kBsRows = 4;     // query blocks per CTA: every pooled key row is fetched once for all of them

// order-preserving map of a bf16 value (held in a float) to 16 bits: negative values have all bits flipped,
// the others the sign bit set, so unsigned comparison of the keys is comparison of the values
__device__ __forceinline__ uint32_t bf16_key(float x) {
    const uint32_t u = __float_as_uint(x) >> 16;
    return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
}

__global__ void __launch_bounds__(256) bs_select_kernel(const BsSelectArgs a) {
    extern __shared__ uint16_t keys16[];      // [kBsRows][rows_pad] score keys
    __shared__ float qv[kBsRows][128];
    __shared__ uint32_t hist[256];
    __shared__ uint32_t sh_prefix, sh_remaining;
    __shared__ int warp_cnt[8];
    __shared__ int sh_base, sh_ties;
    __shared__ unsigned take_word[8];

    const int h = blockIdx.y, b = blockIdx.z;
    if (a.head_select && a.head_select[h] == 0) return;
    const int hk = h / (a.hq / a.hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t bh = (size_t)b * a.hq + h;
    const int m_loc0 = blockIdx.x * kBsRows;                  // first query block of this CTA (inside qpool / the plan)
    const int nr = min(kBsRows, a.rows_q - m_loc0);

    for (int i = threadIdx.x; i < kBsRows * 128; i += 256) {
        const int r = i >> 7;
        qv[r][i & 127] = r < nr ? __bfloat162float(a.qpool[(bh * a.rows_q + m_loc0 + r) * 128 + (i & 127)]) : 0.f;
    }
    __syncthreads();

    // ---- scores of key blocks 0..m of the CTA's last query block against all its query blocks: four key blocks per
    // warp step, eight lanes (16 of the 128 dimensions each) per key block; fp32 dot products rounded to bf16 like the
    // reference's bf16 einsum
    {
        const int n_max = a.m_base + m_loc0 + nr;
        const int sub = lane >> 3, part = lane & 7;
        float q[kBsRows][16];
#pragma unroll
        for (int r = 0; r < kBsRows; ++r)
#pragma unroll
            for (int i = 0; i < 16; ++i) q[r][i] = qv[r][16 * part + i];
        const __nv_bfloat16* kp = a.kpool + ((size_t)b * a.hkv + hk) * a.rows_pad * 128;
        for (int n0 = warp * 4; n0 < n_max; n0 += 32) {
            const int n = n0 + sub;
            uint4 raw[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
            if (n < n_max) {
                const uint4* src = reinterpret_cast<const uint4*>(kp + (size_t)n * 128 + 16 * part);
                raw[0] = src[0];
                raw[1] = src[1];
            }
            const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(raw);
            float s[kBsRows];
#pragma unroll
            for (int r = 0; r < kBsRows; ++r) s[r] = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 kf = __bfloat1622float2(k2[i]);
#pragma unroll
                for (int r = 0; r < kBsRows; ++r) s[r] = fmaf(q[r][2 * i + 1], kf.y, fmaf(q[r][2 * i], kf.x, s[r]));
            }
#pragma unroll
            for (int r = 0; r < kBsRows; ++r) {
                s[r] += __shfl_xor_sync(0xffffffffu, s[r], 4);
                s[r] += __shfl_xor_sync(0xffffffffu, s[r], 2);
                s[r] += __shfl_xor_sync(0xffffffffu, s[r], 1);
            }
            if (part == 0 && n < n_max) {
#pragma unroll
                for (int r = 0; r < kBsRows; ++r)
                    if (r < nr) keys16[(size_t)r * a.rows_pad + n] = (uint16_t)bf16_key(__bfloat162float(__float2bfloat16_rn(s[r])));
            }
        }
    }
    __syncthreads();

    for (int r = 0; r < nr; ++r) {
        const int m_loc = m_loc0 + r;
        const int m = a.m_base + m_loc;           // position of the query block in the sequence
        const int n_blocks = m + 1;               // causal key blocks 0..m
        const int k = min(a.top_k, n_blocks);     // blocks the attention kernel consumes (:81)
        const uint16_t* keys = keys16 + (size_t)r * a.rows_pad;

        uint32_t thr = 0;
        int ties_needed = 0;
        if (k < n_blocks) {
            uint32_t prefix = 0, prefix_mask = 0, remaining = k;
            for (int shift = 8; shift >= 0; shift -= 8) {
                hist[threadIdx.x] = 0;
                __syncthreads();
                // scores of one head lie close together, so most keys of a warp share the digit: one shared-memory
                // atomic per distinct digit of the warp instead of one per key
                for (int base = warp * 32; base < n_blocks; base += 256) {
                    const int n = base + lane;
                    const bool act = n < n_blocks && ((uint32_t)keys[n] & prefix_mask) == prefix;
                    const uint32_t digit = act ? ((uint32_t)keys[n] >> shift) & 255u : 0xffffffffu;
                    const unsigned peers = __match_any_sync(0xffffffffu, digit);
                    if (act && lane == __ffs(peers) - 1) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
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
            thr = prefix;
            ties_needed = (int)remaining;
        }

        // ordered compaction of the selected block ids (ascending), 256 candidates per round
        int32_t* bi = a.block_index ? a.block_index + (bh * a.rows_pad + m) * a.top_k : nullptr;
        int2* rng = nullptr;
        if (a.plan && m < a.rows)
            rng = reinterpret_cast<int2*>(a.plan + bh * a.layout.head_bytes + a.layout.rng_off) + plan_rng_offset(a.layout, m_loc);
        if (threadIdx.x == 0) { sh_base = 0; sh_ties = 0; }
        __syncthreads();
        int nrng = 0;          // maintained by thread 0 only
        int cur_lo = -1, cur_hi = -1;
        for (int start = 0; start < n_blocks; start += 256) {
            const int n = start + threadIdx.x;
            const bool in = n < n_blocks;
            const uint32_t key = in ? keys[n] : 0u;
            const bool tie = in && k < n_blocks && key == thr;
            const unsigned tb = __ballot_sync(0xffffffffu, tie);
            if (lane == 0) warp_cnt[warp] = __popc(tb);
            __syncthreads();
            int tie_rank = sh_ties + __popc(tb & ((1u << lane) - 1u));
            int round_ties = 0;
            for (int w = 0; w < 8; ++w) { if (w < warp) tie_rank += warp_cnt[w]; round_ties += warp_cnt[w]; }
            __syncthreads();
            const bool take = in && (k >= n_blocks || key > thr || (tie && tie_rank < ties_needed));
            const unsigned kb = __ballot_sync(0xffffffffu, take);
            if (lane == 0) warp_cnt[warp] = __popc(kb);
            __syncthreads();
            int dst = sh_base + __popc(kb & ((1u << lane) - 1u));
            int round_take = 0;
            for (int w = 0; w < 8; ++w) { if (w < warp) dst += warp_cnt[w]; round_take += warp_cnt[w]; }
            if (take && bi) bi[dst] = n;
            if (lane == 0) take_word[warp] = kb;     // staged so thread 0 can merge adjacent blocks into ranges
            __syncthreads();
            if (threadIdx.x == 0) {
                sh_base += round_take;
                sh_ties += round_ties;
                if (rng) {
                    for (int w = 0; w < 8; ++w) {    // runs of ones, cut out of the ballot words with bit scans
                        unsigned word = take_word[w];
                        while (word) {
                            const int lo = __ffs(word) - 1;
                            const unsigned inv = ~(word >> lo);
                            const int len = inv ? __ffs(inv) - 1 : 32 - lo;
                            const int first = (start + 32 * w + lo) * 64;
                            if (first == cur_hi) cur_hi += 64 * len;
                            else {
                                if (cur_lo >= 0) rng[nrng++] = make_int2(cur_lo, cur_hi);
                                cur_lo = first; cur_hi = first + 64 * len;
                            }
                            word = lo + len >= 32 ? 0u : word & ~((1u << (lo + len)) - 1u);
                        }
                    }
                }
            }
            __syncthreads();
        }
        if (threadIdx.x == 0 && rng) {
            if (cur_lo >= 0) rng[nrng++] = make_int2(cur_lo, cur_hi);
            reinterpret_cast<int32_t*>(a.plan + bh * a.layout.head_bytes)[m_loc] = nrng;
        }
        if (a.plan && m < a.rows) {
            uint32_t* wb = reinterpret_cast<uint32_t*>(a.plan + bh * a.layout.head_bytes + a.layout.bits_off) + (size_t)m_loc * a.layout.words_v;
            for (int w = threadIdx.x; w < a.layout.words_v; w += blockDim.x) wb[w] = 0u;
        }
        // tail of the reference-format row: the reference holds arbitrary masked block ids there
        // (ties among -inf scores); the first causally masked ids in ascending order are used here
        if (bi) {
            for (int j = k + threadIdx.x; j < a.top_k; j += blockDim.x) bi[j] = min(n_blocks + (j - k), a.rows_pad - 1);
        }
        __syncthreads();
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
    if ((size_t)rows_pad * 2 * kBsRows > 200 * 1024) return fail(MINF_E_UNSUPPORTED, "context too long for the block score buffer");
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
    const size_t smem = (size_t)rows_pad * kBsRows * sizeof(uint16_t);
    MINF_CUDA_OK(cudaFuncSetAttribute(bs_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    bs_select_kernel<<<dim3((rows_pad + kBsRows - 1) / kBsRows, hq, batch), 256, smem, st>>>(s);
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
    if ((size_t)rows_k * 2 * kBsRows > 200 * 1024) return fail(MINF_E_UNSUPPORTED, "context too long for the block score buffer");
    BsSelectArgs s{};
    s.qpool = static_cast<const __nv_bfloat16*>(q_pooled); s.kpool = static_cast<const __nv_bfloat16*>(k_pooled);
    s.batch = batch; s.hq = hq; s.hkv = hkv; s.n_ctx = context_size;
    s.rows = rows_k; s.rows_pad = rows_k; s.top_k = k_eff;
    s.head_select = head_select;
    s.block_index = nullptr;
    s.plan = static_cast<unsigned char*>(plan);
    s.layout = make_plan_layout_window(q_pos0 / 64, rows_loc, cap_v, cap_s);
    s.m_base = q_pos0 / 64; s.rows_q = rows_loc;
    const size_t smem = (size_t)rows_k * kBsRows * sizeof(uint16_t);
    MINF_CUDA_OK(cudaFuncSetAttribute(bs_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    bs_select_kernel<<<dim3((rows_loc + kBsRows - 1) / kBsRows, hq, batch), 256, smem, static_cast<cudaStream_t>(stream)>>>(s);
    MINF_LAUNCH_OK("bs_select_kernel");
    return MINF_OK;
}
