// Attention plan from a block mask: for every head a square 0/1 matrix over blocks of `block_tokens` tokens
// (a multiple of 64), entry (i, j) set <=> query block i attends key block j, causal inside every block.
// This is the index set of the reference's FlexPrefill path (modules/flexprefill.py:903-927 builds it as
// flattened block ids, :353-495 walks them per query block); here it becomes the merged [start, end) token
// ranges per 64-row block that the attention kernel reads, so runs of neighbouring key blocks are streamed
// as one range and nothing is gathered.
//
// One warp per 64-row block: the row of the mask is read 32 key blocks at a time, a ballot turns them into
// a bit word, and the runs of ones are cut out of the words with bit scans (every lane computes the same,
// lane 0 writes).  A range is clipped at the last row of its row block: keys beyond it are in the future.
#include "common.h"
#include "plan_layout.h"

namespace minf {

constexpr int kMaskPlanWarps = 8;

struct MaskPlanArgs {
    const uint8_t* mask;      // [batch*heads, nb, nb]
    int rows;                 // 64-row blocks of the sequence
    int nb;                   // blocks per side of the mask
    int rows_per_block;       // block_tokens / 64
    int block_tokens;
    unsigned char* plan;
    PlanLayout layout;
    int32_t* status;
};

__global__ void __launch_bounds__(kMaskPlanWarps * 32) block_mask_plan_kernel(const MaskPlanArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = blockIdx.x * kMaskPlanWarps + warp;
    if (m >= a.rows) return;
    const size_t bh = blockIdx.y;
    const int i = m / a.rows_per_block;                       // block row of the mask
    const uint8_t* row = a.mask + (bh * a.nb + i) * (size_t)a.nb;
    unsigned char* slot = a.plan + bh * a.layout.head_bytes;
    int2* rng = reinterpret_cast<int2*>(slot + a.layout.rng_off) + plan_rng_offset(a.layout, m);
    const int cap = min(a.layout.cap_s, m + 2);
    const int limit = 64 * (m + 1);                           // first key no row of this row block can see

    int n = 0;
    bool overflow = false;
    int run_start = -1;                                       // open run: first key block, or -1
    auto emit = [&](int first_blk, int end_blk) {
        const int s = first_blk * a.block_tokens;
        const int e = min(end_blk * a.block_tokens, limit);
        if (s >= e) return;
        if (n < cap) {
            if (lane == 0 && MINF_IN_BOUNDS(a.status, n >= 0 && n < cap)) rng[n] = make_int2(s, e);
            ++n;
        } else {
            overflow = true;
        }
    };
    // four words of the row per round: the four loads are in flight together
    for (int j00 = 0; j00 <= i; j00 += 128) {
        unsigned char b4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j00 + 32 * u + lane;
            b4[u] = j <= i ? row[j] : (unsigned char)0;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j0 = j00 + 32 * u;
            if (j0 > i) break;
            const unsigned w = __ballot_sync(0xffffffffu, b4[u] != 0);
            int pos = 0;                                          // bits below pos are done
            while (pos < 32) {
                if (run_start < 0) {
                    const unsigned rest = pos ? (w >> pos) << pos : w;
                    if (rest == 0u) break;
                    pos = __ffs(rest) - 1;
                    run_start = j0 + pos;
                }
                // the run goes on from bit pos: find its first zero
                const unsigned zeros = ~w & (pos ? (0xffffffffu >> pos) << pos : 0xffffffffu);
                if (zeros == 0u) break;                           // runs to the end of this word
                pos = __ffs(zeros) - 1;
                emit(run_start, j0 + pos);
                run_start = -1;
            }
        }
    }
    if (run_start >= 0) emit(run_start, i + 1);
    if (lane == 0) {
        reinterpret_cast<int32_t*>(slot)[m] = n;
        if (overflow) atomicOr(a.status + MINF_ST_ERROR, 4);  // more runs than the plan was sized for
    }
    uint32_t* bits = reinterpret_cast<uint32_t*>(slot + a.layout.bits_off) + (size_t)m * a.layout.words_v;
    for (int w = lane; w < a.layout.words_v; w += 32) bits[w] = 0u;
}

}  // namespace minf

using namespace minf;

extern "C" int minf_block_mask_build_plan(
    const uint8_t* mask, int batch, int heads, int context_size, int block_tokens, int cap_s,
    void* plan, int32_t* status, void* stream) {
    if (!mask || !plan || !status) return fail(MINF_E_ARG, "null pointer argument");
    if (batch < 1 || heads < 1 || context_size < 1 || cap_s < 1 || (long long)batch * heads > 65535)
        return fail(MINF_E_ARG, "bad sizes");
    if (block_tokens < 64 || block_tokens % 64) return fail(MINF_E_ARG, "block_tokens must be a multiple of 64 (got %d)", block_tokens);
    MaskPlanArgs a{};
    a.mask = mask;
    a.rows = (context_size + 63) / 64;
    a.nb = (context_size + block_tokens - 1) / block_tokens;
    a.rows_per_block = block_tokens / 64;
    a.block_tokens = block_tokens;
    a.plan = static_cast<unsigned char*>(plan);
    a.layout = make_plan_layout(context_size, 0, cap_s);
    a.status = status;
    dim3 grid((a.rows + kMaskPlanWarps - 1) / kMaskPlanWarps, batch * heads);
    block_mask_plan_kernel<<<grid, kMaskPlanWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
    MINF_LAUNCH_OK("block_mask_plan_kernel");
    return MINF_OK;
}
