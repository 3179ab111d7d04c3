// Sparse flash-attention forward for sm_100a: tcgen05 MMA with TMEM accumulators, TMA tile
// loads for contiguous key ranges, cp.async gathers for vertical columns.
//
// One CTA owns 256 consecutive query rows of one head (4 row blocks of 64, the granularity at
// which the reference defines its index set, ops/pit_sparse_flash_attention_v2.py:64-153) as two
// 128-row slots.  Warp roles (three warpgroups of four warps):
//   warp 0          producer: merges the plans of the four row blocks into one stream of steps.
//                   A step is 64 or 128 keys -- a contiguous token range (TMA) or gathered
//                   vertical columns (cp.async) -- with a 128-bit key mask per row block.
//                   K and V travel through separate rings so a K stage is recycled as soon as
//                   both QK^T products have read it.
//   warp 1          issues every tcgen05.mma and tcgen05.commit (the whole warp follows the control
//                   flow, one lane elected per instruction) and owns the TMEM allocation
//   warp 2          copies the V rows of gathered steps (the producer copies their K rows)
//   warp 3          spare (keeps the roles aligned to warpgroups of four; setmaxnreg hands the
//                   registers of warps 0-3 to the softmax warps)
//   warps 4-7/8-11  softmax of slot 0 / slot 1, one thread per query row, the whole 128-key row
//                   of S in registers
// TMEM (512 columns): per slot 128 columns of O and 128 columns of S.  P (bf16) is written back
// over the first half of S and feeds the PV product straight from TMEM, so it never touches
// shared memory.  The two slots alternate: while one slot's softmax runs, the tensor pipe
// executes the other slot's PV and next QK^T.  CTAs are ordered one KV head at a time (its query
// heads and all their 256-row items, most work first) so that the CTAs in flight share K/V in L2.
// status[2..3] (one uint64) counts the 64x64 tile equivalents sent to the tensor pipe.
//
// Positions are global token positions throughout; `q_pos0` / `kv_pos0` say where the local Q
// and K/V tensors sit in the sequence, so the same kernel serves a whole sequence on one GPU
// (both zero) and one (query chunk, key chunk) pair of a sequence-sharded ring step, where keys
// outside the local chunk are left to another step and the partial results are merged through
// the per-row log-sum-exp written to `lse`.
//
// Semantics kept from the reference kernels: causal mask inside contiguous tiles, none in the
// gathered-column loop, keys >= context masked, fp32 accumulation, P rounded to bf16,
// 1/sqrt(d) scale applied with exp2.  A row with no visible key yields zeros (lse = -inf).
// The running maximum is only raised when it grows by more than 2^8, so the O rescale in TMEM
// is rare.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>

#include "common.h"
#include "plan_layout.h"
#include "sm100_ptx.cuh"

namespace minf {

constexpr int kHeadDim = 128;
constexpr int kNK = 2, kNV = 3, kNM = 8;           // K stages, V stages, step-descriptor ring
constexpr uint32_t kTile = 128 * 256;              // 128 rows x 128 bf16
constexpr uint32_t kQOff = 0;
constexpr uint32_t kKOff = 2 * kTile;
constexpr uint32_t kVOff = kKOff + kNK * kTile;
constexpr uint32_t kCtlOff = kVOff + kNV * kTile;

enum StepKind : int { kTileStep = 0, kGatherStep = 1, kEndStep = 2 };

struct alignas(16) Step {
    int kind;
    int t;        // first key (global position) of a contiguous tile
    int width;    // 64 or 128 keys
    int parts;    // bit s set <=> query slot s has a visible key in this step
    unsigned long long mask[4][2];   // per row block: visible keys (bit i of word w = key 64*w + i)
};

struct Control {
    unsigned long long q_full;
    unsigned long long k_full[kNK], k_empty[kNK], v_full[kNV], v_empty[kNV];
    unsigned long long m_full[kNM], m_empty[kNM];
    unsigned long long s_full[2], p_half[2][2], o_done[2];   // P is published in two halves per step
    uint32_t tmem_base;
    int abort;
    Step step[kNM];
    int colring[512];               // gathered columns waiting for a step: (row-block bits << 28) | position
    int4 gmsg[2];                   // planner -> V-gather warp, alternating: (step, first ring entry, count, 0); count 0 = done
};
static_assert(kCtlOff + sizeof(Control) <= 232448, "shared memory of one CTA");

struct AttnArgs {
    __nv_bfloat16* o;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    float* lse;                       // optional [batch, hq, n_q], base-2 log-sum-exp of the scaled logits
    float* o_acc;                     // optional carry [batch, hq, n_q, 128] fp32: merged, normalised output so far
    float* lse_acc;                   // its log-sum-exp [batch, hq, n_q]; -inf = nothing accumulated yet
    long long o_sb, o_sh, o_sn;
    long long k_sb, k_sh, k_sn;
    long long v_sb, v_sh, v_sn;
    int batch, hq, hkv;
    int n_ctx;                        // length of the whole sequence
    int n_q, q_pos0;                  // local query rows and the position of the first one
    int n_kv, kv_pos0;                // local keys and the position of the first one
    float scale_log2;                 // sm_scale * log2(e)
    const int32_t* head_mode;
    const int32_t* head_param;
    const unsigned char* plan;        // covers the row blocks of the local queries
    PlanLayout layout;
    const int32_t* v_idx;
    int cap_v;
    int items_per_head;
    int32_t* status;
};

struct Maps {
    CUtensorMap q, k64, k128, v64, v128;
};

// Cursor over the merged ranges of one row block, clipped to the local key window; 32 ranges
// are buffered across the warp.
struct RangeCursor {
    const int2* rng;
    int n, ri, base;
    int2 buf;
    int a, b;
    int last_row, kv_lo, kv_hi;
    int floor_end;      // end of the previous range: a plan whose ranges are not ascending and disjoint is refused
    bool bad;
    __device__ __forceinline__ void fetch(int lane) {
        for (;;) {
            if (ri >= n) { a = INT32_MAX; b = INT32_MAX; return; }
            if (ri - base >= 32 || ri < base) {
                base = ri;
                buf = (base + lane < n) ? rng[base + lane] : make_int2(INT32_MAX, INT32_MAX);
            }
            const int ra = __shfl_sync(0xffffffffu, buf.x, ri - base);
            const int rb = __shfl_sync(0xffffffffu, buf.y, ri - base);
            if (ra < floor_end || rb <= ra) {    // not a plan this library wrote: stop here instead of wandering
                bad = true; ri = n; a = INT32_MAX; b = INT32_MAX;
                return;
            }
            floor_end = rb;
            a = max(ra, kv_lo);
            b = min(rb, kv_hi);
            if (a < b || a >= kv_hi) return;     // usable, or everything from here on lies past the window
            ++ri;                                // range entirely before the window
        }
    }
    __device__ __forceinline__ void init(const int2* r, int count, int first, int last, int lo, int hi, int lane) {
        rng = r; n = count; ri = first; base = -64; last_row = last; kv_lo = lo; kv_hi = hi;
        floor_end = INT32_MIN; bad = false;
        fetch(lane);
    }
    __device__ __forceinline__ bool live() const { return ri < n && a <= last_row && a < kv_hi; }
};

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ unsigned long long below64(int x) {   // bits [0, x) for any integer x
    return x >= 64 ? ~0ull : (x <= 0 ? 0ull : ((1ull << x) - 1ull));
}
// bits [lo, hi) of a 128-bit mask are added to (w0, w1)
__device__ __forceinline__ void span128(int lo, int hi, unsigned long long& w0, unsigned long long& w1) {
    w0 |= below64(hi) & ~below64(lo);
    w1 |= below64(hi - 64) & ~below64(lo - 64);
}
// keys 0..lim visible (lim may be negative or >= 127)
__device__ __forceinline__ void upto128(int lim, unsigned long long& w0, unsigned long long& w1) {
    w0 = below64(lim + 1);
    w1 = below64(lim + 1 - 64);
}

// One softmax step of one query row: S (fp32, NCH*32 columns at t_s) -> P (bf16 pairs written
// back over the first NCH*16 columns).  The whole row is held in registers, so TMEM is read
// once.  m0/m1 hold the visibility bits of keys 0-63 / 64-127.
// (Skipping the exponentials of a 32- or 64-key part that no row of the warp can see -- the other row
// block's half of an isolated diagonal -- was built and measured in two forms: it changed nothing on
// scattered index sets, whose steps are bound by the softmax -> PV -> QK^T chain of a slot and not by the
// MUFU, and it cost 4 % on dense ones, so every chunk is processed.  Taking a quarter or half of the
// exponentials from a cubic on the FMA pipe (packed two-wide arithmetic, exponent written by an integer add)
// was measured as well: 1 % and 9 % slower on dense index sets, 9 % and 17 % on scattered ones -- the cubic's
// ten instructions per key pair cost a softmax warp more time than the two MUFU operations they replace.)
template <int NCH>
__device__ __forceinline__ void softmax_row(uint32_t t_s, uint32_t t_o, unsigned long long m0, unsigned long long m1,
                                            float scale_log2, bool have_o, float& m_ref, float& l_sum,
                                            uint32_t bar_half0, uint32_t bar_half1) {
    // The row maximum of a chunk is taken while the next chunk's load is in flight.
    uint32_t sr[NCH][32];
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    tmem_ld32(t_s, sr[0]);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        tmem_wait_ld();
        if (c + 1 < NCH) tmem_ld32(t_s + 32 * (c + 1), sr[c + 1]);
        const uint32_t cm = (uint32_t)((c < 2 ? m0 : m1) >> (32 * (c & 1)));
        if (cm != 0xffffffffu) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (!((cm >> i) & 1u)) sr[c][i] = 0xff800000u;   // -inf
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2)
            mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
    }
    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
    float alpha = 1.f;
    if (mx > m_ref + 8.f) {          // raise the reference maximum only on a jump of more than 2^8
        alpha = fast_exp2(m_ref - mx);
        l_sum *= alpha;
        m_ref = mx;
    }
    const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
    // O of this slot is at rest here: the QK^T that filled S was issued after the previous PV
    if (have_o && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            uint32_t orow[32];
            tmem_ld32(t_o + 32 * c, orow);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
            tmem_st32(t_o + 32 * c, orow);
        }
    }
    // P = 2^(S*scale - m): scale and subtract two keys per instruction, exponentials on the MUFU.
    // The first half of the keys is published on its own barrier so that the PV product can
    // start on it while the second half is still being exponentiated.
    const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2), negm2 = pack_f32x2(neg_m, neg_m);
    uint64_t ps2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float x0, x1;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), scale2, negm2), x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            ps2[(i >> 1) & 3] = add_f32x2(ps2[(i >> 1) & 3], pack_f32x2(p0, p1));
            pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st16(t_s + 16 * c, pk);
        if (c == NCH / 2 - 1) {
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_half0);
        }
    }
    float a0, a1;
    unpack_f32x2(add_f32x2(add_f32x2(ps2[0], ps2[1]), add_f32x2(ps2[2], ps2[3])), a0, a1);
    l_sum += a0 + a1;
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(bar_half1);
}

// One warp copies `width` gathered rows (256 B each) of K or V into a 128-byte-swizzled stage: lanes 0-15 fetch the
// sixteen 16-byte pieces of one row, lanes 16-31 those of the next; col[q] holds this lane's row index for rows
// 32q + lane.  The copies are asynchronous; the caller arrives on the stage barrier with cp_async_arrive_noinc.
__device__ __forceinline__ void gather_rows(uint32_t dst, const __nv_bfloat16* base, long long row_stride,
                                            const int (&col)[4], int width, int lane) {
    const int chunk = lane & 15, sub = lane >> 4;
    const uint32_t half_off = (uint32_t)(chunk >> 3) * 16384u;                  // which 64-column half of the stage
    const char* src0 = reinterpret_cast<const char*>(base + chunk * 8);
    const long long stride_b = row_stride * 2;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (32 * q >= width) break;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
            const int rr = 2 * i + sub;
            const int c = __shfl_sync(0xffffffffu, col[q], rr);
            const int r = 32 * q + rr;
            cp_async_16(dst + half_off + (uint32_t)r * 128u + (uint32_t)(((chunk ^ r) & 7) << 4), src0 + (long long)c * stride_b);
        }
    }
}

__global__ void __launch_bounds__(384, 1)
sparse_attn_fwd_kernel(const __grid_constant__ Maps tm, const AttnArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    Control* ctl = reinterpret_cast<Control*>(smem + kCtlOff);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Block order: one KV head at a time (its query heads and all their items, latest rows = most
    // work first), so that the CTAs in flight stream the same K/V and find it in L2; the K and V
    // of one KV head at 131072 tokens are 64 MB, half of L2.
    const int group = a.hq / a.hkv;
    const int per_kv = a.items_per_head * group;
    const int kv_slot = (int)(blockIdx.x / per_kv), rem = (int)(blockIdx.x % per_kv);
    const int item = a.items_per_head - 1 - rem / group;
    const int b = kv_slot / a.hkv, h = (kv_slot % a.hkv) * group + rem % group;
    const int bh = b * a.hq + h;
    const int hk = h / (a.hq / a.hkv);
    const int rb_loc0 = item * 4;                   // first row block of the item inside the local queries
    const int lrow0 = rb_loc0 * 64;                 // first local query row
    const int row0 = a.q_pos0 + lrow0;              // its position in the sequence
    const int rows_loc = (a.n_q + 63) / 64;         // row blocks covered by the plan
    const int kv_lo = a.kv_pos0, kv_hi = a.kv_pos0 + a.n_kv;

    // an earlier CTA gave up: leave at once (decision made by one thread so it is uniform)
    if (__syncthreads_or(threadIdx.x == 0 && *(volatile int32_t*)(a.status + MINF_ST_ERROR) != 0)) return;
    if ((smem_base & 1023u) != 0u) {
        if (threadIdx.x == 0) atomicOr(a.status + MINF_ST_ERROR, 2);
        return;
    }
    const int mode = a.head_mode ? a.head_mode[h] : MINF_MODE_PLAN;
    const int n_init = mode == MINF_MODE_ASHAPE ? a.head_param[2 * h] : 0;
    const int n_local = mode == MINF_MODE_ASHAPE ? a.head_param[2 * h + 1] : 0;

    auto bar = [&](const unsigned long long* p) { return smem_u32(p); };
    volatile int* abort_flag = &ctl->abort;

    if (threadIdx.x == 0) {
        mbar_init(bar(&ctl->q_full), 1);
        // a stage is full when all 32 producer lanes have arrived: at once for a TMA tile (lane 0 adds the byte
        // count), each lane as its own copies land for a gathered one
        for (int s = 0; s < kNK; ++s) { mbar_init(bar(&ctl->k_full[s]), 32); mbar_init(bar(&ctl->k_empty[s]), 1); }
        for (int s = 0; s < kNV; ++s) { mbar_init(bar(&ctl->v_full[s]), 32); mbar_init(bar(&ctl->v_empty[s]), 1); }
        for (int s = 0; s < kNM; ++s) { mbar_init(bar(&ctl->m_full[s]), 1); mbar_init(bar(&ctl->m_empty[s]), 9); }   // MMA lane + 8 softmax warps
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(&ctl->s_full[s]), 1);
            mbar_init(bar(&ctl->p_half[s][0]), 128);
            mbar_init(bar(&ctl->p_half[s][1]), 128);
            mbar_init(bar(&ctl->o_done[s]), 1);
        }
        ctl->abort = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&ctl->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        if (lane == 0) {
            tma_prefetch_desc(&tm.q); tma_prefetch_desc(&tm.k64); tma_prefetch_desc(&tm.k128);
            tma_prefetch_desc(&tm.v64); tma_prefetch_desc(&tm.v128);
            mbar_arrive_expect_tx(bar(&ctl->q_full), 2 * kTile);
            for (int s = 0; s < 2; ++s) {
                tma_load_4d(smem_base + kQOff + s * kTile, &tm.q, bar(&ctl->q_full), 0, lrow0 + 128 * s, h, b);
                tma_load_4d(smem_base + kQOff + s * kTile + 16384, &tm.q, bar(&ctl->q_full), 64, lrow0 + 128 * s, h, b);
            }
        }
        int step = 0;
        int n_gather = 0;              // gather steps handed to the V-gather warp so far
        unsigned issued = 0;           // 64x64 tile equivalents this CTA sends to the tensor pipe
        bool ok = true;
        bool bad_plan = false;         // the plan of this head cannot have been written by the plan builders
        auto wait_use = [&](unsigned long long* bars, int ring, int idx) -> bool {
            const int s = idx % ring, use = idx / ring;
            if (use > 0 && !mbar_wait(bar(&bars[s]), (use - 1) & 1, abort_flag)) { ok = false; return false; }
            return true;
        };
        auto publish = [&](int kind, int t, int width, const unsigned long long (&mk)[4][2]) -> bool {
            if (!wait_use(ctl->m_empty, kNM, step)) return false;
            if (lane == 0) {
                Step& st = ctl->step[step % kNM];
                const int parts = ((mk[0][0] | mk[0][1] | mk[1][0] | mk[1][1]) != 0ull ? 1 : 0) |
                                  ((mk[2][0] | mk[2][1] | mk[3][0] | mk[3][1]) != 0ull ? 2 : 0);
                *reinterpret_cast<int4*>(&st) = make_int4(kind, t, width, parts);
                issued += (unsigned)(__popc(parts) * (width >> 5));     // a slot is two row blocks tall
#pragma unroll
                for (int r = 0; r < 4; ++r)       // one 16-byte store per row block
                    *reinterpret_cast<ulonglong2*>(&st.mask[r][0]) = make_ulonglong2(mk[r][0], mk[r][1]);
                mbar_arrive(bar(&ctl->m_full[step % kNM]));
            }
            return true;
        };
        auto load_tile = [&](int t, int width) -> bool {     // t: global position, inside the local key window
            const int lt = t - a.kv_pos0;
            if (!MINF_IN_BOUNDS(a.status, lt >= 0 && lt < a.n_kv)) return true;      // a tile that starts outside the local keys
            if (!wait_use(ctl->k_empty, kNK, step)) return false;
            {
                const uint32_t fb = bar(&ctl->k_full[step % kNK]);
                if (lane == 0) {
                    const uint32_t dst = smem_base + kKOff + (step % kNK) * kTile;
                    mbar_arrive_expect_tx(fb, width * 256);
                    const CUtensorMap* m = width == 128 ? &tm.k128 : &tm.k64;
                    tma_load_4d(dst, m, fb, 0, lt, hk, b);
                    tma_load_4d(dst + 16384, m, fb, 64, lt, hk, b);
                } else {
                    mbar_arrive(fb);
                }
            }
            if (!wait_use(ctl->v_empty, kNV, step)) return false;
            {
                const uint32_t fb = bar(&ctl->v_full[step % kNV]);
                if (lane == 0) {
                    const uint32_t dst = smem_base + kVOff + (step % kNV) * kTile;
                    mbar_arrive_expect_tx(fb, width * 256);
                    const CUtensorMap* m = width == 128 ? &tm.v128 : &tm.v64;
                    tma_load_4d(dst, m, fb, 0, lt, hk, b);
                    tma_load_4d(dst + 16384, m, fb, 64, lt, hk, b);
                } else {
                    mbar_arrive(fb);
                }
            }
            return true;
        };

        if (mode == MINF_MODE_ASHAPE) {
            const int r_hi = min(row0 + 256, a.q_pos0 + a.n_q) - 1;
            int w0 = row0 - n_local + 1;
            w0 = w0 < 0 ? 0 : (w0 & ~63);
            const bool sinks = a.n_ctx > n_local && r_hi >= n_local;
            const int sink_end = sinks ? min(min(n_init, w0), a.n_ctx) : 0;
            for (int phase = 0; phase < 2 && ok; ++phase) {
                // sink tiles [0, sink_end), then window tiles [w0, r_hi], both clipped to the local keys
                const int t_lo = max(phase == 0 ? 0 : w0, kv_lo);
                const int t_hi = min(phase == 0 ? sink_end : r_hi + 1, kv_hi);
                for (int t = t_lo; t < t_hi && ok;) {
                    const int width = (t_hi - t > 64) ? 128 : 64;
                    // a row block takes part only if one of its rows can see a key of the tile: the
                    // tile starts at or before its last row and reaches its window (or holds sinks)
                    unsigned long long mk[4][2];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int first = row0 + 64 * r, last = first + 63;
                        const bool sees = last >= t && (phase == 0 || t + width - 1 >= first - n_local + 1 ||
                                                        (a.n_ctx > n_local && t < n_init));
                        mk[r][0] = sees ? ~0ull : 0ull;
                        mk[r][1] = sees ? ~0ull : 0ull;
                    }
                    if (!publish(kTileStep, t, width, mk)) break;
                    if (!load_tile(t, width)) break;
                    ++step;
                    t += width;
                }
            }
        } else if (a.plan == nullptr) {
            bad_plan = true;           // a head in plan mode without a plan: no keys, reported below
        } else {
            const unsigned char* slot = a.plan + (size_t)bh * a.layout.head_bytes;
            const int32_t* rng_cnt = reinterpret_cast<const int32_t*>(slot);
            const int2* rng_all = reinterpret_cast<const int2*>(slot + a.layout.rng_off);
            RangeCursor cur[4];
            const int2* rp[4];
            int rn[4], first[4], hi_[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int ml = rb_loc0 + r;                       // row block inside the plan
                const bool present = ml < rows_loc;
                rp[r] = present ? rng_all + plan_rng_offset(a.layout, ml) : nullptr;
                rn[r] = present ? rng_cnt[ml] : 0;
                // a slot nobody wrote holds an arbitrary count: never walk past the slot's capacity
                const int cap = min(a.layout.cap_s, a.layout.rb_base + ml + 2);
                if (rn[r] < 0 || rn[r] > cap) { bad_plan = true; rn[r] = 0; }
                first[r] = 0; hi_[r] = rn[r];
            }
            if (kv_lo > 0) {
                // first range that ends after the start of the key window (ranges are ascending and
                // disjoint); the four searches advance together so their loads overlap
                bool more = true;
                while (more) {
                    more = false;
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        if (first[r] < hi_[r]) {
                            const int mid = (first[r] + hi_[r]) >> 1;
                            if (rp[r][mid].y <= kv_lo) first[r] = mid + 1; else hi_[r] = mid;
                            more = true;
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) cur[r].init(rp[r], rn[r], first[r], row0 + 64 * r + 63, kv_lo, kv_hi, lane);
            // ---- contiguous ranges, merged over the four row blocks
            while (ok) {
                int t = INT32_MAX;
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (cur[r].live()) t = min(t, cur[r].a);
                if (t == INT32_MAX) break;
                unsigned long long mk[4][2];
                unsigned long long any_hi = 0ull;
                // inside long ranges every live row block covers [t, t+128) entirely and runs on: no mask arithmetic
                bool whole = true;
                bool lv[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    lv[r] = cur[r].live();
                    whole = whole && (!lv[r] || (cur[r].a == t && cur[r].b > t + 128));
                }
                if (whole) {
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        mk[r][0] = mk[r][1] = lv[r] ? ~0ull : 0ull;
                        if (lv[r]) cur[r].a = t + 128;
                    }
                    any_hi = ~0ull;
                } else {
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        mk[r][0] = 0ull; mk[r][1] = 0ull;
                        while (cur[r].live() && cur[r].a < t + 128) {      // every range of the row block inside [t, t+128)
                            const int hi = min(cur[r].b, t + 128);
                            span128(cur[r].a - t, hi - t, mk[r][0], mk[r][1]);
                            if (cur[r].b <= t + 128) { ++cur[r].ri; cur[r].fetch(lane); }
                            else { cur[r].a = t + 128; break; }
                        }
                        any_hi |= mk[r][1];
                    }
                }
                const int width = any_hi ? 128 : 64;
                if (!publish(kTileStep, t, width, mk)) break;
                if (!load_tile(t, width)) break;
                ++step;
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) bad_plan = bad_plan || cur[r].bad;
            // ---- gathered columns: union of the row blocks' bit masks over the vertical list,
            //      restricted to columns inside the local key window
            const int words = a.layout.words_v;
            const uint32_t* bits = reinterpret_cast<const uint32_t*>(slot + a.layout.bits_off);
            const int32_t* vlist = a.v_idx ? a.v_idx + (size_t)bh * a.cap_v : nullptr;
            int filled = 0, emitted = 0;
            auto flush_chunk = [&](int count) {   // count <= 128 ring entries starting at `emitted`
                const int width = count > 64 ? 128 : 64;
                int e[4];
                bool val[4];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    val[q4] = lane + 32 * q4 < count;
                    e[q4] = ctl->colring[(emitted + 32 * q4 + lane) & 511];
                }
                unsigned long long mk[4][2];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    unsigned bl[4];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) bl[q4] = __ballot_sync(0xffffffffu, val[q4] && ((e[q4] >> (28 + r)) & 1));
                    mk[r][0] = (unsigned long long)bl[0] | ((unsigned long long)bl[1] << 32);
                    mk[r][1] = (unsigned long long)bl[2] | ((unsigned long long)bl[3] << 32);
                }
                // hand the step to the V-gather warp (warp 2) before any wait of this warp can fail: both meet at
                // named barrier 2 once per gather step and once more when the planner is done
                if (lane == 0) ctl->gmsg[n_gather & 1] = make_int4(step, emitted, count, 0);
                ++n_gather;
                named_bar_sync(2, 64);
                if (!publish(kGatherStep, 0, width, mk)) return;
                int col[4];      // local key rows
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    col[q4] = val[q4] ? (e[q4] & 0x0fffffff) - a.kv_pos0 : 0;
                    if (!MINF_IN_BOUNDS(a.status, col[q4] >= 0 && col[q4] < a.n_kv)) col[q4] = 0;
                }
                if (!wait_use(ctl->k_empty, kNK, step)) return;
                gather_rows(smem_base + kKOff + (step % kNK) * kTile, a.k + b * a.k_sb + hk * a.k_sh, a.k_sn, col, width, lane);
                cp_async_arrive_noinc(bar(&ctl->k_full[step % kNK]));      // each lane's K rows, whenever they land
                emitted += count;
                ++step;
            };
            for (int w = 0; w < words && ok; ++w) {
                uint32_t wr[4];
                uint32_t any = 0;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int ml = rb_loc0 + r;
                    wr[r] = ml < rows_loc ? bits[(size_t)ml * words + w] : 0u;
                    any |= wr[r];
                }
                if (any == 0u) continue;
                if (vlist == nullptr) { bad_plan = true; break; }     // columns marked but no vertical list given
                const int vi = 32 * w + lane;
                const int colv = (((any >> lane) & 1u) && vi < a.cap_v) ? vlist[vi] : -1;
                const unsigned sel = __ballot_sync(0xffffffffu, colv >= kv_lo && colv < kv_hi);
                if (sel == 0u) continue;
                const int pos = filled + __popc(sel & ((1u << lane) - 1u));
                if ((sel >> lane) & 1u) {
                    int e = colv & 0x0fffffff;
#pragma unroll
                    for (int r = 0; r < 4; ++r) e |= (int)((wr[r] >> lane) & 1u) << (28 + r);
                    ctl->colring[pos & 511] = e;
                }
                filled += __popc(sel);
                __syncwarp();
                if (filled - emitted >= 128) flush_chunk(128);
            }
            if (ok && filled > emitted) flush_chunk(filled - emitted);
        }
        if (lane == 0) ctl->gmsg[n_gather & 1] = make_int4(0, 0, 0, 0);      // no more gather steps
        named_bar_sync(2, 64);
        if (ok) {
            // the end marker travels like a step: the MMA warp reads a step's descriptor once the
            // step's K stage is full, so the marker completes a K stage too (with no load)
            const unsigned long long none[4][2] = {{0ull, 0ull}, {0ull, 0ull}, {0ull, 0ull}, {0ull, 0ull}};
            if (publish(kEndStep, 0, 0, none) && wait_use(ctl->k_empty, kNK, step))
                mbar_arrive(bar(&ctl->k_full[step % kNK]));          // all 32 lanes
        }
        if (lane == 0 && bad_plan) atomicOr(a.status + MINF_ST_ERROR, 4);
        if (lane == 0 && issued)
            atomicAdd(reinterpret_cast<unsigned long long*>(a.status + MINF_ST_AUX0), (unsigned long long)issued);
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        {   // the whole warp follows the control flow and computes the operands; one elected
            // lane issues each single-thread instruction (see elect_one)
            auto wait = [&](const unsigned long long* b, int parity) {
                return __all_sync(0xffffffffu, mbar_wait(bar(b), parity, abort_flag)) != 0;
            };
            bool ok = wait(&ctl->q_full, 0);
            // A step's descriptor is written by the producer before it completes the step's K
            // stage, so waiting for that stage also makes the descriptor visible; it is read once,
            // as one 16-byte word (kind, first key, width, live slots).
            auto read_step = [&](int j) { return *reinterpret_cast<const int4*>(&ctl->step[j % kNM]); };
            // Descriptor words: the high word (stride offset 1024 B, version 1, 128-byte swizzle) is
            // constant; the low word is (address >> 4) | (leading offset >> 4) << 16, so walking
            // along K is an integer add of a compile-time constant.
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
            auto issue_s = [&](int j, int slot, int width) {
                const uint32_t idesc = width == 128 ? umma_idesc(128, 128, true, false, false)
                                                    : umma_idesc(128, 64, true, false, false);
                const uint32_t d = tmem + slot * 256 + 128;
                const uint32_t a_lo = ((smem_base + kQOff + slot * kTile) >> 4) | (1u << 16);
                const uint32_t b_lo = ((smem_base + kKOff + (j % kNK) * kTile) >> 4) | (1u << 16);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint32_t adv = (kk >> 2) * (16384 >> 4) + (kk & 3) * (32 >> 4);
                        umma_ss(d, desc(a_lo + adv), desc(b_lo + adv), idesc, kk > 0);
                    }
                    umma_commit(bar(&ctl->s_full[slot]));
                }
            };
            int npv[2] = {0, 0};
            // PV product of one half of a step's keys (P arrives in two halves, see softmax_row)
            auto issue_pv_half = [&](int j, int kv, int slot, int width, int half) {
                constexpr uint32_t idesc = umma_idesc(128, 128, true, false, true);
                const uint32_t d = tmem + slot * 256;
                const uint32_t p = tmem + slot * 256 + 128;
                const uint32_t b_lo = ((smem_base + kVOff + kv * kTile) >> 4) | ((16384u >> 4) << 16);
                const uint32_t acc0 = (npv[slot] > 0 || half > 0) ? 1u : 0u;
                if (elect_one()) {
                    if (width == 128) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int kk = 4 * half + i;
                            umma_ts(d, p + kk * 8, desc(b_lo + kk * (2048 >> 4)), idesc, i > 0 ? 1u : acc0);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const int kk = 2 * half + i;
                            umma_ts(d, p + kk * 8, desc(b_lo + kk * (2048 >> 4)), idesc, i > 0 ? 1u : acc0);
                        }
                    }
                }
                if (half == 1) ++npv[slot];
            };

            // Steps are issued in order, slot 0 then slot 1: PV(s, j) as soon as P(s, j) is ready,
            // followed at once by QK^T(s, j+1) so that the slot's next softmax can start while
            // the other slot's products run.  Waits are blocking (the hardware suspends the
            // thread), which keeps this warp out of the issue slots of the softmax warps.
            int j = 0, kv = 0, kv_par = 0;         // kv = j % kNV and the parity of its use
            int4 cur = make_int4(kEndStep, 0, 0, 0);
            if (ok) ok = wait(&ctl->k_full[0], 0);
            if (ok) {
                fence_proxy_async_smem();      // rows gathered with cp.async were written through the generic proxy
                cur = read_step(0);
                if (cur.x != kEndStep) {
#pragma unroll
                    for (int s = 0; s < 2; ++s)
                        if ((cur.w >> s) & 1) issue_s(0, s, cur.z);
                    if (elect_one()) umma_commit(bar(&ctl->k_empty[0]));
                }
            }
            while (ok && cur.x != kEndStep) {
                ok = wait(&ctl->k_full[(j + 1) % kNK], ((j + 1) / kNK) & 1);
                if (!ok) break;
                const int4 nxt = read_step(j + 1);
                const bool nxt_live = nxt.x != kEndStep;
                ok = wait(&ctl->v_full[kv], kv_par);
                if (!ok) break;
                fence_proxy_async_smem();      // gathered stages: generic-proxy writes before the tensor pipe reads them
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    if ((cur.w >> s) & 1) {
                        ok = wait(&ctl->p_half[s][0], npv[s] & 1);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv_half(j, kv, s, cur.z, 0);
                        ok = wait(&ctl->p_half[s][1], npv[s] & 1);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv_half(j, kv, s, cur.z, 1);
                    }
                    if (nxt_live && ((nxt.w >> s) & 1)) issue_s(j + 1, s, nxt.z);
                }
                if (!ok) break;
                if (elect_one()) {
                    umma_commit(bar(&ctl->v_empty[kv]));
                    if (nxt_live) umma_commit(bar(&ctl->k_empty[(j + 1) % kNK]));
                    mbar_arrive(bar(&ctl->m_empty[j % kNM]));
                }
                cur = nxt;
                ++j;
                if (++kv == kNV) { kv = 0; kv_par ^= 1; }
            }
            if (ok && elect_one()) {
                mbar_arrive(bar(&ctl->m_empty[j % kNM]));   // the end marker itself
                umma_commit(bar(&ctl->o_done[0]));
                umma_commit(bar(&ctl->o_done[1]));
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ V rows of the gather steps
        // The planner copies the K rows of a gather step, this warp its V rows: issuing the 16-byte copies is what
        // a gather step costs, and two warps halve it.  The warps meet at named barrier 2 per step.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        bool ok = true;
        for (int g = 0;; ++g) {
            named_bar_sync(2, 64);
            const int4 msg = ctl->gmsg[g & 1];          // (step, first ring entry, count)
            if (msg.z == 0) break;
            if (!ok) continue;                          // keep meeting the planner until it is done
            const int step = msg.x, width = msg.z > 64 ? 128 : 64;
            int col[4];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int e = ctl->colring[(msg.y + 32 * q4 + lane) & 511];
                col[q4] = lane + 32 * q4 < msg.z ? (e & 0x0fffffff) - a.kv_pos0 : 0;
                if (!MINF_IN_BOUNDS(a.status, col[q4] >= 0 && col[q4] < a.n_kv)) col[q4] = 0;
            }
            const int s = step % kNV, use = step / kNV;
            if (use > 0 && !mbar_wait(bar(&ctl->v_empty[s]), (use - 1) & 1, abort_flag)) { ok = false; continue; }
            gather_rows(smem_base + kVOff + s * kTile, a.v + b * a.v_sb + hk * a.v_sh, a.v_sn, col, width, lane);
            cp_async_arrive_noinc(bar(&ctl->v_full[s]));
        }
    } else if (warp == 3) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    } else {
        // ------------------------------------------------------------------ softmax / epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int slot = (warp - 4) >> 2;
        const int sub = warp & 3;                      // TMEM lane quarter this warp may access
        const int row_local = 32 * sub + lane;         // row inside the slot
        const int rb_local = 2 * slot + (row_local >> 6);
        const int lrow = lrow0 + 128 * slot + row_local;   // local query row
        const int row = a.q_pos0 + lrow;                   // position in the sequence
        const bool row_ok = lrow < a.n_q;
        const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
        const uint32_t t_o = tmem + slot * 256 + lane_base;
        const uint32_t t_s = t_o + 128;

        float m_ref = -INFINITY, l_sum = 0.f;
        int n = 0;
        bool ok = true;
        for (int j = 0; ok; ++j) {
            ok = mbar_wait(bar(&ctl->m_full[j % kNM]), (j / kNM) & 1, abort_flag);
            if (!ok) break;
            const Step& st = ctl->step[j % kNM];
            const int kind = st.kind;
            const int t = st.t, width = st.width;
            unsigned long long m0 = st.mask[rb_local][0], m1 = st.mask[rb_local][1];
            const bool slot_in = (st.parts >> slot) & 1;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(&ctl->m_empty[j % kNM]));
            if (kind == kEndStep) break;
            if (!slot_in) continue;

            if (kind == kTileStep) {
                unsigned long long c0, c1;
                upto128(min(row - t, kv_hi - 1 - t), c0, c1);         // causal and inside the local keys
                if (mode == MINF_MODE_ASHAPE) {
                    unsigned long long far0, far1, s0, s1;
                    upto128(row - n_local - t, far0, far1);           // keys at distance >= n_local ...
                    upto128(n_init - 1 - t, s0, s1);                  // ... are only visible as sinks
                    m0 = c0 & (~far0 | s0);
                    m1 = c1 & (~far1 | s1);
                } else {
                    m0 &= c0; m1 &= c1;
                }
            }
            if (!row_ok) { m0 = 0ull; m1 = 0ull; }

            ok = mbar_wait(bar(&ctl->s_full[slot]), n & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            if (width == 128)
                softmax_row<4>(t_s, t_o, m0, m1, a.scale_log2, n > 0, m_ref, l_sum, bar(&ctl->p_half[slot][0]), bar(&ctl->p_half[slot][1]));
            else
                softmax_row<2>(t_s, t_o, m0, m1, a.scale_log2, n > 0, m_ref, l_sum, bar(&ctl->p_half[slot][0]), bar(&ctl->p_half[slot][1]));
            ++n;
        }

        // epilogue: TMEM loads are warp-collective, so the whole warp runs them
        bool warp_ok = __all_sync(0xffffffffu, ok);
        if (warp_ok) {
            const bool w = mbar_wait(bar(&ctl->o_done[slot]), 0, abort_flag);
            warp_ok = __all_sync(0xffffffffu, w);
        }
        if (warp_ok) {
            tc_fence_after();
            const bool any_key = n > 0 && m_ref != -INFINITY;   // the row saw a visible key
            const float lse_cur = any_key ? m_ref + log2f(l_sum) : -INFINITY;
            const size_t row_idx = ((size_t)b * a.hq + h) * a.n_q + lrow;
            if (a.lse && row_ok) a.lse[row_idx] = lse_cur;
            // out = w_cur * O (unnormalised, reference maximum m_ref) + w_prev * carried output
            float w_cur = any_key ? 1.f / l_sum : 0.f, w_prev = 0.f;
            if (a.lse_acc && row_ok) {
                const float lse_prev = a.lse_acc[row_idx];
                float lse_new = lse_cur;
                if (lse_prev != -INFINITY) {
                    const float top = fmaxf(lse_prev, lse_cur);
                    lse_new = top + log2f(exp2f(lse_prev - top) + exp2f(lse_cur - top));
                    w_prev = exp2f(lse_prev - lse_new);
                    w_cur = any_key ? exp2f(m_ref - lse_new) : 0.f;
                }
                a.lse_acc[row_idx] = lse_new;
            }
            __nv_bfloat16* dst = a.o ? a.o + b * a.o_sb + h * a.o_sh + (long long)lrow * a.o_sn : nullptr;
            float* acc = a.o_acc ? a.o_acc + row_idx * kHeadDim : nullptr;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t orow[32];
                if (n > 0) {
                    tmem_ld32(t_o + 32 * c, orow);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) orow[i] = 0u;
                }
                if (row_ok) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {        // eight output values at a time
                        float val[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) val[i] = __uint_as_float(orow[8 * q4 + i]) * w_cur;
                        if (w_prev != 0.f) {
                            const float4 p0 = *reinterpret_cast<const float4*>(acc + 32 * c + 8 * q4);
                            const float4 p1 = *reinterpret_cast<const float4*>(acc + 32 * c + 8 * q4 + 4);
                            val[0] = fmaf(p0.x, w_prev, val[0]); val[1] = fmaf(p0.y, w_prev, val[1]);
                            val[2] = fmaf(p0.z, w_prev, val[2]); val[3] = fmaf(p0.w, w_prev, val[3]);
                            val[4] = fmaf(p1.x, w_prev, val[4]); val[5] = fmaf(p1.y, w_prev, val[5]);
                            val[6] = fmaf(p1.z, w_prev, val[6]); val[7] = fmaf(p1.w, w_prev, val[7]);
                        }
                        if (acc) {
                            *reinterpret_cast<float4*>(acc + 32 * c + 8 * q4) = make_float4(val[0], val[1], val[2], val[3]);
                            *reinterpret_cast<float4*>(acc + 32 * c + 8 * q4 + 4) = make_float4(val[4], val[5], val[6], val[7]);
                        }
                        if (dst) {
                            uint4 out;
                            out.x = pack_bf16x2(val[0], val[1]);
                            out.y = pack_bf16x2(val[2], val[3]);
                            out.z = pack_bf16x2(val[4], val[5]);
                            out.w = pack_bf16x2(val[6], val[7]);
                            *reinterpret_cast<uint4*>(dst + 32 * c + 8 * q4) = out;
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (ctl->abort) {
        // a wait was abandoned: give the copies and products this CTA may still have in flight time to land
        // before its shared memory and TMEM go to the next CTA
        __nanosleep(50000);
        if (threadIdx.x == 0) atomicOr(a.status + MINF_ST_ERROR, 1);
    }
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [batch, heads, tokens, 128] bf16 with element strides (sb, sh, sn); box = 64 x box_rows.
int make_tmap_bhnd(CUtensorMap* tm, const void* base, int batch, int heads, int tokens,
                   const int64_t st[3], int box_rows, const char* what) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(MINF_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (st[0] % 8) || (st[1] % 8) || (st[2] % 8))
        return fail(MINF_E_ARG, "%s: base and strides must be 16-byte aligned", what);
    cuuint64_t dims[4] = {(cuuint64_t)kHeadDim, (cuuint64_t)tokens, (cuuint64_t)heads, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)st[2] * 2, (cuuint64_t)st[1] * 2, (cuuint64_t)st[0] * 2};
    // a size-1 dimension may carry any stride in the caller's tensor; TMA still wants a sane one
    if (heads == 1) strides[1] = strides[0] * tokens;
    if (batch == 1) strides[2] = strides[1] * (heads > 1 ? heads : 1);
    cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MINF_E_CUDA, "%s: cuTensorMapEncodeTiled failed with code %d", what, (int)r);
    return MINF_OK;
}


}  // namespace minf

using namespace minf;

extern "C" int minf_sparse_attention_fwd_window(
    const void* q, const void* k, const void* v, void* o, float* lse, float* o_acc, float* lse_acc,
    const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3], const int64_t o_strides[3],
    int batch, int hq, int hkv, int context_size, int n_q, int q_pos0, int n_kv, int kv_pos0,
    int head_dim, float sm_scale,
    const int32_t* head_mode, const int32_t* head_param,
    const void* plan, const int32_t* vertical_indexes, int cap_v, int cap_s,
    int32_t* status, void* stream) {
    if (!q || !k || !v || !status || !q_strides || !k_strides || !v_strides || (o && !o_strides))
        return fail(MINF_E_ARG, "null pointer argument");
    if (!o && !o_acc) return fail(MINF_E_ARG, "neither o nor o_acc given: the call would have no output");
    if ((o_acc != nullptr) != (lse_acc != nullptr)) return fail(MINF_E_ARG, "o_acc and lse_acc go together");
    if (reinterpret_cast<uintptr_t>(o_acc) & 15) return fail(MINF_E_ARG, "o_acc must be 16-byte aligned");
    if (head_dim != kHeadDim) return fail(MINF_E_UNSUPPORTED, "head_dim must be 128 (got %d)", head_dim);
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || context_size < 1)
        return fail(MINF_E_ARG, "bad sizes: batch=%d hq=%d hkv=%d context=%d", batch, hq, hkv, context_size);
    if (context_size >= (1 << 28)) return fail(MINF_E_UNSUPPORTED, "context_size must be below 2^28");
    if (n_q < 1 || n_kv < 1 || q_pos0 < 0 || kv_pos0 < 0 || q_pos0 + n_q > context_size || kv_pos0 + n_kv > context_size)
        return fail(MINF_E_ARG, "query window [%d,+%d) or key window [%d,+%d) outside the context of %d tokens",
                    q_pos0, n_q, kv_pos0, n_kv, context_size);
    if ((q_pos0 % 256) || (kv_pos0 % 64))
        return fail(MINF_E_ARG, "q_pos0 must be a multiple of 256 and kv_pos0 a multiple of 64");
    if (reinterpret_cast<uintptr_t>(status) & 7) return fail(MINF_E_ARG, "status must be 8-byte aligned (words 2-3 are updated as one 64-bit counter)");
    if (head_mode && !head_param) return fail(MINF_E_ARG, "head_mode given without head_param");
    if (!head_mode && !plan) return fail(MINF_E_ARG, "plan is required when every head uses it");
    if (o && ((reinterpret_cast<uintptr_t>(o) & 15) || (o_strides[0] % 8) || (o_strides[1] % 8) || (o_strides[2] % 8)))
        return fail(MINF_E_ARG, "o: base and strides must be 16-byte aligned");
    if (cap_v < 0 || cap_s < 1 || cap_v > (1 << 20)) return fail(MINF_E_ARG, "bad plan capacities");

    Maps tm;
    int rc;
    if ((rc = make_tmap_bhnd(&tm.q, q, batch, hq, n_q, q_strides, 128, "q"))) return rc;
    if ((rc = make_tmap_bhnd(&tm.k64, k, batch, hkv, n_kv, k_strides, 64, "k"))) return rc;
    if ((rc = make_tmap_bhnd(&tm.k128, k, batch, hkv, n_kv, k_strides, 128, "k"))) return rc;
    if ((rc = make_tmap_bhnd(&tm.v64, v, batch, hkv, n_kv, v_strides, 64, "v"))) return rc;
    if ((rc = make_tmap_bhnd(&tm.v128, v, batch, hkv, n_kv, v_strides, 128, "v"))) return rc;

    AttnArgs a{};
    a.o = static_cast<__nv_bfloat16*>(o);
    a.k = static_cast<const __nv_bfloat16*>(k);
    a.v = static_cast<const __nv_bfloat16*>(v);
    a.lse = lse; a.o_acc = o_acc; a.lse_acc = lse_acc;
    if (o) { a.o_sb = o_strides[0]; a.o_sh = o_strides[1]; a.o_sn = o_strides[2]; }
    a.k_sb = k_strides[0]; a.k_sh = k_strides[1]; a.k_sn = k_strides[2];
    a.v_sb = v_strides[0]; a.v_sh = v_strides[1]; a.v_sn = v_strides[2];
    a.batch = batch; a.hq = hq; a.hkv = hkv; a.n_ctx = context_size;
    a.n_q = n_q; a.q_pos0 = q_pos0; a.n_kv = n_kv; a.kv_pos0 = kv_pos0;
    a.scale_log2 = sm_scale * 1.4426950408889634f;
    a.head_mode = head_mode; a.head_param = head_param;
    a.plan = static_cast<const unsigned char*>(plan);
    a.layout = make_plan_layout_window(q_pos0 / 64, (n_q + 63) / 64, cap_v, cap_s);
    a.v_idx = vertical_indexes; a.cap_v = cap_v;
    a.status = status;
    a.items_per_head = ((n_q + 63) / 64 + 3) / 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = kCtlOff + sizeof(Control);
    MINF_CUDA_OK(cudaFuncSetAttribute(sparse_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long ctas = (long long)a.items_per_head * batch * hq;
    if (ctas > 0x7fffffffLL) return fail(MINF_E_UNSUPPORTED, "grid too large");
    sparse_attn_fwd_kernel<<<(unsigned)ctas, 384, smem, st>>>(tm, a);
    MINF_LAUNCH_OK("sparse_attn_fwd_kernel");
    return MINF_OK;
}

extern "C" int minf_sparse_attention_fwd(
    const void* q, const void* k, const void* v, void* o,
    const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3], const int64_t o_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim, float sm_scale,
    const int32_t* head_mode, const int32_t* head_param,
    const void* plan, const int32_t* vertical_indexes, int cap_v, int cap_s,
    int32_t* status, void* stream) {
    if (!o) return fail(MINF_E_ARG, "null pointer argument");
    return minf_sparse_attention_fwd_window(q, k, v, o, nullptr, nullptr, nullptr, q_strides, k_strides, v_strides, o_strides,
                                            batch, hq, hkv, context_size, context_size, 0, context_size, 0,
                                            head_dim, sm_scale, head_mode, head_param, plan, vertical_indexes,
                                            cap_v, cap_s, status, stream);
}
