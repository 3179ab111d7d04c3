// Sparse flash-attention forward for sm_100a: tcgen05 MMA with TMEM accumulators, TMA tile
// loads for contiguous key ranges, cp.async gathers for vertical columns.
//
// One CTA owns 128*NSLOT consecutive query rows of one head (2*NSLOT row blocks of 64, the
// granularity at which the reference defines its index set,
// ops/pit_sparse_flash_attention_v2.py:64-153).  Warp roles:
//   warp 0            producer: walks the plan of its row blocks, merges them into a single
//                     stream of 64-key steps (a contiguous tile or 64 gathered columns) with
//                     one 64-bit column mask per row block, and fills the K/V stage ring
//   warp 1            issues every tcgen05.mma (lane 0) and owns the TMEM allocation
//   warps 2..5 (+4)   one thread per query row: masks, online softmax in registers, P as
//                     bf16 into shared memory, final normalisation and store
// Per step and slot:  S = Q K^T (128x64x128) -> softmax -> O += P V (128x128x64); S is double
// buffered in TMEM so the next QK^T overlaps the softmax.  The running maximum is only
// raised when it grows by more than 2^8, which keeps the O rescale in TMEM rare.
//
// Semantics kept from the reference kernels: causal mask inside contiguous tiles, none in
// the gathered-column loop, keys >= context masked, fp32 accumulation, P rounded to bf16,
// 1/sqrt(d) scale applied with exp2.  A row with no visible key yields zeros.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>

#include "common.h"
#include "plan_layout.h"
#include "sm100_ptx.cuh"

namespace minf {

constexpr int kHeadDim = 128;
constexpr uint32_t kQBytes = 128 * 256;     // one 128-row Q tile
constexpr uint32_t kStageBytes = 2 * 64 * 256;  // K tile + V tile, 64 keys each
constexpr uint32_t kPBytes = 128 * 128;     // 128 rows x 64 bf16

enum StepKind : int { kStepTile = 0, kStepGather = 1, kStepEnd = 2 };

struct StepMeta {
    int kind;
    int t;        // first key of a contiguous tile
    int pad0, pad1;
    unsigned long long mask[4];  // per row block of the CTA: which of the 64 keys it may see
};

template <int NSLOT>
struct SmemLayout {
    static constexpr int kStages = NSLOT == 1 ? 2 : 4;
    static constexpr uint32_t q_off = 0;
    static constexpr uint32_t kv_off = NSLOT * kQBytes;
    static constexpr uint32_t p_off = kv_off + kStages * kStageBytes;
    static constexpr uint32_t ctl_off = p_off + NSLOT * kPBytes;
};

template <int NSLOT>
struct Control {
    unsigned long long q_full;
    unsigned long long kv_full[SmemLayout<NSLOT>::kStages];
    unsigned long long kv_empty[SmemLayout<NSLOT>::kStages];
    unsigned long long s_full[NSLOT][2];
    unsigned long long p_full[NSLOT];
    unsigned long long pv_done[NSLOT];
    uint32_t tmem_base;
    int abort;
    StepMeta step[SmemLayout<NSLOT>::kStages];
    int colring[128];
};

struct AttnArgs {
    __nv_bfloat16* o;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    long long o_sb, o_sh, o_sn;
    long long k_sb, k_sh, k_sn;
    long long v_sb, v_sh, v_sn;
    int batch, hq, hkv, n_ctx, rows;
    float scale_log2;                 // sm_scale * log2(e)
    const int32_t* head_mode;
    const int32_t* head_param;
    const unsigned char* plan;
    PlanLayout layout;
    const int32_t* v_idx;
    int cap_v;
    int items_per_head;               // CTAs per (batch, head)
    int32_t* status;
};

// Cursor over the merged ranges of one row block, 32 ranges buffered across the warp.
struct RangeCursor {
    const int2* rng;
    int n;         // number of ranges
    int ri;        // current range
    int base;      // first range held in `buf`
    int2 buf;      // lane l holds range base + l
    int a, b;      // current range, a already advanced past consumed keys
    int last_row;  // last query row of the row block

    __device__ __forceinline__ void fetch(int lane) {
        if (ri >= n) { a = INT32_MAX; b = INT32_MAX; return; }
        if (ri - base >= 32 || ri < base) {
            base = ri;
            buf = (base + lane < n) ? rng[base + lane] : make_int2(INT32_MAX, INT32_MAX);
        }
        a = __shfl_sync(0xffffffffu, buf.x, ri - base);
        b = __shfl_sync(0xffffffffu, buf.y, ri - base);
    }
    __device__ __forceinline__ void init(const int2* r, int count, int last, int lane) {
        rng = r; n = count; ri = 0; base = -64; last_row = last;
        fetch(lane);
    }
    __device__ __forceinline__ bool live(int n_ctx) const { return ri < n && a <= last_row && a < n_ctx; }
};

__device__ __forceinline__ unsigned long long bit_span(int lo, int hi) {  // bits [lo, hi), 0 <= lo < hi <= 64
    const unsigned long long upper = hi >= 64 ? ~0ull : ((1ull << hi) - 1ull);
    return upper & (~0ull << lo);
}

template <int NSLOT>
__global__ void __launch_bounds__(64 + 128 * NSLOT, NSLOT == 1 ? 2 : 1)
sparse_attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const AttnArgs a) {
    using SL = SmemLayout<NSLOT>;
    constexpr int NS = SL::kStages;
    constexpr int NRB = 2 * NSLOT;
    extern __shared__ __align__(1024) unsigned char smem[];
    Control<NSLOT>* ctl = reinterpret_cast<Control<NSLOT>*>(smem + SL::ctl_off);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // work item: heaviest (latest) rows first; the heads of one item index are neighbours
    const int bh_count = a.batch * a.hq;
    const int item = a.items_per_head - 1 - (int)(blockIdx.x / bh_count);
    const int bh = (int)(blockIdx.x % bh_count);
    const int b = bh / a.hq, h = bh % a.hq;
    const int hk = h / (a.hq / a.hkv);
    const int rb0 = item * NRB;             // first row block
    const int row0 = rb0 * 64;              // first query row

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
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar(&ctl->kv_full[s]), 1);
            mbar_init(bar(&ctl->kv_empty[s]), 1 + 4 * NSLOT);
        }
        for (int s = 0; s < NSLOT; ++s) {
            mbar_init(bar(&ctl->s_full[s][0]), 1);
            mbar_init(bar(&ctl->s_full[s][1]), 1);
            mbar_init(bar(&ctl->p_full[s]), 128);
            mbar_init(bar(&ctl->pv_done[s]), 1);
        }
        ctl->abort = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&ctl->tmem_base), 256 * NSLOT);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
            mbar_arrive_expect_tx(bar(&ctl->q_full), NSLOT * kQBytes);
            for (int s = 0; s < NSLOT; ++s) {
                tma_load_4d(smem_base + SL::q_off + s * kQBytes, &tm_q, bar(&ctl->q_full), 0, row0 + 128 * s, h, b);
                tma_load_4d(smem_base + SL::q_off + s * kQBytes + 16384, &tm_q, bar(&ctl->q_full), 64, row0 + 128 * s, h, b);
            }
        }
        int step = 0;
        bool ok = true;
        // acquire a stage for `step`; returns stage index or -1 after an abandoned wait
        auto acquire = [&]() -> int {
            const int s = step % NS, use = step / NS;
            if (use > 0 && !mbar_wait(bar(&ctl->kv_empty[s]), (use - 1) & 1, abort_flag)) { ok = false; return -1; }
            return s;
        };
        auto issue_tile = [&](int s, int t) {
            if (lane == 0) {
                const uint32_t dst = smem_base + SL::kv_off + s * kStageBytes;
                const uint32_t fb = bar(&ctl->kv_full[s]);
                mbar_arrive_expect_tx(fb, kStageBytes);
                tma_load_4d(dst, &tm_k, fb, 0, t, hk, b);
                tma_load_4d(dst + 8192, &tm_k, fb, 64, t, hk, b);
                tma_load_4d(dst + 16384, &tm_v, fb, 0, t, hk, b);
                tma_load_4d(dst + 24576, &tm_v, fb, 64, t, hk, b);
            }
        };

        if (mode == MINF_MODE_ASHAPE) {
            const int r_hi = min(row0 + 64 * NRB, a.n_ctx) - 1;
            int w0 = row0 - n_local + 1;
            w0 = w0 < 0 ? 0 : (w0 & ~63);
            const bool sinks = a.n_ctx > n_local && r_hi >= n_local;
            const int sink_end = sinks ? min(min(n_init, w0), a.n_ctx) : 0;
            for (int phase = 0; phase < 2 && ok; ++phase) {
                const int t_lo = phase == 0 ? 0 : w0;
                const int t_hi = phase == 0 ? sink_end : r_hi + 1;
                for (int t = t_lo; t < t_hi && ok; t += 64) {
                    const int s = acquire();
                    if (s < 0) break;
                    if (lane == 0) {
                        ctl->step[s].kind = kStepTile;
                        ctl->step[s].t = t;
#pragma unroll
                        for (int r = 0; r < 4; ++r) ctl->step[s].mask[r] = ~0ull;
                    }
                    __syncwarp();
                    issue_tile(s, t);
                    ++step;
                }
            }
        } else {
            const unsigned char* slot = a.plan + (size_t)bh * a.layout.head_bytes;
            const int32_t* rng_cnt = reinterpret_cast<const int32_t*>(slot);
            const int2* rng_all = reinterpret_cast<const int2*>(slot + a.layout.rng_off);
            RangeCursor cur[NRB];
#pragma unroll
            for (int r = 0; r < NRB; ++r) {
                const int m = rb0 + r;
                const bool present = m < a.rows;
                cur[r].init(present ? rng_all + plan_rng_index(m, a.layout.cap_s) : nullptr,
                            present ? rng_cnt[m] : 0, m * 64 + 63, lane);
            }
            // ---- contiguous ranges, merged over the row blocks of this CTA
            while (ok) {
                int t = INT32_MAX;
#pragma unroll
                for (int r = 0; r < NRB; ++r)
                    if (cur[r].live(a.n_ctx)) t = min(t, cur[r].a);
                if (t == INT32_MAX) break;
                unsigned long long mk[NRB];
#pragma unroll
                for (int r = 0; r < NRB; ++r) {
                    mk[r] = 0ull;
                    // consume every range of this row block that intersects [t, t+64)
                    while (cur[r].live(a.n_ctx) && cur[r].a < t + 64) {
                        const int hi = min(cur[r].b, t + 64);
                        mk[r] |= bit_span(cur[r].a - t, hi - t);
                        if (cur[r].b <= t + 64) { ++cur[r].ri; cur[r].fetch(lane); }
                        else { cur[r].a = t + 64; break; }
                    }
                }
                const int s = acquire();
                if (s < 0) break;
                if (lane == 0) {
                    ctl->step[s].kind = kStepTile;
                    ctl->step[s].t = t;
#pragma unroll
                    for (int r = 0; r < 4; ++r) ctl->step[s].mask[r] = r < NRB ? mk[r] : 0ull;
                }
                __syncwarp();
                issue_tile(s, t);
                ++step;
            }
            // ---- gathered columns: union of the row blocks' bit masks over the vertical list
            const int words = a.layout.words_v;
            const uint32_t* bits = reinterpret_cast<const uint32_t*>(slot + a.layout.bits_off);
            const int32_t* vlist = a.v_idx ? a.v_idx + (size_t)bh * a.cap_v : nullptr;
            int filled = 0, emitted = 0;  // entries pushed to the ring / consumed from it
            auto flush_chunk = [&](int count) {  // gather `count` (<=64) ring entries starting at `emitted`
                const int s = acquire();
                if (s < 0) return;
                const int e0 = ctl->colring[(emitted + lane) & 127];
                const int e1 = ctl->colring[(emitted + 32 + lane) & 127];
                const bool v0 = lane < count, v1 = lane + 32 < count;
                unsigned long long mk[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                for (int r = 0; r < NRB; ++r) {
                    const unsigned lo = __ballot_sync(0xffffffffu, v0 && ((e0 >> (28 + r)) & 1));
                    const unsigned hi = __ballot_sync(0xffffffffu, v1 && ((e1 >> (28 + r)) & 1));
                    mk[r] = (unsigned long long)lo | ((unsigned long long)hi << 32);
                }
                if (lane == 0) {
                    ctl->step[s].kind = kStepGather;
                    ctl->step[s].t = 0;
#pragma unroll
                    for (int r = 0; r < 4; ++r) ctl->step[s].mask[r] = mk[r];
                }
                const int c0 = v0 ? (e0 & 0x0fffffff) : 0, c1 = v1 ? (e1 & 0x0fffffff) : 0;
                const uint32_t kdst = smem_base + SL::kv_off + s * kStageBytes;
                const __nv_bfloat16* kb = a.k + b * a.k_sb + hk * a.k_sh;
                const __nv_bfloat16* vb = a.v + b * a.v_sb + hk * a.v_sh;
                const int chunk = lane & 15, sub = lane >> 4;
#pragma unroll 4
                for (int it = 0; it < 32; ++it) {
                    const int r = 2 * it + sub;
                    const int col = __shfl_sync(0xffffffffu, r < 32 ? c0 : c1, r & 31);
                    const uint32_t off = (uint32_t)(chunk >> 3) * 8192u + (uint32_t)r * 128u +
                                         (uint32_t)(((chunk & 7) ^ (r & 7)) << 4);
                    cp_async_16(kdst + off, kb + (long long)col * a.k_sn + chunk * 8);
                    cp_async_16(kdst + 16384u + off, vb + (long long)col * a.v_sn + chunk * 8);
                }
                cp_async_commit();
                cp_async_wait<0>();
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(&ctl->kv_full[s]));
                emitted += count;
                ++step;
            };
            for (int w = 0; w < words && ok; ++w) {
                uint32_t wr[NRB];
                uint32_t any = 0;
#pragma unroll
                for (int r = 0; r < NRB; ++r) {
                    const int m = rb0 + r;
                    wr[r] = m < a.rows ? bits[(size_t)m * words + w] : 0u;
                    any |= wr[r];
                }
                if (any == 0u) continue;
                const bool mine = (any >> lane) & 1u;
                const int pos = filled + __popc(any & ((1u << lane) - 1u));
                if (mine) {
                    int e = vlist[32 * w + lane] & 0x0fffffff;
#pragma unroll
                    for (int r = 0; r < NRB; ++r) e |= (int)((wr[r] >> lane) & 1u) << (28 + r);
                    ctl->colring[pos & 127] = e;
                }
                filled += __popc(any);
                __syncwarp();
                if (filled - emitted >= 64) flush_chunk(64);
            }
            if (ok && filled > emitted) flush_chunk(filled - emitted);
        }
        // ---- end marker
        if (ok) {
            const int s = acquire();
            if (s >= 0) {
                if (lane == 0) {
                    ctl->step[s].kind = kStepEnd;
                    mbar_arrive(bar(&ctl->kv_full[s]));
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(128, 64, true, false, false);
            constexpr uint32_t idesc_o = umma_idesc(128, 128, true, false, true);
            int ns[NSLOT];       // participating steps issued so far, per slot (S side)
            int npv[NSLOT];      // per slot (PV side)
#pragma unroll
            for (int s = 0; s < NSLOT; ++s) { ns[s] = 0; npv[s] = 0; }
            bool ok = mbar_wait(bar(&ctl->q_full), 0, abort_flag);

            auto part = [&](const StepMeta& m, int slot) { return (m.mask[2 * slot] | m.mask[2 * slot + 1]) != 0ull; };
            auto issue_s = [&](int stage, int slot) {
                const uint32_t d = tmem + slot * 256 + 128 + (ns[slot] & 1) * 64;
                const uint32_t qb = smem_base + SL::q_off + slot * kQBytes;
                const uint32_t kb = smem_base + SL::kv_off + stage * kStageBytes;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t ad = umma_desc_sw128(qb + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    const uint64_t bd = umma_desc_sw128(kb + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024);
                    umma_ss(d, ad, bd, idesc_s, kk > 0);
                }
                umma_commit(bar(&ctl->s_full[slot][ns[slot] & 1]));
                ++ns[slot];
            };
            auto issue_pv = [&](int stage, int slot) {
                const uint32_t d = tmem + slot * 256;
                const uint32_t pb = smem_base + SL::p_off + slot * kPBytes;
                const uint32_t vb = smem_base + SL::kv_off + stage * kStageBytes + 16384;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t ad = umma_desc_sw128(pb + kk * 32, 16, 1024);
                    const uint64_t bd = umma_desc_sw128(vb + kk * 2048, 8192, 1024);
                    umma_ss(d, ad, bd, idesc_o, (npv[slot] > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar(&ctl->pv_done[slot]));
                ++npv[slot];
            };

            int j = 0;
            StepMeta cur_m;
            cur_m.kind = kStepEnd;
            if (ok) ok = mbar_wait(bar(&ctl->kv_full[0]), 0, abort_flag);
            if (ok) {
                cur_m = ctl->step[0];
                tc_fence_after();
                if (cur_m.kind != kStepEnd)
                    for (int s = 0; s < NSLOT; ++s)
                        if (part(cur_m, s)) issue_s(0, s);
            }
            while (ok && cur_m.kind != kStepEnd) {
                const int stage = j % NS;
                const int nstage = (j + 1) % NS;
                StepMeta nxt;
                ok = mbar_wait(bar(&ctl->kv_full[nstage]), ((j + 1) / NS) & 1, abort_flag);
                if (!ok) break;
                nxt = ctl->step[nstage];
                tc_fence_after();
                if (nxt.kind != kStepEnd)
                    for (int s = 0; s < NSLOT; ++s)
                        if (part(nxt, s)) issue_s(nstage, s);
                for (int s = 0; s < NSLOT && ok; ++s) {
                    if (!part(cur_m, s)) continue;
                    ok = mbar_wait(bar(&ctl->p_full[s]), npv[s] & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(stage, s);
                }
                if (!ok) break;
                umma_commit(bar(&ctl->kv_empty[stage]));
                cur_m = nxt;
                ++j;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / epilogue
        const int slot = (warp - 2) >> 2;
        const int sub = warp & 3;                      // TMEM lane quarter this warp may access
        const int row_local = 32 * sub + lane;         // 0..127 inside the slot
        const int rb_local = 2 * slot + (row_local >> 6);
        const int row = row0 + 128 * slot + row_local;
        const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
        const uint32_t t_o = tmem + slot * 256 + lane_base;
        const uint32_t p_row = smem_base + SL::p_off + slot * kPBytes + row_local * 128;

        float m_ref = -INFINITY, l_sum = 0.f;
        int n = 0;
        bool ok = true;
        for (int j = 0; ok; ++j) {
            const int stage = j % NS;
            ok = mbar_wait(bar(&ctl->kv_full[stage]), (j / NS) & 1, abort_flag);
            if (!ok) break;
            const int kind = ctl->step[stage].kind;
            if (kind == kStepEnd) break;
            const int t = ctl->step[stage].t;
            unsigned long long mask = ctl->step[stage].mask[rb_local];
            const bool slot_in = (ctl->step[stage].mask[2 * slot] | ctl->step[stage].mask[2 * slot + 1]) != 0ull;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(&ctl->kv_empty[stage]));  // metadata read
            if (!slot_in) continue;

            if (kind == kStepTile) {
                const int lim = row - t;  // keys t..t+lim are causal
                unsigned long long cm = lim >= 63 ? ~0ull : (lim < 0 ? 0ull : ((2ull << lim) - 1ull));
                const int nl = a.n_ctx - t;
                if (nl < 64) cm &= (1ull << nl) - 1ull;
                if (mode == MINF_MODE_ASHAPE) {
                    const int j_lo = row - n_local + 1 - t;
                    const unsigned long long wm = j_lo <= 0 ? ~0ull : (j_lo >= 64 ? 0ull : (~0ull << j_lo));
                    const int ns_ = n_init - t;
                    const unsigned long long sm = ns_ >= 64 ? ~0ull : (ns_ <= 0 ? 0ull : ((1ull << ns_) - 1ull));
                    mask = cm & (wm | sm);
                } else {
                    mask &= cm;
                }
            }
            if (row >= a.n_ctx) mask = 0ull;

            ok = mbar_wait(bar(&ctl->s_full[slot][n & 1]), (n >> 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[64];
            {
                uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[0]);
                uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[32]);
                const uint32_t t_s = tmem + slot * 256 + 128 + (n & 1) * 64 + lane_base;
                tmem_ld32(t_s, lo);
                tmem_ld32(t_s + 32, hi);
                tmem_wait_ld();
            }
            float mx = -INFINITY;
            if (mask == ~0ull) {
#pragma unroll
                for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(sr[c]));
            } else {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const float x = ((mask >> c) & 1ull) ? __uint_as_float(sr[c]) : -INFINITY;
                    sr[c] = __float_as_uint(x);
                    mx = fmaxf(mx, x);
                }
            }
            mx *= a.scale_log2;  // scale > 0, so the maximum commutes with it
            float alpha = 1.f;
            if (mx > m_ref + 8.f) {
                alpha = fast_exp2(m_ref - mx);  // 0 when m_ref is still -inf
                l_sum *= alpha;
                m_ref = mx;
            }
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
            float psum = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c]), a.scale_log2, neg_m));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), a.scale_log2, neg_m));
                psum += p0 + p1;
                pk[c >> 1] = pack_bf16x2(p0, p1);
            }
            l_sum += psum;

            if (n > 0) {
                ok = mbar_wait(bar(&ctl->pv_done[slot]), (n - 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t orow[32];
                        tmem_ld32(t_o + 32 * c, orow);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * alpha);
                        tmem_st32(t_o + 32 * c, orow);
                    }
                    tmem_wait_st();
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t dst = p_row + (uint32_t)((c ^ (row_local & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * c]),
                             "r"(pk[4 * c + 1]), "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3])
                             : "memory");
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(bar(&ctl->p_full[slot]));
            ++n;
        }

        // TMEM loads are warp-collective: run them for the whole warp, store only live rows.
        {
            bool warp_ok = __all_sync(0xffffffffu, ok);
            if (warp_ok && n > 0) {
                bool w = mbar_wait(bar(&ctl->pv_done[slot]), (n - 1) & 1, abort_flag);
                warp_ok = __all_sync(0xffffffffu, w);
            }
            if (warp_ok) {
                tc_fence_after();
                const float inv = (n > 0 && l_sum > 0.f) ? 1.f / l_sum : 0.f;
                __nv_bfloat16* dst = a.o + b * a.o_sb + h * a.o_sh + (long long)row * a.o_sn;
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
                    if (row < a.n_ctx) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 out;
                            out.x = pack_bf16x2(__uint_as_float(orow[8 * q4 + 0]) * inv, __uint_as_float(orow[8 * q4 + 1]) * inv);
                            out.y = pack_bf16x2(__uint_as_float(orow[8 * q4 + 2]) * inv, __uint_as_float(orow[8 * q4 + 3]) * inv);
                            out.z = pack_bf16x2(__uint_as_float(orow[8 * q4 + 4]) * inv, __uint_as_float(orow[8 * q4 + 5]) * inv);
                            out.w = pack_bf16x2(__uint_as_float(orow[8 * q4 + 6]) * inv, __uint_as_float(orow[8 * q4 + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + 32 * c + 8 * q4) = out;
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && ctl->abort) atomicOr(a.status + MINF_ST_ERROR, 1);
    if (warp == 1) tmem_dealloc(tmem, 256 * NSLOT);
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

template <int NSLOT>
static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, AttnArgs a,
                       cudaStream_t st) {
    const size_t smem = SmemLayout<NSLOT>::ctl_off + sizeof(Control<NSLOT>);
    MINF_CUDA_OK(cudaFuncSetAttribute(sparse_attn_fwd_kernel<NSLOT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    a.items_per_head = (a.rows + 2 * NSLOT - 1) / (2 * NSLOT);
    const long long ctas = (long long)a.items_per_head * a.batch * a.hq;
    if (ctas > 0x7fffffffLL) return fail(MINF_E_UNSUPPORTED, "grid too large");
    sparse_attn_fwd_kernel<NSLOT><<<(unsigned)ctas, 64 + 128 * NSLOT, smem, st>>>(tq, tk, tv, a);
    MINF_LAUNCH_OK("sparse_attn_fwd_kernel");
    return MINF_OK;
}

static int attn_slots() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MINFER_B200_SLOTS");
        v = (e && e[0] == '2') ? 2 : 1;
    }
    return v;
}

int launch_sparse_attention_v2(const void* q, const void* k, const void* v, void* o,
                               const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                               const int64_t o_strides[3], int batch, int hq, int hkv, int context_size,
                               float sm_scale, const int32_t* head_mode, const int32_t* head_param,
                               const void* plan, const int32_t* vertical_indexes, int cap_v, int cap_s,
                               int32_t* status, cudaStream_t st);

static int attn_variant() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MINFER_B200_ATTN");
        v = (e && e[0] == 'v' && e[1] == '1') ? 1 : 2;
    }
    return v;
}

}  // namespace minf

using namespace minf;

extern "C" int minf_sparse_attention_fwd(
    const void* q, const void* k, const void* v, void* o,
    const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3], const int64_t o_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim, float sm_scale,
    const int32_t* head_mode, const int32_t* head_param,
    const void* plan, const int32_t* vertical_indexes, int cap_v, int cap_s,
    int32_t* status, void* stream) {
    if (!q || !k || !v || !o || !status || !q_strides || !k_strides || !v_strides || !o_strides)
        return fail(MINF_E_ARG, "null pointer argument");
    if (head_dim != kHeadDim) return fail(MINF_E_UNSUPPORTED, "head_dim must be 128 (got %d)", head_dim);
    if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || context_size < 1)
        return fail(MINF_E_ARG, "bad sizes: batch=%d hq=%d hkv=%d context=%d", batch, hq, hkv, context_size);
    if (context_size >= (1 << 28)) return fail(MINF_E_UNSUPPORTED, "context_size must be below 2^28");
    if (head_mode && !head_param) return fail(MINF_E_ARG, "head_mode given without head_param");
    if (!head_mode && !plan) return fail(MINF_E_ARG, "plan is required when every head uses it");
    if ((reinterpret_cast<uintptr_t>(o) & 15) || (o_strides[0] % 8) || (o_strides[1] % 8) || (o_strides[2] % 8))
        return fail(MINF_E_ARG, "o: base and strides must be 16-byte aligned");
    if (cap_v < 0 || cap_s < 1 || cap_v > (1 << 20)) return fail(MINF_E_ARG, "bad plan capacities");

    if (attn_variant() == 2)
        return launch_sparse_attention_v2(q, k, v, o, q_strides, k_strides, v_strides, o_strides, batch, hq, hkv,
                                          context_size, sm_scale, head_mode, head_param, plan, vertical_indexes,
                                          cap_v, cap_s, status, static_cast<cudaStream_t>(stream));
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tmap_bhnd(&tq, q, batch, hq, context_size, q_strides, 128, "q"))) return rc;
    if ((rc = make_tmap_bhnd(&tk, k, batch, hkv, context_size, k_strides, 64, "k"))) return rc;
    if ((rc = make_tmap_bhnd(&tv, v, batch, hkv, context_size, v_strides, 64, "v"))) return rc;

    AttnArgs a{};
    a.o = static_cast<__nv_bfloat16*>(o);
    a.k = static_cast<const __nv_bfloat16*>(k);
    a.v = static_cast<const __nv_bfloat16*>(v);
    a.o_sb = o_strides[0]; a.o_sh = o_strides[1]; a.o_sn = o_strides[2];
    a.k_sb = k_strides[0]; a.k_sh = k_strides[1]; a.k_sn = k_strides[2];
    a.v_sb = v_strides[0]; a.v_sh = v_strides[1]; a.v_sn = v_strides[2];
    a.batch = batch; a.hq = hq; a.hkv = hkv; a.n_ctx = context_size; a.rows = (context_size + 63) / 64;
    a.scale_log2 = sm_scale * 1.4426950408889634f;
    a.head_mode = head_mode; a.head_param = head_param;
    a.plan = static_cast<const unsigned char*>(plan);
    a.layout = make_plan_layout(context_size, cap_v, cap_s);
    a.v_idx = vertical_indexes; a.cap_v = cap_v;
    a.status = status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (attn_slots() == 2) return launch_attn<2>(tq, tk, tv, a, st);
    return launch_attn<1>(tq, tk, tv, a, st);
}
