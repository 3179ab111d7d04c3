"""Zigzag ring attention for sequence-sharded vertical-slash prefill (one process per GPU).

The reference has no sequence parallelism; this module shards one long sequence over the
ranks of a process group.  The sequence is cut into 2P equal chunks and rank r owns chunks r
and 2P-1-r of Q, K, V and O, which balances the causal work.  Index estimation needs one
exchange (the last 64 queries are broadcast, per-chunk softmax statistics are gathered and the
vertical / slash score arrays are summed over the ranks), after which every rank holds the
same global index lists and builds the plans of its own query chunks.  The attention itself
is a ring: in step t a rank holds the K/V shard of rank r-t, attends its two query chunks to
the shard's two key chunks (pairs that lie entirely in the future are skipped) and passes the
shard on while it computes.  Partial results of different key chunks are merged through the
per-row log-sum-exp: the kernel carries an fp32 accumulator from one key chunk to the next and
rounds the output once, with the last chunk.

Everything that touches the GPU goes through the C ABI; the orchestration (chunk schedule,
communication, merge) is plain torch so that it can be exercised on CPU ranks (gloo) with a
stand-in for the attention call.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from .. import _cabi

NEG_INF = float("-inf")


# ------------------------------------------------------------------------------ layout

def chunk_size(n_ctx: int, world: int) -> int:
    c, rem = divmod(n_ctx, 2 * world)
    if rem or c % 256:
        raise ValueError(f"the sequence ({n_ctx}) must split into {2 * world} chunks that are multiples of 256 tokens")
    return c


def owned_chunks(rank: int, world: int):
    return (rank, 2 * world - 1 - rank)


def zigzag_split(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """``[B,H,N,D]`` (or ``[..., N, D]``) -> the two chunks of ``rank`` concatenated along the token axis."""
    n = x.shape[-2]
    c = chunk_size(n, world)
    a, b = owned_chunks(rank, world)
    return torch.cat((x[..., a * c:(a + 1) * c, :], x[..., b * c:(b + 1) * c, :]), dim=-2).contiguous()


def zigzag_merge(parts, world: int) -> torch.Tensor:
    """Inverse of ``zigzag_split`` given the local tensors of all ranks in rank order."""
    c = parts[0].shape[-2] // 2
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = owned_chunks(r, world)
        chunks[a], chunks[b] = p[..., :c, :], p[..., c:, :]
    return torch.cat(chunks, dim=-2)


def pair_is_visible(q_chunk: int, kv_chunk: int) -> bool:
    """A key chunk matters to a query chunk unless it lies entirely in the future."""
    return kv_chunk <= q_chunk


# ------------------------------------------------------------------------------ merge

def merge_partial(acc_o: torch.Tensor, acc_lse: torch.Tensor, o: torch.Tensor, lse: torch.Tensor):
    """Fold one partial result into the accumulator (base-2 log-sum-exp, see minfer_b200.h).

    ``acc_o`` fp32 ``[B,H,C,D]``, ``acc_lse`` fp32 ``[B,H,C]``; rows that have seen no key carry
    ``-inf`` and zeros.  Returns the new pair (in place on the accumulators).
    """
    new_lse = torch.logaddexp2(acc_lse, lse)
    safe = torch.where(torch.isinf(new_lse), torch.zeros_like(new_lse), new_lse)
    w_old = torch.exp2(acc_lse - safe)
    w_new = torch.exp2(lse - safe)
    acc_o.mul_(w_old.unsqueeze(-1)).add_(o.float() * w_new.unsqueeze(-1))
    acc_lse.copy_(new_lse)
    return acc_o, acc_lse


# ------------------------------------------------------------------------------ CUDA pieces

def build_plan_window(v_idx, s_idx, nnz_v, nnz_s, n_ctx: int, q_pos0: int, n_q: int):
    """Plan of the query rows ``[q_pos0, q_pos0 + n_q)`` from the global index lists."""
    B, H, cap_v = v_idx.shape
    cap_s = s_idx.shape[2]
    dev = v_idx.device
    L = _cabi.lib()
    plan = torch.empty(L.minf_plan_bytes_window(B, H, q_pos0, n_q, cap_v, cap_s), dtype=torch.uint8, device=dev)
    status = _cabi.new_status(dev)
    seqlens = torch.full((B,), n_ctx, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(L.minf_vs_build_plan_window(
            _cabi.ptr(seqlens), _cabi.ptr(v_idx), _cabi.ptr(s_idx), _cabi.ptr(nnz_v), _cabi.ptr(nnz_s),
            B, H, q_pos0, n_q, cap_v, cap_s, _cabi.ptr(plan), _cabi.ptr(status), _cabi.stream_ptr(dev)))
    return plan, status


def count_tiles_window(plan, batch: int, heads: int, q_pos0: int, n_q: int, cap_v: int, cap_s: int) -> int:
    """64x64 tiles of the reference index set for the rows a window plan covers."""
    out = torch.zeros(1, dtype=torch.int64, device=plan.device)
    with torch.cuda.device(plan.device):
        _cabi.check(_cabi.lib().minf_plan_count_tiles_window(_cabi.ptr(plan), batch, heads, q_pos0, n_q, cap_v, cap_s,
                                                             _cabi.ptr(out), _cabi.stream_ptr(plan.device)))
    return int(out.item())


def attention_window(q, k, v, n_ctx: int, q_pos0: int, kv_pos0: int, plan, v_idx, cap_s: int, status, sm_scale=None,
                     head_mode=None, head_param=None, cap_v: int | None = None, carry=None, out=None):
    """One (query chunk, key chunk) pair through ``minf_sparse_attention_fwd_window``.
    ``head_mode`` / ``head_param`` select per head between the plan and the A-shape mask.

    Without ``carry`` the call returns the normalised partial output and its base-2 log-sum-exp.
    With ``carry = (o_acc fp32 [B,H,n_q,D], lse_acc fp32 [B,H,n_q])`` the kernel folds this key chunk
    into the carried result itself (in fp32, see the header) and ``out`` -- given for the last key
    chunk of a query chunk -- receives the merged result rounded to the input dtype once."""
    B, H, n_q, D = q.shape
    n_kv = k.shape[2]
    dev = q.device
    lse = None
    if carry is None:
        out = torch.empty((B, H, n_q, D), dtype=q.dtype, device=dev) if out is None else out
        lse = torch.empty((B, H, n_q), dtype=torch.float32, device=dev)
    o_acc, lse_acc = carry if carry is not None else (None, None)
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().minf_sparse_attention_fwd_window(
            _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(out), _cabi.ptr(lse), _cabi.ptr(o_acc), _cabi.ptr(lse_acc),
            _cabi.strides3(q), _cabi.strides3(k), _cabi.strides3(v), _cabi.strides3(out) if out is not None else None,
            B, H, k.shape[1], n_ctx, n_q, q_pos0, n_kv, kv_pos0, D, float(sm_scale or D ** -0.5),
            _cabi.ptr(head_mode), _cabi.ptr(head_param), _cabi.ptr(plan), _cabi.ptr(v_idx),
            cap_v if cap_v is not None else (v_idx.shape[2] if v_idx is not None else 0), cap_s,
            _cabi.ptr(status), _cabi.stream_ptr(dev)))
    return out, lse


def _ordered_blocks(gathered: torch.Tensor, world: int, bl: int) -> torch.Tensor:
    """``[world, R, 64, 2*bl, 2]`` (every rank's two chunks, rank-major) -> ``[R, 64, 2*world*bl, 2]`` with the
    statistics blocks in ascending key order: chunk r is rank r's first, chunk 2*world-1-r its second."""
    g = gathered.view(world, gathered.shape[1], 64, 2, bl, 2)
    first = g[:, :, :, 0].permute(1, 2, 0, 3, 4)
    second = g[:, :, :, 1].flip(0).permute(1, 2, 0, 3, 4)
    return torch.cat((first, second), dim=2).reshape(gathered.shape[1], 64, 2 * world * bl, 2).contiguous()


def slash_window(n_ctx: int, chunk: int, c: int):
    """Diagonal offsets the keys of chunk ``chunk`` can contribute to: ``[lo, hi)``.  A diagonal is 64 queries
    long, so neighbouring chunks share 63 offsets."""
    last_q = min(64, n_ctx)
    lo = max(0, (n_ctx - last_q) - (chunk + 1) * c + 1)
    hi = min(n_ctx, n_ctx - chunk * c)
    return lo, hi


def rank_score_pack(score_pass, chunks, n_ctx: int, c: int, B: int, H: int, dev) -> torch.Tensor:
    """What one rank contributes to the score exchange, ``[B, H, 2, c + (c + 64)]``: per owned chunk the vertical
    scores of its ``c`` keys and the window of diagonal offsets those keys reach (``slash_window``).
    ``score_pass(i, vertical, slash)`` runs the score pass of the rank's i-th chunk into full-length arrays.  The two
    chunks are scored one after the other, each into a cleared window: the middle rank's chunks are neighbours, and
    the 63 offsets their windows share must not be summed before the exchange."""
    scores = torch.empty((2, B, H, n_ctx), dtype=torch.float32, device=dev)
    pack = torch.zeros((B, H, 2, 2 * c + 64), dtype=torch.float32, device=dev)
    for i, ci in enumerate(chunks):
        lo, hi = slash_window(n_ctx, ci, c)
        scores[1][:, :, lo:hi].zero_()
        score_pass(i, scores[0], scores[1])
        pack[:, :, i, :c] = scores[0][:, :, ci * c:(ci + 1) * c]
        pack[:, :, i, c:c + hi - lo] = scores[1][:, :, lo:hi]
    return pack


def assemble_scores(everyone: torch.Tensor, n_ctx: int, c: int, world: int) -> torch.Tensor:
    """``[world, B, H, 2, 2c + 64]`` (every rank's pack) -> ``[2, B, H, n_ctx]`` vertical and slash scores of the whole
    sequence.  Chunks are added in ascending order, so the 63 offsets two neighbouring chunks share are summed in
    a fixed order (and a sum of two terms does not depend on it anyway)."""
    B, H = everyone.shape[1], everyone.shape[2]
    scores = torch.zeros((2, B, H, n_ctx), dtype=torch.float32, device=everyone.device)
    for chunk in range(2 * world):
        r, i = (chunk, 0) if chunk < world else (2 * world - 1 - chunk, 1)
        lo, hi = slash_window(n_ctx, chunk, c)
        scores[0][:, :, chunk * c:(chunk + 1) * c] = everyone[r, :, :, i, :c]
        scores[1][:, :, lo:hi] += everyone[r, :, :, i, c:c + hi - lo]
    return scores


def ring_vertical_slash_estimate(q_loc, k_loc, n_ctx: int, vertical_size, slash_size, group=None,
                                 cap_v: int | None = None, cap_s: int | None = None):
    """Global index lists from sharded K: ``(v_idx, s_idx, nnz_v, nnz_s)``, identical on all ranks.
    The budgets are ints (every head) or int32 tensors ``[H]`` with -1 for heads that are not
    vertical-slash (their lists are left unset and ``nnz`` is -1); tensors need ``cap_v`` / ``cap_s``.

    Exchanges: the last 64 queries (broadcast), the per-block softmax statistics (all-gather, a few MB),
    and each rank's own part of the score arrays (one all-gather: vertical scores of its keys and the
    diagonal offsets its keys reach).  Overlapping diagonal parts are added in chunk order, and the
    statistics blocks are combined in key order, so the lists do not depend on the number of ranks
    (for chunks that are multiples of 2048 tokens)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, H, n_loc, D = q_loc.shape
    Hkv = k_loc.shape[1]
    dev = q_loc.device
    c = chunk_size(n_ctx, world)
    L = _cabi.lib()
    # the last 64 queries live at the end of rank 0's second chunk
    q_last = q_loc[:, :, -64:, :].contiguous() if rank == 0 else torch.empty((B, H, 64, D), dtype=q_loc.dtype, device=dev)
    dist.broadcast(q_last, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    bl = L.minf_vs_scores_blocks(c)
    stats = torch.empty((B * H, 64, 2 * bl, 2), dtype=torch.float32, device=dev)
    status = _cabi.new_status(dev)
    chunks = owned_chunks(rank, world)
    k_parts = [k_loc[:, :, :c], k_loc[:, :, c:]]

    def run(pass_, i, stats_t, total, row_stats, vertical, slash):
        ci, kp = chunks[i], k_parts[i]
        with torch.cuda.device(dev):
            _cabi.check(L.minf_vs_scores_pass(
                pass_, _cabi.ptr(q_last), _cabi.ptr(kp), _cabi.strides3(q_last), _cabi.strides3(kp),
                B, H, Hkv, n_ctx, c, ci * c, D, _cabi.ptr(stats_t), i * bl, total, _cabi.ptr(row_stats),
                _cabi.ptr(vertical), _cabi.ptr(slash), _cabi.ptr(status), _cabi.stream_ptr(dev)))

    for i in range(2):
        run(1, i, stats, 2 * bl, None, None, None)
    gathered = torch.empty((world,) + tuple(stats.shape), dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(gathered, stats, group=group)
    all_stats = _ordered_blocks(gathered, world, bl)            # [B*H, 64, 2*world*bl, 2], ascending key order
    row_stats = torch.empty((B * H, 64, 2), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(L.minf_vs_scores_combine(_cabi.ptr(all_stats), B, H, all_stats.shape[2], _cabi.ptr(row_stats),
                                             _cabi.stream_ptr(dev)))
    pack = rank_score_pack(lambda i, vertical, slash: run(2, i, None, 2 * world * bl, row_stats, vertical, slash),
                           chunks, n_ctx, c, B, H, dev)
    everyone = torch.empty((world,) + tuple(pack.shape), dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(everyone, pack, group=group)
    scores = assemble_scores(everyone, n_ctx, c, world)
    if torch.is_tensor(vertical_size):
        vs = vertical_size.to(device=dev, dtype=torch.int32).repeat(B).contiguous()
        ss = slash_size.to(device=dev, dtype=torch.int32).repeat(B).contiguous()
    else:
        cap_v, cap_s = min(n_ctx, max(vertical_size, 30)), min(n_ctx, max(slash_size, 50))
        vs = torch.full((B * H,), vertical_size, dtype=torch.int32, device=dev)
        ss = torch.full((B * H,), slash_size, dtype=torch.int32, device=dev)
    v_idx = torch.empty((B, H, cap_v), dtype=torch.int32, device=dev)
    s_idx = torch.empty((B, H, cap_s), dtype=torch.int32, device=dev)
    nnz_v = torch.empty((B * H,), dtype=torch.int32, device=dev)
    nnz_s = torch.empty((B * H,), dtype=torch.int32, device=dev)
    scratch = torch.empty(L.minf_vs_select_scratch_bytes(B, H, n_ctx), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(L.minf_vs_select(_cabi.ptr(scores[0]), _cabi.ptr(scores[1]), B, H, n_ctx, _cabi.ptr(vs), _cabi.ptr(ss),
                                     cap_v, cap_s, _cabi.ptr(v_idx), _cabi.ptr(s_idx), _cabi.ptr(nnz_v), _cabi.ptr(nnz_s),
                                     *_cabi.SELECT_RULES["online"], _cabi.ptr(scratch), _cabi.stream_ptr(dev)))
    _cabi.raise_on_status(status, "ring_vertical_slash_estimate")
    return v_idx, s_idx, nnz_v, nnz_s


# ------------------------------------------------------------------------------ the ring

AttnFn = Callable[..., tuple]


def ring_attention(q_loc, k_loc, v_loc, n_ctx: int, attn_fn: AttnFn, group=None, fused_merge: bool = False):
    """Ring schedule and communication.

    ``fused_merge=False``: ``attn_fn(q_chunk, k_chunk, v_chunk, q_chunk_index, q_pos0, kv_pos0)`` returns the
    normalised partial output and its base-2 log-sum-exp for the keys it was given, and the partials
    are merged here with torch ops (the CPU stand-ins of the tests work this way).
    ``fused_merge=True``: ``attn_fn(..., carry, out)`` folds the key chunk into ``carry = (o_acc, lse_acc)``
    itself and writes the merged rows to ``out`` when it is not ``None`` (the CUDA kernel does both
    in its epilogue); ``out`` is passed with the last key chunk a query chunk sees.
    Returns the local output ``[B,H,2C,D]`` in the dtype of ``q_loc``.  The K/V receive buffers,
    the accumulators and the output are allocated once per call.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    c = chunk_size(n_ctx, world)
    B, H, _, D = q_loc.shape
    dev = q_loc.device
    # every rank can check its own shard against the layout all ranks derive from (n_ctx, world): a rank with a
    # wrong shard stops here, before it sends anything, and its neighbours' receives end in the group's timeout
    for name, t in (("q_loc", q_loc), ("k_loc", k_loc), ("v_loc", v_loc)):
        if t.shape[2] != 2 * c or t.shape[0] != B or t.shape[3] != D:
            raise ValueError(f"{name} has shape {tuple(t.shape)}; rank {rank} of {world} owns two chunks of {c} tokens "
                             f"of a {n_ctx}-token sequence")
    if k_loc.shape != v_loc.shape:
        raise ValueError(f"k_loc {tuple(k_loc.shape)} and v_loc {tuple(v_loc.shape)} differ")
    q_chunks = owned_chunks(rank, world)
    q_parts = [q_loc[:, :, :c], q_loc[:, :, c:]]
    acc_o = torch.empty((2, B, H, c, D), dtype=torch.float32, device=dev)
    if not fused_merge:
        acc_o.zero_()
    acc_l = torch.full((2, B, H, c), NEG_INF, dtype=torch.float32, device=dev)
    out = torch.empty((B, H, 2 * c, D), dtype=q_loc.dtype, device=dev)
    # how many key chunks each query chunk will see over the whole ring
    pairs_left = [sum(1 for kc in range(2 * world) if pair_is_visible(qc, kc)) for qc in q_chunks]

    kv = (k_loc, v_loc)                                   # the caller's tensors are sent as they are
    bufs = [tuple(torch.empty_like(t) for t in kv) for _ in range(2 if world > 2 else 1)] if world > 1 else []
    send_to = (rank + 1) % world
    recv_from = (rank - 1) % world
    if group is not None:
        send_to, recv_from = dist.get_global_rank(group, send_to), dist.get_global_rank(group, recv_from)

    for step in range(world):
        src = (rank - step) % world
        reqs = []
        nxt = None
        nvtx = _cabi.nvtx_range(f"ring:step{step}")
        nvtx.__enter__()
        if step + 1 < world:       # pass the shard on while this step computes
            nxt = bufs[step % len(bufs)]
            ops = [dist.P2POp(dist.isend, kv[0], send_to, group), dist.P2POp(dist.isend, kv[1], send_to, group),
                   dist.P2POp(dist.irecv, nxt[0], recv_from, group), dist.P2POp(dist.irecv, nxt[1], recv_from, group)]
            reqs = dist.batch_isend_irecv(ops)
        kv_chunks = owned_chunks(src, world)
        for qi, qc in enumerate(q_chunks):
            for ki, kc in enumerate(kv_chunks):
                if not pair_is_visible(qc, kc):
                    continue
                k_part = kv[0][:, :, ki * c:(ki + 1) * c]
                v_part = kv[1][:, :, ki * c:(ki + 1) * c]
                pairs_left[qi] -= 1
                if fused_merge:
                    attn_fn(q_parts[qi], k_part, v_part, qi, qc * c, kc * c, (acc_o[qi], acc_l[qi]),
                            out[:, :, qi * c:(qi + 1) * c] if pairs_left[qi] == 0 else None)
                else:
                    o, lse = attn_fn(q_parts[qi], k_part, v_part, qi, qc * c, kc * c)
                    merge_partial(acc_o[qi], acc_l[qi], o, lse)
        for r in reqs:
            r.wait()
        nvtx.__exit__(None, None, None)
        if nxt is not None:
            kv = nxt               # the next receive into the other buffer set is ordered after this step's kernels
    if not fused_merge:
        out[:, :, :c] = acc_o[0].to(q_loc.dtype)
        out[:, :, c:] = acc_o[1].to(q_loc.dtype)
    return out


def ring_vertical_slash_attention(q_loc, k_loc, v_loc, n_ctx: int, vertical_size: int = 1000, slash_size: int = 6096,
                                  group=None, indices=None, stats: Optional[dict] = None):
    """Sequence-sharded vertical-slash prefill attention of one layer.

    ``q_loc [1,Hq,2C,128]``, ``k_loc / v_loc [1,Hkv,2C,128]`` hold this rank's two zigzag chunks.
    ``indices = (v_idx, s_idx, nnz_v, nnz_s)`` skips the distributed estimation (the lists must be
    the sorted int32 global lists, identical on all ranks).
    """
    _cabi.require_cuda(q_loc, k_loc, v_loc)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    c = chunk_size(n_ctx, world)
    if indices is None:
        indices = ring_vertical_slash_estimate(q_loc, k_loc, n_ctx, vertical_size, slash_size, group)
    v_idx, s_idx, nnz_v, nnz_s = indices
    plans = []
    for qc in owned_chunks(rank, world):
        plans.append(build_plan_window(v_idx, s_idx, nnz_v, nnz_s, n_ctx, qc * c, c))

    def attn_fn(q, k, v, qi, q_pos0, kv_pos0, carry, out):
        plan, status = plans[qi]
        if stats is not None:      # CUDA-event timing of the attention launches (benchmarks)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        attention_window(q, k, v, n_ctx, q_pos0, kv_pos0, plan, v_idx, s_idx.shape[2], status, carry=carry, out=out)
        if stats is not None:
            e1.record()
            stats.setdefault("attn_events", []).append((e0, e1))

    out = ring_attention(q_loc, k_loc, v_loc, n_ctx, attn_fn, group, fused_merge=True)
    if stats is not None:
        stats["indices"] = indices
        if stats.get("count_tiles"):
            B, H = q_loc.shape[0], q_loc.shape[1]
            stats["tiles"] = sum(count_tiles_window(plan, B, H, qc * c, c, v_idx.shape[2], s_idx.shape[2])
                                 for (plan, _), qc in zip(plans, owned_chunks(rank, world)))
            stats["issued"] = sum(issued_tiles(status) for _, status in plans)
    for plan, status in plans:
        _cabi.raise_on_status(status, "ring_vertical_slash_attention")
    return out


def issued_tiles(status: torch.Tensor) -> int:
    """64x64 tile equivalents the attention launches that shared ``status`` sent to the tensor pipe."""
    st = status.tolist()
    return (st[2] & 0xFFFFFFFF) | ((st[3] & 0xFFFFFFFF) << 32)


def _pooled_blocks(x):
    """bf16 means of the 64-row blocks of ``x [B,H,n,128]`` -> ``[B,H,ceil(n/64),128]``."""
    B, H, n, D = x.shape
    x = x if x.stride(3) == 1 else x.contiguous()
    out = torch.empty((B, H, (n + 63) // 64, D), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_cabi.lib().minf_block_sparse_pool(_cabi.ptr(x), _cabi.strides3(x), B, H, n, _cabi.ptr(out),
                                                       _cabi.stream_ptr(x.device)))
    return out


def ring_prefill_attention(q_loc, k_loc, v_loc, n_ctx: int, pattern, group=None, block_sparse_top_k: int = 100):
    """Sequence-sharded attention of one layer with a per-head pattern table
    (``modules.minference_forward.LayerPattern``).  Vertical-slash heads use the distributed
    estimator and windowed plans; block-sparse heads pool their local Q and K, all-gather the
    pooled keys (``n_ctx/64`` vectors per KV head) and select their blocks locally; A-shape heads
    need no index.  All heads run in the same launches."""
    _cabi.require_cuda(q_loc, k_loc, v_loc)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    c = chunk_size(n_ctx, world)
    dev = q_loc.device
    B, H = q_loc.shape[0], q_loc.shape[1]
    L = _cabi.lib()
    chunks = owned_chunks(rank, world)
    v_idx, cap_v, cap_s = None, (pattern.cap_v if pattern.any_vs else 0), pattern.cap_s
    plans = []
    if pattern.any_vs:
        v_idx, s_idx, nnz_v, nnz_s = ring_vertical_slash_estimate(
            q_loc, k_loc, n_ctx, pattern.vertical_size, pattern.slash_size, group, cap_v=pattern.cap_v, cap_s=pattern.cap_s)
        for qc in chunks:
            plans.append(build_plan_window(v_idx, s_idx, nnz_v, nnz_s, n_ctx, qc * c, c))
    elif pattern.any_bs:
        for qc in chunks:
            plan = torch.empty(L.minf_plan_bytes_window(B, H, qc * c, c, cap_v, cap_s), dtype=torch.uint8, device=dev)
            plans.append((plan, _cabi.new_status(dev)))
    else:
        plans = [(None, _cabi.new_status(dev)) for _ in chunks]
    if pattern.any_bs:
        k_pool = _pooled_blocks(k_loc)                               # [B, Hkv, 2c/64, 128], this rank's two chunks
        gathered = [torch.empty_like(k_pool) for _ in range(world)]
        dist.all_gather(gathered, k_pool, group=group)
        k_pool_all = zigzag_merge(gathered, world).contiguous()      # blocks of the whole sequence in order
        for qi, qc in enumerate(chunks):
            q_pool = _pooled_blocks(q_loc[:, :, qi * c:(qi + 1) * c])
            with torch.cuda.device(dev):
                _cabi.check(L.minf_block_sparse_select_window(
                    _cabi.ptr(q_pool), _cabi.ptr(k_pool_all), B, H, k_loc.shape[1], n_ctx, qc * c, c, int(block_sparse_top_k),
                    _cabi.ptr(pattern.block_select), cap_v, cap_s, _cabi.ptr(plans[qi][0]), _cabi.stream_ptr(dev)))

    def attn_fn(q, k, v, qi, q_pos0, kv_pos0, carry, out):
        plan, status = plans[qi]
        attention_window(q, k, v, n_ctx, q_pos0, kv_pos0, plan, v_idx, cap_s, status,
                         head_mode=pattern.head_mode, head_param=pattern.head_param, cap_v=cap_v, carry=carry, out=out)

    out = ring_attention(q_loc, k_loc, v_loc, n_ctx, attn_fn, group, fused_merge=True)
    for _, status in plans:
        _cabi.raise_on_status(status, "ring_prefill_attention")
    return out
