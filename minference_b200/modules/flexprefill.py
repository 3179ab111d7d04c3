"""FlexPrefill: per-head adaptive block budgets from the last query block (mirrors minference/modules/flexprefill.py
of the reference: ``get_active_blocks`` :953-1067, ``flex_prefill_attention`` :1070-1112, ``flexprefill_forward``
:1115-1131).

The reference takes the softmax of the last ``block_size`` queries against all keys, sums it along columns and
diagonals, asks how many of the best tokens it takes to cover ``gamma`` of the mass (that sets each head's budget of
vertical and slash *blocks*), pools the sums to blocks and takes the best ones; heads whose pooled column profile is
close (square-root Jensen-Shannon distance below ``tau``) to the profile of mean-pooled keys fall back to the smallest
budget plus a block-sparse selection over mean-pooled queries and keys.  The selected blocks are attended block-wise.

Here the column and diagonal sums come from the estimator kernels of this package (two groups of 64 queries, no
``[block_size, N]`` tensor), the budget logic is a few small torch calls on ``[B, H, N]`` score arrays, the block set
becomes merged token ranges (``minf_block_mask_build_plan``) and the attention kernel is the one every other pattern uses.
Tensors are ``[B, H, N, D]`` in ``flexprefill_forward`` and ``[B, N, H, D]`` in ``flex_prefill_attention``, as in
the reference.
"""
from __future__ import annotations

import math

import torch

from .. import _cabi
from ..cuda import _status_checks_enabled
from ..ops.sparse_forward import SparsePlan, sparse_attention_forward

SUPPORTED_BLOCK_SIZES = (64, 128)


def last_block_scores(query, key, block_size: int):
    """``(vertical [B,H,N], slash_by_offset [B,H,N], last_q [B,H,block_size,D])``: column means and diagonal means of
    ``softmax(last_q k^T)`` over the last ``block_size`` queries, ``last_q = q[-block_size:] / sqrt(D)`` rounded to
    bf16 first and the product rounded to bf16 once, as :968-993.  Entry ``o`` of the slash array is the diagonal at
    distance ``o`` from the main one (the reference's index ``j`` is ``N - 1 - o``)."""
    B, H, N, D = query.shape
    Hkv = key.shape[1]
    dev = query.device
    L = _cabi.lib()
    last_q = (query[:, :, -block_size:, :] / math.sqrt(D)).contiguous()
    k = key if key.stride(3) == 1 else key.contiguous()
    vertical = torch.zeros((B, H, N), dtype=torch.float32, device=dev)
    slash = torch.zeros((B, H, N), dtype=torch.float32, device=dev)
    status = _cabi.new_status(dev)
    groups = block_size // 64
    for g in range(groups):
        # queries at positions ctx-64 .. ctx-1 see the first ctx keys; the last group is the usual estimator
        ctx = N - 64 * (groups - 1 - g)
        q_g = last_q[:, :, 64 * g:64 * (g + 1), :].contiguous()
        k_g = k[:, :, :ctx]
        blocks = L.minf_vs_scores_blocks(ctx)
        stats = torch.empty((B * H, 64, blocks, 2), dtype=torch.float32, device=dev)
        row_stats = torch.empty((B * H, 64, 2), dtype=torch.float32, device=dev)
        scores = torch.zeros((2, B, H, ctx), dtype=torch.float32, device=dev)

        def run(pass_, rs, vert, sl):
            with torch.cuda.device(dev):
                _cabi.check(L.minf_vs_scores_pass_divisor(
                    pass_, _cabi.ptr(q_g), _cabi.ptr(k_g), _cabi.strides3(q_g), _cabi.strides3(k_g),
                    B, H, Hkv, ctx, ctx, 0, D, 1.0, _cabi.ptr(stats), 0, blocks, _cabi.ptr(rs),
                    _cabi.ptr(vert), _cabi.ptr(sl), _cabi.ptr(status), _cabi.stream_ptr(dev)))

        run(1, None, None, None)
        with torch.cuda.device(dev):
            _cabi.check(L.minf_vs_scores_combine(_cabi.ptr(stats), B, H, blocks, _cabi.ptr(row_stats), _cabi.stream_ptr(dev)))
        run(2, row_stats, scores[0], scores[1])
        vertical[:, :, :ctx] += scores[0]
        slash[:, :, :ctx] += scores[1]
    if _status_checks_enabled():
        _cabi.raise_on_status(status, "flexprefill estimator")
    return vertical / block_size, slash / block_size, last_q


def _sum_pool(x: torch.Tensor, kernel: int) -> torch.Tensor:
    n = x.shape[-1]
    x = torch.nn.functional.pad(x, (0, math.ceil(n / kernel) * kernel - n))
    return x.view(*x.shape[:-1], -1, kernel).sum(-1)


def _mean_pool_rows(x: torch.Tensor, kernel: int, short_block_by_length: bool) -> torch.Tensor:
    """``[B,H,N,D] -> [B,H,nb,D]`` in the input dtype, fp32 accumulation.  The keys' pooling divides a short last
    block by its own length (:702-703); the queries' pads with zeros, divides by the block size and rescales the
    last mean in bf16 (:1052-1058)."""
    B, H, N, D = x.shape
    nb = math.ceil(N / kernel)
    full = N // kernel
    parts = []
    if full:
        parts.append(torch.sum(x[:, :, :full * kernel].reshape(B, H, full, kernel, D), dim=3, dtype=torch.float32) / kernel)
    if nb > full:
        tail = torch.sum(x[:, :, full * kernel:], dim=2, keepdim=True, dtype=torch.float32)
        parts.append(tail / ((N - full * kernel) if short_block_by_length else kernel))
    out = torch.cat(parts, dim=2).to(x.dtype)
    if nb > full and not short_block_by_length:
        out[:, :, -1] = out[:, :, -1] * kernel / (N - full * kernel)
    return out


def _score_cover_topk(x: torch.Tensor, score: float) -> torch.Tensor:
    csum = torch.cumsum(torch.sort(x, dim=-1, descending=True).values, dim=-1)          # :880-883
    return torch.sum(csum <= score, dim=-1) + 1


def _sqrt_js(p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    m = (p + q) / 2                                                                        # :946-950
    return torch.sqrt(0.5 * (p * torch.log(p / m)).sum(-1) + 0.5 * (q * torch.log(q / m)).sum(-1))


@torch.no_grad()
def active_block_mask(query, key, block_size: int, gamma: float, min_budget: int, max_budget: int, tau: float = 0.0,
                      return_details: bool = False):
    """The block set of ``get_active_blocks`` (:953-1067) as a boolean matrix ``[B,H,nb,nb]`` on the device
    (entry (i, j): query block i attends key block j; only j <= i is set).  Budgets are in blocks.  Query head h reads
    KV head ``h // (H / Hkv)``."""
    vertical, slash_o, last_q = last_block_scores(query, key, block_size)
    return select_blocks(vertical, slash_o, last_q, query, key, block_size, gamma, min_budget, max_budget, tau, return_details)


@torch.no_grad()
def select_blocks(vertical, slash_o, last_q, query, key, block_size: int, gamma: float, min_budget: int, max_budget: int,
                  tau: float = 0.0, return_details: bool = False):
    """From the column means ``vertical [B,H,N]`` and diagonal means ``slash_o [B,H,N]`` (by distance from the main
    diagonal) of the last query block to the block set: budgets, pooling, the Jensen-Shannon test, top-k and the
    block-sparse fallback (:994-1066).  Plain torch on whatever device the tensors live on."""
    B, H, N, D = query.shape
    Hkv = key.shape[1]
    rep = H // Hkv
    dev = query.device
    nb = math.ceil(N / block_size)
    max_budget = min(max_budget, nb)
    slash = slash_o.flip(-1)                                       # the reference's index j = N-1-o
    n_vert = (_score_cover_topk(vertical, gamma) // 128 + 1).clamp(min_budget, max_budget)      # :995-1000
    n_slash = (_score_cover_topk(slash, gamma) // 128 + 1).clamp(min_budget, max_budget)
    vertical = _sum_pool(vertical, block_size)                     # :1002-1003
    slash = _sum_pool(slash, block_size)
    avg_k = _mean_pool_rows(key, block_size, True)                 # [B,Hkv,nb,D]  :1005-1008
    avg_k_h = avg_k.repeat_interleave(rep, dim=1) if rep > 1 else avg_k
    avg_qk = torch.einsum("bhd,bhjd->bhj", last_q.mean(2), avg_k_h)                              # :1009-1012
    avg_qk = torch.softmax(avg_qk, dim=-1, dtype=torch.float32)
    js = _sqrt_js(avg_qk, vertical)
    block_sparse = js < tau                                        # :1013-1016
    n_vert = torch.where(block_sparse, torch.full_like(n_vert, min_budget), n_vert)
    n_slash = torch.where(block_sparse, torch.full_like(n_slash, min_budget), n_slash)
    vertical[..., :1] = torch.inf                                  # :1018-1019
    slash[..., -1:] = torch.inf
    # the best n blocks per head as 0/1 rows over blocks (:1021-1046); ties: torch.topk's choice, as in the reference.
    # No budget exceeds max_budget, so that many candidates are enough and nothing has to be read back for it.
    k_max = max_budget
    rank = torch.arange(k_max, device=dev)

    def chosen(scores, budget):
        idx = scores.topk(k_max, dim=-1).indices
        sel = torch.zeros((B, H, nb), dtype=torch.bool, device=dev)
        return sel.scatter_(-1, idx, rank[None, None, :] < budget[..., None])

    sel_v = chosen(vertical, n_vert)                               # key blocks
    sel_d = chosen(slash, n_slash).flip(-1)                        # pooled entry b <-> block diagonal nb-1-b
    ii = torch.arange(nb, device=dev)
    dist = ii[:, None] - ii[None, :]
    tril = dist >= 0
    mask = (sel_v[:, :, None, :] | sel_d[:, :, dist.clamp(min=0)]) & tril                       # :903-921
    heads = block_sparse.view(-1).nonzero().view(-1)               # :1049-1066, all such heads of a group at once
    if heads.numel():
        avg_q = _mean_pool_rows(query, block_size, False).view(B * H, nb, D)
        kv_of = (heads // H) * Hkv + (heads % H) // rep
        flat = mask.view(B * H, nb * nb)
        per_group = max(1, (1 << 27) // (nb * nb))                 # heads whose nb x nb score matrices fit 512 MB
        for g0 in range(0, heads.numel(), per_group):
            hs, ks = heads[g0:g0 + per_group], kv_of[g0:g0 + per_group]
            attn = torch.einsum("hid,hjd->hij", avg_q[hs] / math.sqrt(D), avg_k.view(B * Hkv, nb, D)[ks])
            attn = torch.softmax(attn.masked_fill_(~tril, float("-inf")), dim=-1, dtype=torch.float32).view(hs.numel(), -1)
            vals, idx = torch.sort(attn, dim=-1, descending=True)
            keep = torch.cumsum(vals, dim=-1) <= gamma * nb        # :886-890
            flat[hs] |= torch.zeros_like(keep).scatter_(1, idx, keep)
    if return_details:
        return mask, {"n_vertical": n_vert, "n_slash": n_slash, "block_sparse": block_sparse, "js": js,
                      "vertical_pooled": vertical, "slash_pooled": slash}
    return mask


def build_block_mask_plan(mask: torch.Tensor, context_size: int, block_size: int) -> SparsePlan:
    """Attention plan of a block set ``[B,H,nb,nb]`` (bool or uint8 on the device)."""
    B, H, nb, _ = mask.shape
    dev = mask.device
    m8 = mask.to(torch.uint8).contiguous()
    lower = torch.tril(m8)
    starts = lower.clone()
    starts[..., 1:] &= ~lower[..., :-1] & 1                        # a one whose left neighbour is zero starts a run
    cap_s = max(int(starts.sum(-1).max().item()), 1)
    L = _cabi.lib()
    plan = SparsePlan(plan=torch.empty(L.minf_plan_bytes(B, H, context_size, 0, cap_s), dtype=torch.uint8, device=dev),
                      v_idx=None, cap_v=0, cap_s=cap_s, context_size=context_size, batch=B, heads=H,
                      status=_cabi.new_status(dev))
    with torch.cuda.device(dev):
        _cabi.check(L.minf_block_mask_build_plan(_cabi.ptr(lower), B, H, context_size, block_size, cap_s,
                                                 _cabi.ptr(plan.plan), _cabi.ptr(plan.status), _cabi.stream_ptr(dev)))
    return plan


@torch.no_grad()
def flex_prefill_attention(q, k, v, gamma: float, tau: float = 0, min_budget: int | None = None,
                           max_budget: int | None = None, gqa_interleave: bool = False,
                           softmax_scale: float | None = None, block_size: int = 128):
    """Same call as the reference (:1070-1112): ``q [B,N,H,D]``, ``k, v [B,N,Hkv,D]`` -> ``[B,N,H,D]``.  Budgets are in
    tokens and rounded up to blocks.  ``gqa_interleave`` (query head h reading KV head ``h % Hkv``) is not built."""
    if gqa_interleave and k.shape[2] != q.shape[2]:
        raise _cabi.MInferB200Error("gqa_interleave is not supported; repeat K/V or use the grouped head order")
    out = _flex_bhnd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gamma, tau, min_budget, max_budget,
                     softmax_scale, block_size)
    return out.transpose(1, 2)


def _flex_bhnd(q, k, v, gamma, tau, min_budget, max_budget, softmax_scale, block_size):
    _cabi.require_cuda(q, k, v)
    if block_size not in SUPPORTED_BLOCK_SIZES:
        raise _cabi.MInferB200Error(f"block_size must be one of {SUPPORTED_BLOCK_SIZES} (got {block_size})")
    N = q.shape[2]
    min_budget = 1 if min_budget is None else min_budget
    max_budget = 2147483647 if max_budget is None else max_budget
    if N <= max(2 * block_size, math.ceil(min_budget / block_size) * block_size):              # :1087-1088
        from .minference_forward import dense_prefill_forward

        if softmax_scale is not None:
            raise _cabi.MInferB200Error("softmax_scale is only taken on the sparse path")
        return dense_prefill_forward(q, k, v)
    mask = active_block_mask(q, k, block_size, gamma, math.ceil(min_budget / block_size),
                             math.ceil(max_budget / block_size), tau)
    plan = build_block_mask_plan(mask, N, block_size)
    out = sparse_attention_forward(q, k, v, plan, sm_scale=softmax_scale)
    if _status_checks_enabled():
        _cabi.raise_on_status(plan.status, "flex_prefill_attention")
    return out


def flexprefill_forward(q, k, v, config):
    """The prefill operator of ``attn_type="flexprefill"`` (:1115-1131): ``[B,H,N,D]`` in and out, parameters from
    ``config["attn_forward_config"]`` with the reference's defaults (gamma 0.9, tau 0.1, block size 128).  The
    reference hands ``block_size`` to its attention function in the position of ``gqa_interleave`` (:1128-1130), so
    there the configured block size never takes effect and 128 is always used; here it is honoured."""
    cfg = config["attn_forward_config"]
    return _flex_bhnd(q, k, v, cfg.get("gamma", 0.9), cfg.get("tau", 0.1), cfg.get("min_budget", None),
                      cfg.get("max_budget", None), None, cfg.get("block_size", 128))
