"""Per-head dynamic sparse prefill (mirrors minference/modules/minference_forward.py:594-674).

The reference loops over heads in Python and runs a dozen torch ops plus three kernels per
head.  Here the whole layer is five launches: two estimator passes, the top-k select, the
plan build and the attention forward, each covering every head.
"""
from __future__ import annotations

import math

import torch

from .. import _cabi
from ..cuda import _status_checks_enabled
from ..ops.block_sparse_flash_attention import _rows_pad, build_block_sparse_plan
from ..ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
from ..ops.sparse_forward import SparsePlan, sparse_attention_forward

last_q = 64
BLOCK_SPARSE_TOPK = 100            # fixed in the reference (minference_forward.py:616-618)
DEFAULT_PATTERN = ("vertical_and_slash", 1000, 6096, 1)     # (:621)


def clamp_budgets(n: int, vertical_size: int, slash_size: int):
    """Budget clamping of the reference (:600)."""
    return min(n, max(vertical_size, 30)), min(n, max(slash_size, 50))


def vertical_slash_estimate(query, key, vertical_size, slash_size, cap_v=None, cap_s=None,
                            return_scores: bool = False):
    """Estimate vertical and slash indices for all heads at once.

    ``vertical_size`` / ``slash_size``: int, or int32 tensors ``[B*H]`` on the device (a
    negative entry skips that head).  Returns ``(v_idx [B,H,cap_v] ascending, s_idx
    [B,H,cap_s] descending offsets, nnz_v [B*H], nnz_s [B*H])`` int32.
    """
    _cabi.require_cuda(query, key)
    B, H, N, D = query.shape
    Hkv = key.shape[1]
    dev = query.device
    if isinstance(vertical_size, int):
        cv, cs = clamp_budgets(N, vertical_size, slash_size)
        cap_v, cap_s = cap_v or cv, cap_s or cs
        vertical_size = torch.full((B * H,), vertical_size, dtype=torch.int32, device=dev)
        slash_size = torch.full((B * H,), slash_size, dtype=torch.int32, device=dev)
    assert cap_v and cap_s
    L = _cabi.lib()
    q = query if query.stride(3) == 1 else query.contiguous()
    k = key if key.stride(3) == 1 else key.contiguous()
    v_idx = torch.empty((B, H, cap_v), dtype=torch.int32, device=dev)
    s_idx = torch.empty((B, H, cap_s), dtype=torch.int32, device=dev)
    nnz_v = torch.empty((B * H,), dtype=torch.int32, device=dev)
    nnz_s = torch.empty((B * H,), dtype=torch.int32, device=dev)
    vs = torch.empty((B, H, N), dtype=torch.float32, device=dev) if return_scores else None
    ss = torch.empty((B, H, N), dtype=torch.float32, device=dev) if return_scores else None
    scratch = torch.empty(L.minf_vs_estimate_scratch_bytes(B, H, N), dtype=torch.uint8, device=dev)
    status = _cabi.new_status(dev)
    with torch.cuda.device(dev):
        _cabi.check(L.minf_vs_estimate(
            _cabi.ptr(q), _cabi.ptr(k), _cabi.strides3(q), _cabi.strides3(k), B, H, Hkv, N, D,
            _cabi.ptr(vertical_size), _cabi.ptr(slash_size), cap_v, cap_s,
            _cabi.ptr(v_idx), _cabi.ptr(s_idx), _cabi.ptr(nnz_v), _cabi.ptr(nnz_s),
            _cabi.ptr(vs), _cabi.ptr(ss), _cabi.ptr(scratch), _cabi.ptr(status), _cabi.stream_ptr(dev)))
    if _status_checks_enabled():
        _cabi.raise_on_status(status, "vertical_slash_estimate")
    if return_scores:
        return v_idx, s_idx, nnz_v, nnz_s, vs, ss
    return v_idx, s_idx, nnz_v, nnz_s


def vertical_slash_select(vertical_scores, slash_scores, vertical_size, slash_size, cap_v: int, cap_s: int,
                          rules: str = "online"):
    """Per-head top-k over score arrays ``[B,H,N]`` (as ``vertical_slash_estimate(return_scores=True)`` returns
    them) under one of the reference's rule sets: ``online`` (first 30 columns and the 100 nearest diagonals
    forced, budgets raised to 30 / 50), ``static`` (30 diagonals forced) or ``search`` (30 diagonals forced,
    budgets taken as they are).  Budgets: int32 tensors ``[B*H]``."""
    B, H, N = vertical_scores.shape
    dev = vertical_scores.device
    L = _cabi.lib()
    v_idx = torch.empty((B, H, cap_v), dtype=torch.int32, device=dev)
    s_idx = torch.empty((B, H, cap_s), dtype=torch.int32, device=dev)
    nnz_v = torch.empty((B * H,), dtype=torch.int32, device=dev)
    nnz_s = torch.empty((B * H,), dtype=torch.int32, device=dev)
    scratch = torch.empty(L.minf_vs_select_scratch_bytes(B, H, N), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(L.minf_vs_select(
            _cabi.ptr(vertical_scores), _cabi.ptr(slash_scores), B, H, N, _cabi.ptr(vertical_size), _cabi.ptr(slash_size),
            cap_v, cap_s, _cabi.ptr(v_idx), _cabi.ptr(s_idx), _cabi.ptr(nnz_v), _cabi.ptr(nnz_s),
            *_cabi.SELECT_RULES[rules], _cabi.ptr(scratch), _cabi.stream_ptr(dev)))
    return v_idx, s_idx, nnz_v, nnz_s


class LayerPattern:
    """Per-head pattern of one layer, parsed once from the JSON table entry
    ``{str(head): [type, vertical, slash, score]}`` (configs/*.json of the reference)."""

    def __init__(self, layer_cfg: dict, num_heads: int, n_ctx: int, ratio: float | None, device, head_offset: int = 0):
        """``head_offset``: index of this process's first head in the table -- under tensor parallelism a rank
        holds ``num_heads`` consecutive heads starting at ``rank * num_heads`` (minference_forward.py:902)."""
        modes, params, vsz, ssz, bsel = [], [], [], [], []
        self.cap_v, self.cap_s = 1, 1
        self.any_vs = self.any_bs = False
        for h in range(num_heads):
            ty, v, s, _ = layer_cfg.get(str(head_offset + h), DEFAULT_PATTERN)
            if ratio is not None:
                v, s = int(v * ratio), int(s * ratio)
            if ty == "stream_llm":          # streaming_forward(q, k, v, n_init=v, n_local=s) (:626-631)
                modes.append(_cabi.MODE_ASHAPE); params.append((v, s)); vsz.append(-1); ssz.append(-1); bsel.append(0)
            elif ty == "vertical_and_slash":
                cv, cs = clamp_budgets(n_ctx, v, s)
                self.cap_v, self.cap_s = max(self.cap_v, cv), max(self.cap_s, cs)
                self.any_vs = True
                modes.append(_cabi.MODE_PLAN); params.append((0, 0)); vsz.append(v); ssz.append(s); bsel.append(0)
            elif ty == "block_sparse":
                self.cap_s = max(self.cap_s, min(BLOCK_SPARSE_TOPK, _rows_pad(n_ctx)))
                self.any_bs = True
                modes.append(_cabi.MODE_PLAN); params.append((0, 0)); vsz.append(-1); ssz.append(-1); bsel.append(1)
            else:
                raise KeyError(ty)
        t = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
        self.head_mode, self.head_param = t(modes), t(params)
        self.vertical_size, self.slash_size, self.block_select = t(vsz), t(ssz), t(bsel)
        self.any_plan = self.any_vs or self.any_bs


_PATTERN_CACHE_ENTRIES = 256


def _layer_pattern(cfg: dict, layer_idx: int, num_heads: int, n_ctx: int, device, head_offset: int = 0) -> LayerPattern:
    """Device tables of one layer's pattern, parsed once per (layer, heads, length).  The cache lives inside the
    attention config it was built from (so it dies with it and never serves another model's table) and keeps the
    most recently used entries only."""
    ratio = cfg.get("minference_ratio") if "minference_ratio" in cfg else None
    cache = cfg.setdefault("_layer_patterns", {})
    key = (layer_idx, num_heads, n_ctx, ratio, str(device), head_offset)
    pat = cache.pop(key, None)
    if pat is None:
        pat = LayerPattern(cfg["best_pattern"][layer_idx], num_heads, n_ctx, ratio, device, head_offset)
        while len(cache) >= _PATTERN_CACHE_ENTRIES:
            cache.pop(next(iter(cache)))
    cache[key] = pat          # most recently used last
    return pat


def minference_prefill_forward(query_states, key_states, value_states, prefill_kwargs):
    """Same call as the reference (minference_forward.py:633-674): ``[B,H,N,D]`` in,
    ``[B,H,N,D]`` out.  ``key_states`` / ``value_states`` may carry either the query head
    count (already repeated, as the reference's caller passes them) or the KV head count.
    ``prefill_kwargs["head_offset"]`` (optional) is the table index of the first local head when the
    heads are sharded over tensor-parallel ranks.
    """
    cfg = prefill_kwargs["attn_forward_config"]
    starting_layer = cfg.get("starting_layer", 0)
    layer_idx = prefill_kwargs["layer_idx"]
    _cabi.require_cuda(query_states, key_states, value_states)
    B, H, N, D = query_states.shape
    assert B == 1, "the estimator of the reference is defined for batch 1 (as_strided view, :114)"
    dev = query_states.device
    is_search = cfg.get("is_search", False)
    if is_search:       # offline search: record this layer's best patterns, run the layer dense (:644-650, :661-666)
        from .pattern_search import search_and_record

        search_and_record(query_states, key_states, value_states, layer_idx,
                          prefill_kwargs.get("num_hidden_layers", 0), cfg.get("config_path"))

    if is_search or layer_idx < starting_layer:          # dense causal layers (:665-666)
        return dense_prefill_forward(query_states, key_states, value_states)

    pat = _layer_pattern(cfg, layer_idx, H, N, dev, int(prefill_kwargs.get("head_offset", 0)))
    plan = None
    if pat.any_plan:
        L = _cabi.lib()
        nbytes = L.minf_plan_bytes(B, H, N, pat.cap_v, pat.cap_s)
        plan = SparsePlan(plan=torch.empty(nbytes, dtype=torch.uint8, device=dev), v_idx=None, cap_v=pat.cap_v,
                          cap_s=pat.cap_s, context_size=N, batch=B, heads=H, status=_cabi.new_status(dev))
        if pat.any_vs:
            with _cabi.nvtx_range("minference:estimate"):
                v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(
                    query_states, key_states, pat.vertical_size, pat.slash_size, cap_v=pat.cap_v, cap_s=pat.cap_s)
            with _cabi.nvtx_range("minference:plan"):
                plan.v_idx = build_vertical_slash_plan_into(plan, v_idx, s_idx, nnz_v, nnz_s)
        if pat.any_bs:
            q = query_states if query_states.stride(3) == 1 else query_states.contiguous()
            k = key_states if key_states.stride(3) == 1 else key_states.contiguous()
            with _cabi.nvtx_range("minference:block_plan"):
                build_block_sparse_plan(q, k, BLOCK_SPARSE_TOPK, plan=plan, head_select=pat.block_select)
    with _cabi.nvtx_range("minference:attention"):
        out = sparse_attention_forward(query_states, key_states, value_states, plan,
                                       head_mode=pat.head_mode, head_param=pat.head_param)
    if _status_checks_enabled():
        _cabi.raise_on_status(plan.status if plan is not None else sparse_attention_forward.last_status,
                              "minference_prefill_forward")
    return out


def build_vertical_slash_plan_into(plan: SparsePlan, v_idx, s_idx, nnz_v, nnz_s):
    """Fill the vertical-slash heads of an existing plan buffer; returns ``v_idx``."""
    dev = v_idx.device
    seqlens = torch.full((plan.batch,), plan.context_size, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().minf_vs_build_plan(
            _cabi.ptr(seqlens), _cabi.ptr(v_idx), _cabi.ptr(s_idx), _cabi.ptr(nnz_v), _cabi.ptr(nnz_s),
            plan.batch, plan.heads, plan.context_size, plan.cap_v, plan.cap_s,
            _cabi.ptr(plan.plan), _cabi.ptr(plan.status), _cabi.stream_ptr(dev)))
    return v_idx


def static_prefill_forward(query_states, key_states, value_states, prefill_kwargs):
    """The reference's static variant (``vertical_and_slash_kernel_static``, minference_forward.py:418-437):
    the index lists are estimated once per layer -- by the first head that runs, with that head's budgets, the
    first 30 columns and only the 30 nearest diagonals forced -- and kept: every head of the layer, and every
    later prompt, attends through the same vertical columns and diagonals.  The lists live in the attention
    config (the reference keeps them on the attention module); a prompt of another length estimates again,
    since indices beyond the new length would point outside it.
    """
    cfg = prefill_kwargs["attn_forward_config"]
    layer_idx = prefill_kwargs["layer_idx"]
    _cabi.require_cuda(query_states, key_states, value_states)
    B, H, N, D = query_states.shape
    assert B == 1, "the estimator of the reference is defined for batch 1"
    dev = query_states.device
    cache = cfg.setdefault("_static_vs", {})
    entry = cache.get(layer_idx)
    if entry is None or entry[0] != N:
        table = cfg.get("best_pattern") or []
        layer_cfg = table[layer_idx] if layer_idx < len(table) else {}
        _, vs, ss, _ = layer_cfg.get("0", DEFAULT_PATTERN)
        q0, k0 = query_states[:, :1], key_states[:, :1]        # query head 0 reads KV head 0, repeated or not
        cap_v, cap_s = clamp_budgets(N, vs, ss)
        *_, vsc, ssc = vertical_slash_estimate(q0, k0, vs, ss, return_scores=True)
        budget = lambda x: torch.full((1,), x, dtype=torch.int32, device=dev)
        v_idx, s_idx, _, _ = vertical_slash_select(vsc, ssc, budget(vs), budget(ss), cap_v, cap_s, rules="static")
        entry = (N, v_idx.expand(B, H, -1).contiguous(), s_idx.expand(B, H, -1).contiguous())
        cache[layer_idx] = entry
    _, v_idx, s_idx = entry
    plan = build_vertical_slash_plan(v_idx, s_idx, N)
    out = sparse_attention_forward(query_states, key_states, value_states, plan)
    if _status_checks_enabled():
        _cabi.raise_on_status(plan.status, "static_prefill_forward")
    return out


def dense_prefill_forward(query_states, key_states, value_states):
    """Plain causal attention through the same kernel (an A-shape window as long as the sequence)."""
    H, N = query_states.shape[1], query_states.shape[2]
    dev = query_states.device
    mode = torch.full((H,), _cabi.MODE_ASHAPE, dtype=torch.int32, device=dev)
    param = torch.tensor([[0, N]] * H, dtype=torch.int32, device=dev)
    return sparse_attention_forward(query_states, key_states, value_states, None, head_mode=mode, head_param=param)
