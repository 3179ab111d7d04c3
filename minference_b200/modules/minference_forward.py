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


class LayerPattern:
    """Per-head pattern of one layer, parsed once from the JSON table entry
    ``{str(head): [type, vertical, slash, score]}`` (configs/*.json of the reference)."""

    def __init__(self, layer_cfg: dict, num_heads: int, n_ctx: int, ratio: float | None, device):
        modes, params, vsz, ssz, bsel = [], [], [], [], []
        self.cap_v, self.cap_s = 1, 1
        self.any_vs = self.any_bs = False
        for h in range(num_heads):
            ty, v, s, _ = layer_cfg.get(str(h), DEFAULT_PATTERN)
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


_PATTERN_CACHE: dict = {}


def _layer_pattern(cfg: dict, layer_idx: int, num_heads: int, n_ctx: int, device) -> LayerPattern:
    ratio = cfg.get("minference_ratio") if "minference_ratio" in cfg else None
    key = (id(cfg["best_pattern"]), layer_idx, num_heads, n_ctx, ratio, str(device))
    pat = _PATTERN_CACHE.get(key)
    if pat is None:
        pat = LayerPattern(cfg["best_pattern"][layer_idx], num_heads, n_ctx, ratio, device)
        _PATTERN_CACHE[key] = pat
    return pat


def minference_prefill_forward(query_states, key_states, value_states, prefill_kwargs):
    """Same call as the reference (minference_forward.py:633-674): ``[B,H,N,D]`` in,
    ``[B,H,N,D]`` out.  ``key_states`` / ``value_states`` may carry either the query head
    count (already repeated, as the reference's caller passes them) or the KV head count.
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
        mode = torch.full((H,), _cabi.MODE_ASHAPE, dtype=torch.int32, device=dev)
        param = torch.tensor([[0, N]] * H, dtype=torch.int32, device=dev)
        return sparse_attention_forward(query_states, key_states, value_states, None, head_mode=mode, head_param=param)

    pat = _layer_pattern(cfg, layer_idx, H, N, dev)
    plan = None
    if pat.any_plan:
        L = _cabi.lib()
        nbytes = L.minf_plan_bytes(B, H, N, pat.cap_v, pat.cap_s)
        plan = SparsePlan(plan=torch.empty(nbytes, dtype=torch.uint8, device=dev), v_idx=None, cap_v=pat.cap_v,
                          cap_s=pat.cap_s, context_size=N, batch=B, heads=H, status=_cabi.new_status(dev))
        if pat.any_vs:
            v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(
                query_states, key_states, pat.vertical_size, pat.slash_size, cap_v=pat.cap_v, cap_s=pat.cap_s)
            vs_plan = build_vertical_slash_plan_into(plan, v_idx, s_idx, nnz_v, nnz_s)
            plan.v_idx = vs_plan
        if pat.any_bs:
            q = query_states if query_states.stride(3) == 1 else query_states.contiguous()
            k = key_states if key_states.stride(3) == 1 else key_states.contiguous()
            build_block_sparse_plan(q, k, BLOCK_SPARSE_TOPK, plan=plan, head_select=pat.block_select)
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
