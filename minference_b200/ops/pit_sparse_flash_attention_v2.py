"""Vertical-slash sparse attention (mirrors minference/ops/pit_sparse_flash_attention_v2.py)."""
from __future__ import annotations

import torch

from .. import _cabi
from ..cuda import _status_checks_enabled, convert_vertical_slash_indexes  # noqa: F401  (re-export like the reference)
from .sparse_forward import SparsePlan, sparse_attention_forward


def build_vertical_slash_plan(v_idx: torch.Tensor, s_idx: torch.Tensor, context_size: int,
                              nnz_v: torch.Tensor | None = None, nnz_s: torch.Tensor | None = None,
                              seqlens: torch.Tensor | None = None) -> SparsePlan:
    """Compact plan from sorted int32 ``v_idx [B,H,cap_v]`` (ascending) and ``s_idx [B,H,cap_s]``
    (descending offsets); ``nnz_v`` / ``nnz_s`` int32 ``[B*H]`` give per-head live lengths."""
    B, H, cap_v = v_idx.shape
    cap_s = s_idx.shape[2]
    dev = v_idx.device
    L = _cabi.lib()
    nbytes = L.minf_plan_bytes(B, H, context_size, cap_v, cap_s)
    plan = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    status = _cabi.new_status(dev)
    if seqlens is None:
        seqlens = torch.full((B,), context_size, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(L.minf_vs_build_plan(
            _cabi.ptr(seqlens), _cabi.ptr(v_idx), _cabi.ptr(s_idx), _cabi.ptr(nnz_v), _cabi.ptr(nnz_s),
            B, H, context_size, cap_v, cap_s, _cabi.ptr(plan), _cabi.ptr(status), _cabi.stream_ptr(dev)))
    return SparsePlan(plan=plan, v_idx=v_idx, cap_v=cap_v, cap_s=cap_s, context_size=context_size,
                      batch=B, heads=H, status=status, s_idx=s_idx)


def vertical_slash_sparse_attention(
    query: torch.Tensor,  # [BATCH, N_HEADS, N_CTX, D_HEAD]
    key: torch.Tensor,    # [BATCH, N_HEADS or N_KV_HEADS, N_CTX, D_HEAD]
    value: torch.Tensor,  # [BATCH, N_HEADS or N_KV_HEADS, N_CTX, D_HEAD]
    v_idx: torch.Tensor,  # [BATCH, N_HEADS, NNZ_V]
    s_idx: torch.Tensor,  # [BATCH, N_HEADS, NNZ_S]
    block_size_M: int = 64,
    block_size_N: int = 64,
):
    """Same call as the reference (ops/pit_sparse_flash_attention_v2.py:195-242).

    Index preparation follows :218-219 (int32 cast, vertical ascending, slash descending);
    no padding copies are made (the kernel masks the ragged tail itself) and K/V may keep
    their un-repeated KV heads.
    """
    assert block_size_M == 64 and block_size_N == 64
    _cabi.require_cuda(query, key, value, v_idx, s_idx)
    batch_size, num_heads, context_size, head_dim = query.shape
    v_sorted = v_idx.to(torch.int32).reshape((batch_size, num_heads, -1)).sort(dim=-1, descending=False)[0]
    s_sorted = s_idx.to(torch.int32).reshape((batch_size, num_heads, -1)).sort(dim=-1, descending=True)[0]
    plan = build_vertical_slash_plan(v_sorted.contiguous(), s_sorted.contiguous(), context_size)
    out = sparse_attention_forward(query, key, value, plan)
    if _status_checks_enabled():
        _cabi.raise_on_status(plan.status, "vertical_slash_sparse_attention")
    return out


def dilated_sparse_attention(query, key, value, kind: str):
    """The fixed index sets of the reference's ``dialted`` variants
    (modules/minference_forward.py:365-379): the first 1024 keys as vertical lines and
    ``dilated1`` every second of the 8192 nearest diagonals, ``dilated2`` the 2048 nearest
    diagonals plus every second of the next 4096."""
    n = query.shape[2]
    dev = query.device
    v_idx = torch.arange(0, min(1024, n), device=dev)[None, None, :].expand(query.shape[0], query.shape[1], -1)
    pos = torch.arange(0, n, device=dev)
    if kind == "dilated1":
        pos = pos[-8192::2]
    elif kind == "dilated2":
        pos = torch.cat([pos[-2048:], pos[-6144:-2048:2]], 0)
    else:
        raise KeyError(kind)
    s_idx = ((n - 1) - pos)[None, None, :].expand(query.shape[0], query.shape[1], -1)
    return vertical_slash_sparse_attention(query, key, value, v_idx, s_idx)
