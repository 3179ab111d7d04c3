"""Block-sparse attention (mirrors minference/ops/block_sparse_flash_attention.py)."""
from __future__ import annotations

import torch

from .. import _cabi
from ..cuda import _status_checks_enabled
from .sparse_forward import SparsePlan, sparse_attention_forward


def _rows_pad(n: int) -> int:
    # the reference pads by 64 - (n & 63): one whole extra block when n is a multiple of 64
    # (ops/block_sparse_flash_attention.py:178)
    return (n + (64 - (n & 63))) // 64


def build_block_sparse_plan(query, key, top_k: int, plan: SparsePlan | None = None,
                            head_select: torch.Tensor | None = None, return_block_index: bool = False):
    """Top-k block selection for every (selected) head; fills ``plan`` (created when None)."""
    B, H, N, D = query.shape
    Hkv = key.shape[1]
    dev = query.device
    L = _cabi.lib()
    k_eff = min(top_k, _rows_pad(N))
    if plan is None:
        nbytes = L.minf_plan_bytes(B, H, N, 0, k_eff)
        plan = SparsePlan(plan=torch.empty(nbytes, dtype=torch.uint8, device=dev), v_idx=None, cap_v=0,
                          cap_s=k_eff, context_size=N, batch=B, heads=H, status=_cabi.new_status(dev))
    scratch = torch.empty(L.minf_block_sparse_scratch_bytes(B, H, Hkv, N), dtype=torch.uint8, device=dev)
    bidx = torch.empty((B, H, _rows_pad(N), k_eff), dtype=torch.int32, device=dev) if return_block_index else None
    with torch.cuda.device(dev):
        _cabi.check(L.minf_block_sparse_build_plan(
            _cabi.ptr(query), _cabi.ptr(key), _cabi.strides3(query), _cabi.strides3(key),
            B, H, Hkv, N, D, int(top_k), _cabi.ptr(head_select), plan.cap_v, plan.cap_s,
            _cabi.ptr(plan.plan), _cabi.ptr(bidx), _cabi.ptr(scratch), _cabi.ptr(plan.status),
            _cabi.stream_ptr(dev)))
    return (plan, bidx) if return_block_index else plan


def _build_block_index(query, key, top_k, block_size_M: int = 64, block_size_N: int = 64):
    """Reference-format ``[B,H,rows_pad,top_k]`` sorted block ids
    (ops/block_sparse_flash_attention.py:151-166).  Unlike the reference, which is handed
    tensors already padded by its caller, this takes the unpadded tensors."""
    assert block_size_M == 64 and block_size_N == 64
    return build_block_sparse_plan(query, key, top_k, return_block_index=True)[1]


def block_sparse_attention(
    query: torch.Tensor,  # [BATCH, N_HEADS, N_CTX, D_HEAD]
    key: torch.Tensor,    # [BATCH, N_HEADS or N_KV_HEADS, N_CTX, D_HEAD]
    value: torch.Tensor,
    top_k: int,
    block_size_M: int = 64,
    block_size_N: int = 64,
):
    """Same call as the reference (ops/block_sparse_flash_attention.py:169-186)."""
    assert block_size_M == 64 and block_size_N == 64
    _cabi.require_cuda(query, key, value)
    if query.dtype != torch.bfloat16:
        raise _cabi.MInferB200Error(f"bf16 inputs required (got {query.dtype})")
    q = query if query.stride(3) == 1 else query.contiguous()
    k = key if key.stride(3) == 1 else key.contiguous()
    plan = build_block_sparse_plan(q, k, top_k)
    out = sparse_attention_forward(q, k, value, plan)
    if _status_checks_enabled():
        _cabi.raise_on_status(plan.status, "block_sparse_attention")
    return out
