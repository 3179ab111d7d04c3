"""Common launcher of the sparse attention forward kernel (all three head patterns)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _cabi


@dataclass
class SparsePlan:
    """Device-resident index plan of one layer (see csrc/plan_layout.h)."""
    plan: torch.Tensor | None
    v_idx: torch.Tensor | None
    cap_v: int
    cap_s: int
    context_size: int
    batch: int
    heads: int
    status: torch.Tensor
    s_idx: torch.Tensor | None = None      # the slash lists the plan was built from (kept for checks)

    def count_tiles(self) -> int:
        """64x64 tiles the reference kernel would compute for this index set."""
        out = torch.zeros(1, dtype=torch.int64, device=self.plan.device)
        with torch.cuda.device(self.plan.device):
            _cabi.check(_cabi.lib().minf_plan_count_tiles(
                _cabi.ptr(self.plan), self.batch, self.heads, self.context_size, self.cap_v, self.cap_s,
                _cabi.ptr(out), _cabi.stream_ptr(self.plan.device)))
        return int(out.item())


def _as_bhnd(t: torch.Tensor) -> torch.Tensor:
    if t.stride(3) != 1 or any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def sparse_attention_forward(query, key, value, plan: SparsePlan | None, head_mode=None, head_param=None,
                             sm_scale: float | None = None, out: torch.Tensor | None = None, return_lse: bool = False):
    """Launch ``minf_sparse_attention_fwd`` on the current stream and return ``[B,H,N,D]``.

    ``return_lse=True`` also returns the per-row base-2 log-sum-exp of the scaled logits over the
    keys the pattern selects, ``[B,H,N]`` fp32 (-inf for a row with no visible key)."""
    if query.dtype != torch.bfloat16:
        raise _cabi.MInferB200Error(f"bf16 inputs required (got {query.dtype}); there is no other kernel")
    if not (key.dtype == value.dtype == query.dtype):
        raise _cabi.MInferB200Error("q, k, v must share one dtype")
    B, H, N, D = query.shape
    Hkv = key.shape[1]
    q, k, v = _as_bhnd(query), _as_bhnd(key), _as_bhnd(value)
    if out is None:
        out = torch.empty((B, H, N, D), dtype=query.dtype, device=query.device)
    if sm_scale is None:
        sm_scale = D ** -0.5
    dev = query.device
    status = plan.status if plan is not None else _cabi.new_status(dev)
    if return_lse:
        lse = torch.empty((B, H, N), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _cabi.check(_cabi.lib().minf_sparse_attention_fwd_window(
                _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(out), _cabi.ptr(lse), None, None,
                _cabi.strides3(q), _cabi.strides3(k), _cabi.strides3(v), _cabi.strides3(out),
                B, H, Hkv, N, N, 0, N, 0, D, float(sm_scale),
                _cabi.ptr(head_mode), _cabi.ptr(head_param),
                _cabi.ptr(plan.plan if plan is not None else None),
                _cabi.ptr(plan.v_idx if plan is not None else None),
                plan.cap_v if plan is not None else 0, plan.cap_s if plan is not None else 1,
                _cabi.ptr(status), _cabi.stream_ptr(dev)))
        if plan is None:
            sparse_attention_forward.last_status = status
        return out, lse
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().minf_sparse_attention_fwd(
            _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(out),
            _cabi.strides3(q), _cabi.strides3(k), _cabi.strides3(v), _cabi.strides3(out),
            B, H, Hkv, N, D, float(sm_scale),
            _cabi.ptr(head_mode), _cabi.ptr(head_param),
            _cabi.ptr(plan.plan if plan is not None else None),
            _cabi.ptr(plan.v_idx if plan is not None else None),
            plan.cap_v if plan is not None else 0, plan.cap_s if plan is not None else 1,
            _cabi.ptr(status), _cabi.stream_ptr(dev)))
    if plan is None:
        sparse_attention_forward.last_status = status
    return out
