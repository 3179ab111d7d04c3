"""A-shape / StreamingLLM attention (mirrors minference/ops/streaming_kernel.py:611-646, 781-818)."""
from __future__ import annotations

import torch

from .. import _cabi
from ..cuda import _status_checks_enabled
from .sparse_forward import sparse_attention_forward


def streaming_forward(q, k, v, n_init, n_local):
    """Sink (first ``n_init`` keys) + sliding window (``n_local`` keys) causal attention.

    One pass: the reference runs a window stage and a complement-window stage with fp32
    O/M/L carried through HBM (streaming_kernel.py:420-499); here both parts share one
    online softmax.  K/V may keep fewer heads than Q.
    """
    assert q.dim() == 4
    _cabi.require_cuda(q, k, v)
    H = q.shape[1]
    dev = q.device
    head_mode = torch.full((H,), _cabi.MODE_ASHAPE, dtype=torch.int32, device=dev)
    head_param = torch.tensor([[int(n_init), int(n_local)]] * H, dtype=torch.int32, device=dev)
    out = sparse_attention_forward(q, k, v, None, head_mode=head_mode, head_param=head_param)
    if _status_checks_enabled():
        _cabi.raise_on_status(sparse_attention_forward.last_status, "streaming_forward")
    return out


def a_shape_kernel(q, k, v, config):
    """Same as ``streaming_forward`` with parameters read from the attention config
    (streaming_kernel.py:781-818)."""
    n_init = config["attn_forward_config"].get("n_init", 128)
    n_local = config["attn_forward_config"].get("n_local", 3968)
    return streaming_forward(q, k, v, n_init, n_local)
