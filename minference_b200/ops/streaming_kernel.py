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


def tri_shape_kernel(q, k, v, config):
    """A-shape attention for all rows but the last ``n_last``, which attend to every earlier key
    (streaming_kernel.py:820-833 of the reference: the A-shape part sees the sequence cut before
    the last rows; the last rows are plain causal attention).

    Two launches of the same kernel: the A-shape rows, then a dense window that starts at the
    256-row boundary at or before the first of the last rows (the kernel's query windows start on
    256-row boundaries); only the last ``n_last`` rows of that window are kept.
    """
    _cabi.require_cuda(q, k, v)
    B, H, N, D = q.shape
    n_last = min(config["attn_forward_config"].get("n_last", 100), N - 1)
    cut = N - n_last
    y1 = a_shape_kernel(q[:, :, :cut], k[:, :, :cut], v[:, :, :cut], config)
    q0 = cut // 256 * 256
    dev = q.device
    mode = torch.full((H,), _cabi.MODE_ASHAPE, dtype=torch.int32, device=dev)
    param = torch.tensor([[0, N]] * H, dtype=torch.int32, device=dev)          # window of N keys = dense causal
    qw = q[:, :, q0:]
    qw = qw if (qw.stride(3) == 1 and qw.data_ptr() % 16 == 0) else qw.contiguous()
    kk = k if k.stride(3) == 1 else k.contiguous()
    vv = v if v.stride(3) == 1 else v.contiguous()
    out = torch.empty((B, H, N - q0, D), dtype=q.dtype, device=dev)
    status = _cabi.new_status(dev)
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().minf_sparse_attention_fwd_window(
            _cabi.ptr(qw), _cabi.ptr(kk), _cabi.ptr(vv), _cabi.ptr(out), None, None, None,
            _cabi.strides3(qw), _cabi.strides3(kk), _cabi.strides3(vv), _cabi.strides3(out),
            B, H, kk.shape[1], N, N - q0, q0, N, 0, D, float(D ** -0.5),
            _cabi.ptr(mode), _cabi.ptr(param), None, None, 0, 1, _cabi.ptr(status), _cabi.stream_ptr(dev)))
    if _status_checks_enabled():
        _cabi.raise_on_status(status, "tri_shape_kernel")
    return torch.cat([y1, out[:, :, cut - q0:]], dim=2)
