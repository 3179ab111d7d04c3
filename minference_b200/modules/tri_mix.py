"""TriangleMix layer policies (mirrors minference/modules/tri_mix.py:19-53).

Shallow layers (below ``starting_layer``) keep their full attention -- dense for ``tri_mix``, the dynamic sparse
prefill for ``tri_mix_minference`` -- and the layers from ``starting_layer`` on use the tri-shape pattern: sink +
sliding window for all rows but the last ``n_last``, which see every earlier key.
"""
from __future__ import annotations

from ..ops.streaming_kernel import tri_shape_kernel
from .minference_forward import dense_prefill_forward, minference_prefill_forward


def tri_mix_forward(query_states, key_states, value_states, prefill_kwargs):
    starting_layer = prefill_kwargs["attn_forward_config"].get("starting_layer", 0)
    if prefill_kwargs["layer_idx"] < starting_layer:
        return dense_prefill_forward(query_states, key_states, value_states)
    return tri_shape_kernel(query_states, key_states, value_states, prefill_kwargs)


def tri_mix_minference_forward(q, k, v, prefill_kwargs):
    cfg = prefill_kwargs["attn_forward_config"]
    if prefill_kwargs["layer_idx"] < cfg.get("starting_layer", 0):
        # the sparse prefill on the shallow layers; its own `starting_layer` gate must not send them to dense.
        # One shallow copy of the config is kept (the reference deep-copies its kwargs on every call).
        inner = cfg.get("_tri_mix_minference_cfg")
        if inner is None:
            inner = dict(cfg)
            inner["starting_layer"] = 0
            cfg["_tri_mix_minference_cfg"] = inner
        return minference_prefill_forward(q, k, v, {**prefill_kwargs, "attn_forward_config": inner})
    return tri_shape_kernel(q, k, v, prefill_kwargs)
