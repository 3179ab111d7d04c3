"""Attach the sparse prefill to a Hugging Face model (mirrors the role of minference/patch.py:850-892).

The reference rebinds ``Attention.forward`` of every layer (written against transformers <= 4.4x).
Current transformers route attention through a registry of functions
(``transformers.modeling_utils.ALL_ATTENTION_FUNCTIONS``) selected by
``config._attn_implementation``: the patch registers one function there.  It receives the rotated
``query [B,H,N,D]`` and the un-repeated ``key/value [B,Hkv,N,D]``, so the 4x K/V copy the
reference makes before its per-head loop (modules/forward.py:128-132) does not exist here.

Prefill calls (query length == key length > 1) run the sparse path of the configured attention type; decode
steps go to the stock scaled-dot-product function, and so does a prefill the kernels cannot serve (another
logit scale, sliding-window layers, batch above 1, another dtype or head size) -- with a warning, once.
"""
from __future__ import annotations

import torch

import warnings

from .modules.flexprefill import flexprefill_forward
from .modules.minference_forward import minference_prefill_forward, static_prefill_forward
from .modules.tri_mix import tri_mix_forward, tri_mix_minference_forward
from .ops.pit_sparse_flash_attention_v2 import dilated_sparse_attention
from .ops.streaming_kernel import a_shape_kernel, tri_shape_kernel

ATTN_NAME = "minference_b200"

# prefill operators by attention type, called as f(q, k, v, prefill_kwargs) (modules/forward.py:237-246 of the reference)
prefill_forwards = {
    "minference": minference_prefill_forward,
    "a_shape": a_shape_kernel,
    "tri_shape": tri_shape_kernel,
    "tri_mix": tri_mix_forward,
    "tri_mix_minference": tri_mix_minference_forward,
    "static": static_prefill_forward,
    "flexprefill": flexprefill_forward,
    "dilated1": lambda q, k, v, kw: dilated_sparse_attention(q, k, v, "dilated1"),
    "dilated2": lambda q, k, v, kw: dilated_sparse_attention(q, k, v, "dilated2"),
}
_warned: set = set()


def _sparse_path_refusal(query, key, scaling, kwargs):
    """Why this call cannot take the sparse prefill kernels (None when it can).  Decode steps are not prefill and
    go to the stock function silently; everything else is said once."""
    q_len, k_len = query.shape[2], key.shape[2]
    if q_len == 1 or q_len != k_len:
        return "decode"
    if query.shape[0] != 1:
        return "batch size above 1 (the estimator is defined per sequence)"
    if query.shape[-1] != 128 or query.dtype != torch.bfloat16 or not query.is_cuda:
        return f"bf16 CUDA tensors with head_dim 128 are required (got {query.dtype}, head_dim {query.shape[-1]}, {query.device.type})"
    if scaling is not None and abs(float(scaling) - query.shape[-1] ** -0.5) > 1e-6 * query.shape[-1] ** -0.5:
        return f"the model scales its logits by {scaling}, the sparse kernels by 1/sqrt(head_dim)"
    if kwargs.get("sliding_window") is not None or kwargs.get("softcap") is not None:
        return "sliding-window or soft-capped attention layers"
    return None


def _make_attention_function(config):
    attn_type = config.attn_type
    attn_kwargs = config.attn_kwargs

    def minference_attention(module, query, key, value, attention_mask=None, dropout=0.0, scaling=None, **kwargs):
        from transformers.integrations.sdpa_attention import sdpa_attention_forward

        why = _sparse_path_refusal(query, key, scaling, kwargs)
        if why is not None:
            if why != "decode" and why not in _warned:
                _warned.add(why)
                warnings.warn(f"minference_b200: this prefill runs on the stock attention instead of the sparse kernels: {why}")
            return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                          scaling=scaling, **kwargs)
        cfg = attn_kwargs
        if attn_type == "dense":
            cfg = {**attn_kwargs, "starting_layer": 1 << 30, "best_pattern": []}
        forward = prefill_forwards.get(attn_type, minference_prefill_forward)
        out = forward(query, key, value, {
            "attention_mask": attention_mask, "layer_idx": module.layer_idx,
            "num_hidden_layers": getattr(module.config, "num_hidden_layers", 0), "attn_forward_config": cfg})
        return out.transpose(1, 2), None       # [B, N, H, D] like the other attention functions

    return minference_attention


def new_patch(model, config):
    """Register the attention function and switch the model to it."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    ALL_ATTENTION_FUNCTIONS[ATTN_NAME] = _make_attention_function(config)
    model.config._attn_implementation = ATTN_NAME
    for sub in model.modules():
        cfg = getattr(sub, "config", None)
        if cfg is not None and hasattr(cfg, "_attn_implementation"):
            cfg._attn_implementation = ATTN_NAME
    return model


def patch_hf(model, attn_type: str = "minference", attn_kwargs: dict = None, **kwargs):
    """Convenience wrapper with the reference's name (minference/patch.py:1313)."""
    from .minference_configuration import MInferenceConfig

    return new_patch(model, MInferenceConfig(attn_type=attn_type, attn_kwargs=attn_kwargs or {}, **kwargs))
