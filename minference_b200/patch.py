"""Attach the sparse prefill to a Hugging Face model (mirrors the role of minference/patch.py:850-892).

The reference rebinds ``Attention.forward`` of every layer (written against transformers <= 4.4x).
Current transformers route attention through a registry of functions
(``transformers.modeling_utils.ALL_ATTENTION_FUNCTIONS``) selected by
``config._attn_implementation``: the patch registers one function there.  It receives the rotated
``query [B,H,N,D]`` and the un-repeated ``key/value [B,Hkv,N,D]``, so the 4x K/V copy the
reference makes before its per-head loop (modules/forward.py:128-132) does not exist here.

Prefill calls (query length == key length > 1) run the dynamic sparse path; decode steps and
anything else go to the stock scaled-dot-product function.
"""
from __future__ import annotations

import torch

from .modules.minference_forward import minference_prefill_forward
from .ops.streaming_kernel import a_shape_kernel, tri_shape_kernel

ATTN_NAME = "minference_b200"


def _make_attention_function(config):
    attn_type = config.attn_type
    attn_kwargs = config.attn_kwargs

    def minference_attention(module, query, key, value, attention_mask=None, dropout=0.0, scaling=None, **kwargs):
        from transformers.integrations.sdpa_attention import sdpa_attention_forward

        q_len, k_len = query.shape[2], key.shape[2]
        usable = (q_len == k_len and q_len > 1 and query.shape[0] == 1 and query.shape[-1] == 128
                  and query.dtype == torch.bfloat16 and query.is_cuda)
        if not usable:
            return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                          scaling=scaling, **kwargs)
        if attn_type == "a_shape":
            out = a_shape_kernel(query, key, value, {"attn_forward_config": attn_kwargs})
        elif attn_type == "tri_shape":
            out = tri_shape_kernel(query, key, value, {"attn_forward_config": attn_kwargs})
        else:
            cfg = attn_kwargs
            if attn_type == "dense":
                cfg = {**attn_kwargs, "starting_layer": 1 << 30, "best_pattern": []}
            out = minference_prefill_forward(query, key, value, {
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
