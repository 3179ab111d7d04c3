"""Sparse prefill inside vLLM (the role of minference_patch_vllm, minference/patch.py:1049-1310, and of the
``*_vllm`` forwards, minference/modules/minference_forward.py:858-1361, written against vLLM 0.4.x).

Current vLLM (the V1 engine, 0.2x) keeps one ``AttentionImpl`` object per attention layer inside every worker
process; its ``forward(layer, query, key, value, kv_cache, attn_metadata, output)`` receives the new tokens as
``[tokens, heads, head_size]`` and the KV cache is filled by the layer outside that call.  The hook wraps that
method on every layer of every worker (``LLM.apply_model``): a batch that is the first and only chunk of one
sequence -- a pure prefill, the case the reference patches -- runs the per-head sparse patterns on Q/K/V as they
arrive; every other batch (decode, chunked or prefix-cached prefill, several sequences) goes to the stock
implementation untouched.  Under tensor parallelism a worker holds ``heads / tp`` consecutive heads: the pattern
table is read at ``tp_rank * local_heads + local_head`` (minference_forward.py:902, 1057, 1216).

For the whole prompt to arrive as one batch the engine needs ``enable_chunked_prefill=False`` or a
``max_num_batched_tokens`` at least as long as the prompt, and ``enable_prefix_caching=False``.
"""
from __future__ import annotations

import json
import re
import types

import torch

from .modules.minference_forward import minference_prefill_forward


def layer_index_of(layer_name: str) -> int:
    """``model.layers.12.self_attn.attn`` -> 12 (the first integer component of the module path)."""
    for part in str(layer_name).split("."):
        if part.isdigit():
            return int(part)
    m = re.search(r"(\d+)", str(layer_name))
    if m:
        return int(m.group(1))
    raise ValueError(f"no layer index in {layer_name!r}")


def is_single_sequence_prefill(attn_metadata) -> bool:
    """One sequence whose tokens are all new: no cached context, no other request in the batch.  Only host-side
    fields of the metadata are read (no device synchronisation).  Two layouts of the metadata are known: the
    FlashAttention backend's (query offsets, longest query, longest sequence) and the FlashInfer backend's, the default
    on this GPU generation (counts of prefill and decode requests and of their tokens; it does not say how long the
    cached context is, which is why ``patch_vllm`` insists on an engine without prefix caching and chunked prefill).
    Anything else is not taken."""
    try:
        if attn_metadata is None or getattr(attn_metadata, "use_cascade", False) or not getattr(attn_metadata, "causal", True):
            return False
        n = attn_metadata.num_actual_tokens
        if hasattr(attn_metadata, "query_start_loc"):
            return (attn_metadata.query_start_loc.shape[0] == 2 and n > 1 and attn_metadata.max_query_len == n
                    and attn_metadata.max_seq_len == n)
        if hasattr(attn_metadata, "num_prefills"):
            return (attn_metadata.num_prefills == 1 and getattr(attn_metadata, "num_decodes", 0) == 0
                    and getattr(attn_metadata, "num_prefill_tokens", n) == n and n > 1)
    except AttributeError:
        pass
    return False


def sparse_prefill_forward(impl, layer, query, key, value, output, attn_metadata, attn_config: dict, head_offset: int,
                           layer_idx: int | None = None):
    """The sparse path of one attention layer for a single-sequence prefill: ``query [tokens, heads, 128]``,
    ``key / value [tokens, kv_heads, 128]`` -> ``output[:tokens]``."""
    n = attn_metadata.num_actual_tokens
    h, hkv, d = impl.num_heads, impl.num_kv_heads, impl.head_size
    q = query[:n].view(n, h, d).transpose(0, 1).unsqueeze(0)          # [1, H, N, D] view, head_dim contiguous
    k = key[:n].view(n, hkv, d).transpose(0, 1).unsqueeze(0)
    v = value[:n].view(n, hkv, d).transpose(0, 1).unsqueeze(0)
    if layer_idx is None:
        layer_idx = layer_index_of(getattr(layer, "layer_name", ""))
    # "vllm_minference" runs the per-head pattern table; "vllm_a_shape", "vllm_tri_shape" and "vllm_flexprefill" (the
    # reference's other vLLM types, minference_configuration.py:24-28) the operator of that name, which has no table
    kind = attn_config.get("prefill_operator", "minference")
    if kind == "minference":
        forward = minference_prefill_forward
    else:
        from .patch import prefill_forwards

        forward = prefill_forwards[kind]
    out = forward(q, k, v, {"attention_mask": None, "layer_idx": layer_idx, "head_offset": head_offset,
                            "num_hidden_layers": len(attn_config.get("best_pattern", [])), "attn_forward_config": attn_config})
    output[:n].view(n, h, d).copy_(out[0].transpose(0, 1))
    return output


def supports(impl, query) -> bool:
    return (impl.head_size == 128 and query.dtype == torch.bfloat16 and query.is_cuda
            and abs(float(impl.scale) - 128 ** -0.5) < 1e-6 and getattr(impl, "alibi_slopes", None) is None
            and tuple(getattr(impl, "sliding_window", (-1, -1)) or (-1, -1)) == (-1, -1)
            and not getattr(impl, "logits_soft_cap", 0) and getattr(impl, "sinks", None) is None)


def wrap_impl(impl, attn_config: dict, head_offset: int):
    """Rebind ``impl.forward``: sparse prefill where it applies, the original method otherwise."""
    if getattr(impl, "_minference_b200_wrapped", False):
        return impl
    stock = impl.forward

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, *args, **kwargs):
        if output is not None and is_single_sequence_prefill(attn_metadata) and supports(self, query):
            return sparse_prefill_forward(self, layer, query, key, value, output, attn_metadata, attn_config, head_offset)
        return stock(layer, query, key, value, kv_cache, attn_metadata, output, *args, **kwargs)

    impl.forward = types.MethodType(forward, impl)
    impl._minference_b200_wrapped = True
    return impl


def install_on_model(model, attn_config: dict) -> int:
    """Runs inside a worker process: wraps the attention implementation of every decoder layer of ``model``.
    Returns the number of layers wrapped."""
    try:
        from vllm.distributed import get_tensor_model_parallel_rank

        tp_rank = get_tensor_model_parallel_rank()
    except Exception:       # not inside a vLLM worker (unit tests): a single rank
        tp_rank = 0
    count = 0
    for _, mod in model.named_modules():
        impl = getattr(mod, "impl", None)
        if impl is None or not hasattr(impl, "num_heads") or not hasattr(impl, "forward"):
            continue
        wrap_impl(impl, attn_config, tp_rank * impl.num_heads)
        count += 1
    return count


def check_engine_settings(llm) -> None:
    """The sparse path sees a prompt only if it arrives as one batch with nothing cached: refuse an engine with prefix
    caching, or with chunked prefill and a token budget below its longest prompt.  Engines whose configuration objects
    are laid out differently are let through (the per-batch test still applies)."""
    cfg = getattr(getattr(llm, "llm_engine", None), "vllm_config", None)
    cache, sched, model = (getattr(cfg, name, None) for name in ("cache_config", "scheduler_config", "model_config"))
    if getattr(cache, "enable_prefix_caching", False):
        raise ValueError("the sparse prefill needs an engine with enable_prefix_caching=False")
    budget, longest = getattr(sched, "max_num_batched_tokens", None), getattr(model, "max_model_len", None)
    if getattr(sched, "enable_chunked_prefill", False) and budget and longest and budget < longest:
        raise ValueError(f"the sparse prefill needs whole prompts in one batch: max_num_batched_tokens={budget} is below "
                         f"max_model_len={longest} with chunked prefill on")


def patch_vllm(llm, config):
    """``MInference("vllm_minference", model_name)(llm)``: install the hook in every worker of a ``vllm.LLM``."""
    attn_config = dict(config.attn_kwargs)
    attn_config["prefill_operator"] = config.attn_type[len("vllm_"):] if config.attn_type.startswith("vllm_") else config.attn_type
    if attn_config["prefill_operator"] == "minference" and "best_pattern" not in attn_config:
        with open(config.config_path) as f:
            attn_config["best_pattern"] = json.load(f)
    attn_config.setdefault("starting_layer", 0)
    if attn_config["starting_layer"] < 0:
        attn_config["starting_layer"] = 0

    check_engine_settings(llm)

    def install(model):     # shipped to the workers
        from minference_b200.vllm_hook import install_on_model

        return install_on_model(model, attn_config)

    counts = llm.apply_model(install)
    if not counts or min(counts) == 0:
        raise RuntimeError("no attention layer was found to attach the sparse prefill to")
    return llm
