"""Configuration object of the patch API (mirrors minference/minference_configuration.py:7-111).

Only the attention types that run on this library's kernels are accepted: the dynamic sparse
prefill ("minference", also with ``is_search=True`` for the offline pattern search; "vllm_minference"
for the vLLM hook, which also takes "vllm_a_shape", "vllm_tri_shape" and "vllm_flexprefill"), its static
variant ("static"), the fixed index sets "dilated1" / "dilated2", the fixed A-shape pattern ("a_shape"),
A-shape with dense last rows ("tri_shape"), the TriangleMix layer
policies ("tri_mix", "tri_mix_minference"), FlexPrefill's adaptive block budgets ("flexprefill"; ``attn_kwargs``: gamma,
tau, min_budget, max_budget, block_size) and dense causal ("dense").  The KV-cache methods of the
reference (kv_type other than "dense") are decode-side features outside this library.
"""
from __future__ import annotations

from .configs.model2path import MODEL2PATH


class MInferenceConfig:
    MINFERENCE_ATTENTION_TYPES = ["minference", "vllm_minference", "tri_mix_minference"]      # need a pattern table
    OTHER_ATTENTION_TYPES = ["dense", "static", "dilated1", "dilated2", "a_shape", "tri_shape", "tri_mix", "flexprefill",
                             "vllm_a_shape", "vllm_tri_shape", "vllm_flexprefill"]
    KV_TYPES = ["dense"]

    def __init__(
        self,
        attn_type: str = "minference",
        model_name: str = None,
        config_path: str = None,
        starting_layer: int = -1,
        kv_cache_cpu: bool = False,
        kv_cache_cpu_device: str = "cpu",
        kv_type: str = "dense",
        is_search: bool = False,
        attn_kwargs: dict = None,
        **kwargs,
    ):
        attn_type, kv_type = self.update_config_type(attn_type, kv_type)
        if attn_type not in self.MINFERENCE_ATTENTION_TYPES + self.OTHER_ATTENTION_TYPES:
            raise ValueError(f"The attn_type {attn_type} you specified is not supported.")
        if kv_type not in self.KV_TYPES:
            raise ValueError(f"The kv_type {kv_type} you specified is not supported.")
        if kv_cache_cpu:
            raise ValueError("kv_cache_cpu is not supported: the KV tensors must be resident on the GPU")
        if is_search and config_path is None:
            raise ValueError("is_search needs config_path: the file the searched pattern table is written to")
        self.attn_type = attn_type
        self.config_path = self.update_config_path(config_path, model_name)
        self.model_name = model_name
        self.is_search = is_search
        self.starting_layer = starting_layer
        self.kv_cache_cpu = kv_cache_cpu
        self.kv_cache_cpu_device = kv_cache_cpu_device
        self.kv_type = kv_type
        print(f"<---- MInference Config Detail ----> attn_type {self.attn_type}, kv_type {self.kv_type}")   # as the reference (:64-66)
        self.attn_kwargs = {
            "is_search": is_search,
            "starting_layer": starting_layer,
            "config_path": config_path,
            **(attn_kwargs or {}),
        }

    def update_config_path(self, config_path: str = None, model_name: str = None):
        if config_path is not None:
            return config_path
        if self.attn_type in self.OTHER_ATTENTION_TYPES:
            return MODEL2PATH.get(model_name, "")     # "static" reads head 0's budgets from a table when one is known
        if model_name not in MODEL2PATH:
            raise ValueError(
                f"No pattern table is registered for {model_name}: pass config_path=... (the JSON schema is "
                "list[layer] of {str(head): [type, vertical, slash, score]}) or register one with "
                "minference_b200.configs.model2path.register_model")
        return MODEL2PATH[model_name]

    def get(self, attr, default=None):
        return getattr(self, attr, default)

    def update_config_type(self, attn_type: str, kv_type: str):
        if kv_type == "":
            kv_type = "dense"
        if attn_type == "minference_with_dense":
            attn_type = "dense"
        return attn_type, kv_type

    @classmethod
    def get_available_attn_types(cls):
        return cls.MINFERENCE_ATTENTION_TYPES + cls.OTHER_ATTENTION_TYPES

    @classmethod
    def get_available_kv_types(cls):
        return cls.KV_TYPES
