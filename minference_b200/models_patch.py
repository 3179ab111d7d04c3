"""``MInference(...)(model)`` (mirrors minference/models_patch.py:19-128)."""
from __future__ import annotations

import json

from .minference_configuration import MInferenceConfig
from .patch import new_patch


class MInference:
    def __init__(
        self,
        attn_type: str = "minference",
        model_name: str = None,
        config_path: str = None,
        starting_layer: int = -1,
        kv_cache_cpu: bool = False,
        kv_type: str = "dense",
        is_search: bool = False,
        attn_kwargs: dict = None,
        **kwargs,
    ):
        self.config = MInferenceConfig(
            attn_type=attn_type, model_name=model_name, config_path=config_path, starting_layer=starting_layer,
            kv_cache_cpu=kv_cache_cpu, kv_type=kv_type, is_search=is_search, attn_kwargs=attn_kwargs or {}, **kwargs)

    def __call__(self, model):
        return self.patch_model(model)

    def patch_model(self, model):
        if hasattr(model, "config"):          # a Hugging Face model; a vllm.LLM carries no config object of this kind
            model.config.starting_layer = self.config.starting_layer
            model.config.config_path = self.config.config_path
        kw = self.config.attn_kwargs
        ty = self.config.attn_type
        for_vllm = ty.startswith("vllm_")
        if for_vllm and ty != "vllm_minference":        # same defaults as the Hugging Face type of that name
            ty = ty[len("vllm_"):]

        def load_table():       # the pattern table is loaded once here (models_patch.py:98-102 of the reference)
            if "best_pattern" not in kw:
                with open(self.config.config_path, "r") as f:
                    kw["best_pattern"] = json.load(f)

        if ty in ("minference", "vllm_minference"):
            if self.config.is_search:
                # every prefill call searches its layer and appends to config_path; layers run dense meanwhile
                kw["config_path"] = self.config.config_path
            else:
                load_table()
            if kw.get("starting_layer", -1) < 0:
                kw["starting_layer"] = 0
        elif ty in ("tri_mix", "tri_mix_minference"):       # defaults of the reference (:103-128)
            if ty == "tri_mix_minference":
                load_table()
            kw.setdefault("n_local", 512)
            kw.setdefault("n_init", 8)
            kw.setdefault("n_last", 128)
            if kw.get("starting_layer", -1) < 0:
                kw["starting_layer"] = 16
        elif ty in ("a_shape", "tri_shape"):
            kw.setdefault("n_local", 3968)
            kw.setdefault("n_init", 128)
            if ty == "tri_shape":
                kw.setdefault("n_last", 100)
        elif ty == "static":
            if self.config.config_path:       # budgets of head 0 come from the table; without one the default (1000, 6096)
                load_table()
        if for_vllm:
            from .vllm_hook import patch_vllm

            return patch_vllm(model, self.config)
        return new_patch(model, self.config)
