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
        model.config.starting_layer = self.config.starting_layer
        model.config.config_path = self.config.config_path
        if self.config.attn_type == "minference":
            # the pattern table is loaded once here (models_patch.py:98-102 of the reference)
            if self.config.is_search:
                # every prefill call searches its layer and appends to config_path; layers run dense meanwhile
                self.config.attn_kwargs["config_path"] = self.config.config_path
            elif "best_pattern" not in self.config.attn_kwargs:
                with open(self.config.config_path, "r") as f:
                    self.config.attn_kwargs["best_pattern"] = json.load(f)
            if self.config.attn_kwargs.get("starting_layer", -1) < 0:
                self.config.attn_kwargs["starting_layer"] = 0
        elif self.config.attn_type in ("a_shape", "tri_shape"):
            self.config.attn_kwargs.setdefault("n_local", 3968)
            self.config.attn_kwargs.setdefault("n_init", 128)
            if self.config.attn_type == "tri_shape":
                self.config.attn_kwargs.setdefault("n_last", 100)
        return new_patch(model, self.config)
