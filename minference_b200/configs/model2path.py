"""Registry of per-model pattern tables (mirrors minference/configs/model2path.py).

A pattern table is a JSON file: ``list[layer] -> {str(head): [type, vertical, slash, score]}`` with
``type`` one of ``vertical_and_slash``, ``stream_llm``, ``block_sparse``.  The reference ships tables
found by its offline search for a set of public checkpoints; those files are data of that project
and are not redistributed here.  Point ``config_path`` at such a file, register it under a model
name, or generate a table with ``synthetic_pattern_table`` for benchmarks.
"""
from __future__ import annotations

import json
import os

import torch

BASE_DIR = os.path.dirname(os.path.abspath(__file__))
MODEL2PATH: dict[str, str] = {}

# File name of the searched table the reference ships for each model name (minference/configs/model2path.py:7-65).
# The files themselves stay with the reference; register_config_dir points this registry at a directory of them.
_BEST = "_kv_out_v32_fit_o_best_pattern"
TABLE_FILE_OF_MODEL: dict[str, str] = {
    **dict.fromkeys(("gradientai/Llama-3-8B-Instruct-262k", "gradientai/Llama-3-8B-Instruct-Gradient-1048k",
                     "gradientai/Llama-3-8B-Instruct-Gradient-4194k"), f"Llama_3_8B_Instruct_262k{_BEST}.json"),
    **dict.fromkeys(("gradientai/Llama-3-70B-Instruct-Gradient-262k", "gradientai/Llama-3-70B-Instruct-Gradient-1048k"),
                    f"Llama_3_70B_Instruct_262k{_BEST}.json"),
    **dict.fromkeys(("meta-llama/Meta-Llama-3.1-8B-Instruct", "meta-llama/Llama-3.1-8B-Instruct"),
                    f"Llama_3.1_8B_Instruct_128k{_BEST}_v2.json"),
    **dict.fromkeys(("meta-llama/Meta-Llama-3.1-70B-Instruct", "meta-llama/Llama-3.1-70B-Instruct"),
                    f"Llama_3.1_70B_Instruct_128k{_BEST}_v2.json"),
    "01-ai/Yi-9B-200K": f"Yi_9B_200k{_BEST}.json",
    "microsoft/Phi-3-mini-128k-instruct": f"Phi_3_mini_128k_instruct{_BEST}.json",
    "THUDM/glm-4-9b-chat-1m": f"GLM_4_9B_1M_instruct{_BEST}.json",
    "Qwen/Qwen2-7B-Instruct": f"Qwen2_7B_Instruct_128k_instruct{_BEST}.json",
    "Qwen/Qwen2.5-7B-Instruct": f"Qwen2.5_7B_Instruct_128k_instruct{_BEST}.json",
    "Qwen/Qwen2.5-32B-Instruct": f"Qwen2.5_32B_Instruct_128k{_BEST}.json",
    "Qwen/Qwen2.5-72B-Instruct": f"Qwen2.5_72B_Instruct_128k{_BEST}.json",
    "Qwen/Qwen2.5-7B-Instruct-1M": "Qwen2.5_7B_Instruct_1M.json",
    "Qwen/Qwen2.5-14B-Instruct-1M": "Qwen2.5_14B_Instruct_1M.json",
}


def register_model(model_name: str, config_path: str) -> None:
    MODEL2PATH[model_name] = config_path


def register_config_dir(path: str, require_files: bool = True):
    """Make ``MInference("minference", model_name)`` work for the model names the reference supports: ``path`` is a
    directory holding the reference's searched tables (its ``minference/configs`` folder, or a copy).  Every model
    whose file is present is registered (all of them with ``require_files=False``); returns the registered names."""
    names = []
    for model, fname in TABLE_FILE_OF_MODEL.items():
        full = os.path.join(path, fname)
        if not require_files or os.path.isfile(full):
            MODEL2PATH[model] = full
            names.append(model)
    return names


if os.environ.get("MINFERENCE_CONFIG_DIR"):       # a directory of pattern tables named by the environment
    register_config_dir(os.environ["MINFERENCE_CONFIG_DIR"])


def get_support_models():
    return list(MODEL2PATH.keys())


def synthetic_pattern_table(num_layers: int, num_heads: int, seed: int = 0, mix=("vertical_and_slash",),
                            vertical: int = 1000, slash: int = 6096, n_init: int = 128, n_local: int = 4096):
    """Seeded per-head pattern assignment in the reference's JSON schema.

    ``mix`` lists the pattern types to draw from uniformly; A-shape heads get
    ``[n_init, n_local]`` in the vertical/slash fields like the reference's stream_llm entries.
    """
    g = torch.Generator().manual_seed(seed)
    table = []
    for _ in range(num_layers):
        layer = {}
        for h in range(num_heads):
            ty = mix[int(torch.randint(len(mix), (1,), generator=g))]
            if ty == "stream_llm":
                layer[str(h)] = [ty, n_init, n_local, 1.0]
            elif ty == "block_sparse":
                layer[str(h)] = [ty, 0, 0, 1.0]
            else:
                layer[str(h)] = [ty, vertical, slash, 1.0]
        table.append(layer)
    return table


def save_pattern_table(table, path: str) -> None:
    with open(path, "w") as f:
        json.dump(table, f)
