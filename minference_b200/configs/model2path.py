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


def register_model(model_name: str, config_path: str) -> None:
    MODEL2PATH[model_name] = config_path


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
