"""Offline per-head pattern search (the job of ``search_pattern``, modules/minference_forward.py:129-227
of the reference, driven by ``is_search`` at :644-673).

The reference materialises the ``[N, N]`` attention matrix of one head, multiplies it by the mask
of each candidate pattern and scores the candidate by the attention mass the mask keeps, averaged
over the rows from 2500 on.  The same quantity falls out of the attention kernels without any
``[N, N]`` tensor: for a row r the kept mass is

    sum_{c in pattern(r)} exp(s_rc) / sum_{c <= r} exp(s_rc) = 2 ** (lse_pattern(r) - lse_dense(r))

with the base-2 log-sum-exp the forward kernel returns next to its output.  One launch scores a
candidate for every head of the layer; the dense log-sum-exp is one more launch.

The candidates, the order they are tried in, the strict ``>`` that keeps the first best one and
the two renaming rules at the end (:217-220) are the reference's, and so are the selection rules of
its vertical-slash candidates: only the 30 nearest diagonals are forced and the budgets are taken as
they are (:140-146; the online path forces 100 and raises budgets to 30 / 50).

Two deviations remain, both on the side of a candidate's score, not of its lists.  A vertical-slash
candidate is scored over the index set the kernels compute -- a 64-wide tile around each selected
diagonal per 64-row block -- which contains the reference's one-token-wide diagonals, so its score
is never lower than the reference's, while the stream_llm candidate is masked exactly as in the
reference.  The block-sparse candidate pools 64-token blocks where the reference's search pools 32
(:178); that candidate is renamed to the default pattern whenever it wins, so only its score differs.
A searched table can therefore differ from the reference's on heads where two candidates are close.
"""
from __future__ import annotations

import json
import os

import torch

from .. import _cabi
from ..ops.block_sparse_flash_attention import _rows_pad, build_block_sparse_plan
from ..ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
from ..ops.sparse_forward import sparse_attention_forward

# (type, vertical_size, slash_size) in the reference's order (:203-210)
CANDIDATES = (
    ("stream_llm", 100, 800),
    ("vertical_and_slash", 30, 800),
    ("vertical_and_slash", 100, 750),
    ("vertical_and_slash", 500, 700),
    ("vertical_and_slash", 3500, 100),
    ("block_sparse", 8, 1),
)
SCORE_FROM_ROW = 2500          # rows before it are left out of the average (:163, :174, :196)


def _dense_lse(q, k, v):
    H, N = q.shape[1], q.shape[2]
    mode = torch.full((H,), _cabi.MODE_ASHAPE, dtype=torch.int32, device=q.device)
    param = torch.tensor([[0, N]] * H, dtype=torch.int32, device=q.device)
    return sparse_attention_forward(q, k, v, None, head_mode=mode, head_param=param, return_lse=True)[1]


def search_vertical_slash_lists(q, k, v_size: int, s_size: int):
    """Index lists of a vertical-slash candidate under the search's selection rules (:140-146): first 30
    columns and the 30 nearest diagonals forced, budgets not raised."""
    from .minference_forward import vertical_slash_estimate, vertical_slash_select

    H, N = q.shape[1], q.shape[2]
    *_, vsc, ssc = vertical_slash_estimate(q, k, v_size, s_size, return_scores=True)
    budget = lambda x: torch.full((q.shape[0] * H,), x, dtype=torch.int32, device=q.device)
    return vertical_slash_select(vsc, ssc, budget(v_size), budget(s_size), min(N, v_size), min(N, s_size), rules="search")


def candidate_lse(q, k, v, ty: str, v_size: int, s_size: int):
    """Base-2 log-sum-exp per row under one candidate pattern applied to every head."""
    H, N = q.shape[1], q.shape[2]
    dev = q.device
    if ty == "stream_llm":          # sink of v_size keys + window of s_size keys (:166-175)
        mode = torch.full((H,), _cabi.MODE_ASHAPE, dtype=torch.int32, device=dev)
        param = torch.tensor([[v_size, s_size + 1]] * H, dtype=torch.int32, device=dev)   # i - j <= s_size
        return sparse_attention_forward(q, k, v, None, head_mode=mode, head_param=param, return_lse=True)[1]
    if ty == "vertical_and_slash":
        v_idx, s_idx, nnz_v, nnz_s = search_vertical_slash_lists(q, k, v_size, s_size)
        plan = build_vertical_slash_plan(v_idx, s_idx, N, nnz_v, nnz_s)
        return sparse_attention_forward(q, k, v, plan, return_lse=True)[1]
    if ty == "block_sparse":        # keep one block in v_size per query block (:177-197)
        top_k = max(1, _rows_pad(N) // v_size)
        plan = build_block_sparse_plan(q, k, top_k)
        return sparse_attention_forward(q, k, v, plan, return_lse=True)[1]
    raise KeyError(ty)


@torch.no_grad()
def search_layer_patterns(query_states, key_states, value_states, candidates=CANDIDATES,
                          score_from_row: int = SCORE_FROM_ROW, return_all: bool = False):
    """Best pattern of every head of one layer: ``{head: (type, vertical, slash, score)}``.

    ``query_states [1,H,N,128]`` bf16 on the GPU, K/V with the query or the KV head count.
    """
    _cabi.require_cuda(query_states, key_states, value_states)
    H, N = query_states.shape[1], query_states.shape[2]
    r0 = score_from_row if N > score_from_row else 0
    dense = _dense_lse(query_states, key_states, value_states)[0, :, r0:]
    best = [("", 0, 0, 0.0)] * H
    table = []
    for ty, v_size, s_size in candidates:
        lse = candidate_lse(query_states, key_states, value_states, ty, v_size, s_size)[0, :, r0:]
        kept = torch.exp2(lse - dense).clamp_(max=1.0)          # attention mass the pattern keeps, per row
        scores = kept.mean(dim=-1).tolist()
        table.append((ty, v_size, s_size, scores))
        for h, sc in enumerate(scores):
            if sc > best[h][3]:
                best[h] = (ty, v_size, s_size, sc)
    out = {}
    for h, (ty, v_size, s_size, sc) in enumerate(best):
        if ty == "stream_llm":                      # (:217-218)
            ty = "vertical_and_slash"
        if ty == "block_sparse":                    # (:219-220)
            ty, v_size, s_size = "vertical_and_slash", 1000, 6096
        out[h] = (ty, v_size, s_size, sc)
    return (out, table) if return_all else out


def search_and_record(query_states, key_states, value_states, layer_idx: int, num_hidden_layers: int,
                      config_path: str | None):
    """The ``is_search`` branch of the prefill forward: search this layer and append the result to
    the JSON list at ``config_path`` (one dict per layer, heads as keys), like :644-650, :669-672."""
    config_list = []
    if config_path and os.path.isfile(config_path):
        with open(config_path, "r") as f:
            config_list = json.load(f)
        if len(config_list) == num_hidden_layers:
            raise RuntimeError(f"Search already completed; see {config_path}.")
    if layer_idx < len(config_list):
        return config_list[layer_idx]
    found = search_layer_patterns(query_states, key_states, value_states)
    new_config = {str(h): list(p) for h, p in found.items()}
    if config_path:
        config_list.append(new_config)
        with open(config_path, "w") as f:
            json.dump(config_list, f, indent=2)
    return new_config
