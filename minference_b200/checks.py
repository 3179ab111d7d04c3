"""fp32 masked-dense recomputation of sampled row blocks on the device.

Not on any product path: the benchmark's parity probes and the full-size GPU tests use it to
compare kernel output with ``softmax(mask(q k^T / sqrt(d))) v`` over exactly the index set the
reference kernels would visit (block_count/block_offset tiles with the causal mask, gathered
columns without one, ops/pit_sparse_flash_attention_v2.py:104-148 of the reference), at sizes
where a CPU recomputation would take minutes.  Plain torch ops in fp32 (TF32 stays off).
"""
from __future__ import annotations

import torch


def vertical_slash_row_block(q_rows: torch.Tensor, k: torch.Tensor, v: torch.Tensor, m: int, n_ctx: int,
                             block_count, block_offset, column_count, column_index, sm_scale: float | None = None):
    """Attention output of row block ``m`` (rows ``64m .. 64m+63``) of one head, fp32 ``[rows, D]``.

    ``q_rows [rows<=64, D]`` are the block's queries, ``k, v [n_ctx, D]`` the head's keys and values
    (any float dtype), ``block_count / column_count`` scalars (or 0-d tensors) and ``block_offset /
    column_index`` the int32 rows of the reference-format tables for this head and row block.
    """
    dev = q_rows.device
    rows, d = q_rows.shape
    r0 = 64 * m
    n_keys = min(n_ctx, r0 + 64)                  # tiles are causal, columns lie below the row block
    scale = float(sm_scale if sm_scale is not None else d ** -0.5)
    bc, cc = int(block_count), int(column_count)
    cover = torch.zeros(n_ctx + 192, dtype=torch.bool, device=dev)
    if bc:
        idx = (block_offset[:bc].long()[:, None] + torch.arange(64, device=dev)[None, :]).reshape(-1)
        cover[idx.clamp_(0, n_ctx + 191)] = True
    cols = torch.arange(n_keys, device=dev)
    rws = r0 + torch.arange(rows, device=dev)
    mask = cover[:n_keys][None, :] & (cols[None, :] <= rws[:, None])
    if cc:
        ci = column_index[:cc].long()
        ci = ci[ci < n_keys]
        mask[:, ci] = True
    s = (q_rows.float() @ k[:n_keys].float().T) * scale
    s.masked_fill_(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)              # a row without a visible key yields zeros
    return p @ v[:n_keys].float()


def compare_row_blocks(out_rows_of, q_rows_of, k, v, n_ctx: int, tables, row_blocks):
    """Max / mean absolute difference between kernel output and the recomputation over ``row_blocks``.

    ``out_rows_of(m)`` / ``q_rows_of(m)`` return the kernel's output rows and the queries of row
    block ``m``; ``tables = (block_count [rows], block_offset [rows, nnz_s], column_count [rows],
    column_index [rows, nnz_v])`` for the head."""
    bc, bo, cc, ci = tables
    worst, total, count = 0.0, 0.0, 0
    for m in row_blocks:
        ref = vertical_slash_row_block(q_rows_of(m), k, v, m, n_ctx, bc[m], bo[m], cc[m], ci[m])
        d = (out_rows_of(m).float() - ref).abs()
        worst = max(worst, d.max().item())
        total += d.sum().item()
        count += d.numel()
    return worst, total / max(count, 1)


def block_mask_row_block(q_rows: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_mask: torch.Tensor, m: int,
                         block: int, sm_scale: float | None = None):
    """Attention output of row block ``m`` of one head over a block set: ``block_mask [nb, nb]`` (bool), entry (i, j)
    set <=> query block i attends key block j, causal inside every block (the index set of the reference's
    FlexPrefill kernel, modules/flexprefill.py:412-436).  fp32 ``[rows, D]``."""
    dev = q_rows.device
    rows, d = q_rows.shape
    r0 = 64 * m
    n_keys = min(k.shape[0], r0 + 64)
    scale = float(sm_scale if sm_scale is not None else d ** -0.5)
    cols = torch.arange(n_keys, device=dev)
    rws = r0 + torch.arange(rows, device=dev)
    mask = block_mask[r0 // block][cols // block][None, :] & (cols[None, :] <= rws[:, None])
    s = (q_rows.float() @ k[:n_keys].float().T) * scale
    s.masked_fill_(~mask, float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    return p @ v[:n_keys].float()
