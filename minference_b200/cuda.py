"""``minference.cuda`` of the reference: the index conversion extension module.

Mirrors the pybind module built from csrc/kernels.cpp:16-18 of the reference.
"""
from __future__ import annotations

import torch

from . import _cabi


def convert_vertical_slash_indexes(seqlens: torch.Tensor, vertical_indexes: torch.Tensor,
                                   slash_indexes: torch.Tensor, context_size: int,
                                   block_size_M: int = 64, block_size_N: int = 64):
    """Reference-format index tensors (csrc/vertical_slash_index.cu:127-167).

    ``seqlens`` int32 ``[B]``; ``vertical_indexes`` int32 ``[B,H,NNZ_V]`` ascending;
    ``slash_indexes`` int32 ``[B,H,NNZ_S]`` descending.  Returns ``[block_count,
    block_offset, column_count, column_index]`` like the reference, int32, zero tails.
    """
    assert block_size_M == 64 and block_size_N == 64  # same restriction as the reference (:135-136)
    _cabi.require_cuda(seqlens, vertical_indexes, slash_indexes)
    seqlens = seqlens.to(torch.int32).contiguous()
    v = vertical_indexes.to(torch.int32).contiguous()
    s = slash_indexes.to(torch.int32).contiguous()
    B, H, nnz_s = s.shape
    nnz_v = v.shape[2]
    rows = (context_size + 63) // 64
    dev = s.device
    block_count = torch.empty((B, H, rows), dtype=torch.int32, device=dev)
    block_offset = torch.empty((B, H, rows, nnz_s), dtype=torch.int32, device=dev)
    column_count = torch.empty((B, H, rows), dtype=torch.int32, device=dev)
    column_index = torch.empty((B, H, rows, nnz_v), dtype=torch.int32, device=dev)
    status = _cabi.new_status(dev)
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().minf_convert_vertical_slash_indexes(
            _cabi.ptr(seqlens), _cabi.ptr(v), _cabi.ptr(s), B, H, context_size, nnz_v, nnz_s,
            _cabi.ptr(block_count), _cabi.ptr(block_offset), _cabi.ptr(column_count), _cabi.ptr(column_index),
            _cabi.ptr(status), _cabi.stream_ptr(dev)))
    if _status_checks_enabled():
        _cabi.raise_on_status(status, "convert_vertical_slash_indexes")
    return [block_count, block_offset, column_count, column_index]


_CHECKS = True


def set_status_checks(enabled: bool) -> None:
    """Turn the synchronising read of the device status words after each call on or off."""
    global _CHECKS
    _CHECKS = bool(enabled)


def _status_checks_enabled() -> bool:
    return _CHECKS
