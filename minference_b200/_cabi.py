"""ctypes binding of ``libminfer_b200.so`` (declared in ``include/minfer_b200.h``).

The library is the only compute path of this package: when it cannot be loaded the
import of any operator raises, there is no fallback.  Tensors are handed over as raw
device pointers plus element strides; outputs and scratch are allocated here with torch
(the caching allocator), never inside the library.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_ulonglong, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# MINFER_B200_LIB selects another build of the same library (the range-checked debug variant of build.py --bounds)
LIB_PATH = os.environ.get("MINFER_B200_LIB") or os.path.join(_HERE, "libminfer_b200.so")

STATUS_WORDS = 4
ST_ERROR, ST_NO_SLASH = 0, 1
MODE_PLAN, MODE_ASHAPE = 0, 1
# (force_columns, force_diagonals, min_vertical, min_slash) of minf_vs_select
SELECT_RULES = {"online": (30, 100, 30, 50), "static": (30, 30, 30, 50), "search": (30, 30, 0, 0)}

_lib = None

# name -> (restype, argtypes); must list every symbol of include/minfer_b200.h
_I64x3 = POINTER(c_int64)
SIGNATURES = {
    "minf_version": (c_char_p, []),
    "minf_last_error": (c_char_p, []),
    "minf_selftest_bounded_wait": (c_int, [c_int, c_void_p, c_void_p]),
    "minf_convert_vertical_slash_indexes": (c_int, [c_void_p] * 3 + [c_int] * 5 + [c_void_p] * 4 + [c_void_p, c_void_p]),
    "minf_plan_bytes": (c_size_t, [c_int] * 5),
    "minf_vs_build_plan": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_void_p, c_void_p, c_void_p]),
    "minf_plan_bytes_window": (c_size_t, [c_int] * 6),
    "minf_vs_build_plan_window": (c_int, [c_void_p] * 5 + [c_int] * 6 + [c_void_p, c_void_p, c_void_p]),
    "minf_block_sparse_scratch_bytes": (c_size_t, [c_int] * 4),
    "minf_block_sparse_build_plan": (c_int, [c_void_p, c_void_p, _I64x3, _I64x3] + [c_int] * 6 + [c_void_p] +
                                     [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "minf_block_sparse_pool": (c_int, [c_void_p, _I64x3, c_int, c_int, c_int, c_void_p, c_void_p]),
    "minf_block_sparse_select_window": (c_int, [c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "minf_vs_estimate_scratch_bytes": (c_size_t, [c_int] * 3),
    "minf_vs_estimate": (c_int, [c_void_p, c_void_p, _I64x3, _I64x3] + [c_int] * 5 + [c_void_p] * 2 +
                         [c_int, c_int] + [c_void_p] * 6 + [c_void_p, c_void_p, c_void_p]),
    "minf_vs_scores_blocks": (c_int, [c_int]),
    "minf_vs_scores_pass": (c_int, [c_int, c_void_p, c_void_p, _I64x3, _I64x3] + [c_int] * 7 +
                            [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "minf_vs_scores_pass_divisor": (c_int, [c_int, c_void_p, c_void_p, _I64x3, _I64x3] + [c_int] * 7 + [c_float] +
                                    [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "minf_block_mask_build_plan": (c_int, [c_void_p] + [c_int] * 5 + [c_void_p, c_void_p, c_void_p]),
    "minf_vs_scores_combine": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "minf_vs_select_scratch_bytes": (c_size_t, [c_int] * 3),
    "minf_vs_select": (c_int, [c_void_p, c_void_p] + [c_int] * 3 + [c_void_p, c_void_p, c_int, c_int] +
                       [c_void_p] * 4 + [c_int] * 4 + [c_void_p, c_void_p]),
    "minf_vs_estimate_static_scratch_limit": (c_size_t, []),
    "minf_vs_estimate_static": (c_int, [c_void_p, c_void_p, _I64x3, _I64x3] + [c_int] * 5 + [c_void_p] * 2 +
                                [c_int, c_int] + [c_void_p] * 4 + [c_void_p, c_void_p]),
    "minf_sparse_attention_fwd": (c_int, [c_void_p] * 4 + [_I64x3] * 4 + [c_int] * 5 + [c_float] +
                                  [c_void_p] * 4 + [c_int, c_int] + [c_void_p, c_void_p]),
    "minf_sparse_attention_fwd_window": (c_int, [c_void_p] * 7 + [_I64x3] * 4 + [c_int] * 9 + [c_float] +
                                         [c_void_p] * 4 + [c_int, c_int] + [c_void_p, c_void_p]),
    "minf_plan_count_tiles": (c_int, [c_void_p] + [c_int] * 5 + [c_void_p, c_void_p]),
    "minf_plan_count_tiles_window": (c_int, [c_void_p] + [c_int] * 6 + [c_void_p, c_void_p]),
}


class MInferB200Error(RuntimeError):
    pass


_NVTX = os.environ.get("MINFER_B200_NVTX", "0") == "1"


@contextlib.contextmanager
def nvtx_range(name: str):
    """An NVTX range around a stage of the path (estimator, plan, attention, ring step) when MINFER_B200_NVTX=1,
    so that a timeline profiler shows the stages by name; nothing otherwise."""
    if not _NVTX:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def lib():
    """Load the shared library once; raise loudly when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MInferB200Error(
                f"{LIB_PATH} is missing: build it with `python -m minference_b200.build` "
                "(there is no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            if not hasattr(L, name):
                continue  # reported by the symbol test; calling it raises AttributeError
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise MInferB200Error(f"minfer_b200 error {rc}: {lib().minf_last_error().decode()}")


def ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


def strides3(t: torch.Tensor):
    assert t.dim() == 4 and t.stride(3) == 1, "expected [B,H,N,D] with contiguous head_dim"
    return (c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def stream_ptr(device=None):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise MInferB200Error("minference_b200 operators run on CUDA tensors only (no CPU path)")


def new_status(device) -> torch.Tensor:
    return torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)


def raise_on_status(status: torch.Tensor, what: str) -> None:
    """Synchronising check of the device status words."""
    st = status.tolist()
    if st[ST_ERROR]:
        raise MInferB200Error(f"{what}: device reported error bits {st[ST_ERROR]:#x} "
                              "(1 = abandoned wait, 2 = misaligned shared memory, 8 = a range check of the debug build failed, 4 = bad plan: a plan-mode head without a plan, "
                              "a range count beyond the slot's capacity, unordered ranges, or columns without a vertical list)")
    if st[ST_NO_SLASH]:
        raise MInferB200Error(f"{what}: {st[ST_NO_SLASH]} row blocks have no slash offset below their last row; "
                              "s_idx must contain an offset < 64")
