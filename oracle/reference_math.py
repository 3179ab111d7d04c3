"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's sparse-prefill arithmetic.

Nothing in the shipped package imports this module; it exists so that tests,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` leg of ``bench.py`` can check or
time the reference's algorithm on host cores.  Every function cites the reference
lines (paths inside microsoft/MInference v0.1.6.0) that it follows.

Parity status per function:

* ``convert_vertical_slash_indexes``  -- pinned: the C restatement ``oracle/vs_index.c``
  is checked against the reference kernel body compiled for the host
  (``oracle/build_ref.py``) and against the fixtures in ``tests/golden/``.
* ``build_block_index``               -- pinned: checked against the reference's own
  ``_build_block_index`` loaded by file path when the reference tree is present, and
  against ``tests/golden/block_index_*.npz`` made from it.
* ``vertical_slash_estimate``         -- pinned against fixtures produced by executing the
  reference's own function bodies (``tests/golden/make_golden.py`` extracts them from the
  reference file and runs them on CPU).  ``torch.topk`` leaves the order among exactly
  equal values unspecified, so comparisons are on index *sets* and on the +inf-forced
  entries.
* masked-dense attention              -- parity unpinned against the reference's Triton
  kernels (they need a GPU and the reference holds no golden vectors for them); the
  semantics follow the kernel source line by line and the tolerance is the one the
  reference's own self-test uses (``ops/pit_sparse_flash_attention.py:688-696``).
"""
from __future__ import annotations

import ctypes
import math
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
_I32P = ctypes.POINTER(ctypes.c_int32)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_I32P)


def _load(path: str, sym: str):
    lib = ctypes.CDLL(path)
    fn = getattr(lib, sym)
    fn.argtypes = [_I32P] * 7 + [ctypes.c_int] * 5
    return fn


def oracle_lib_path() -> str:
    return os.path.join(HERE, "liboracle_vs_index.so")


def ref_host_lib_path() -> str:
    return os.path.join(HERE, "_ref", "libref_vs_index_host.so")


def build_oracle_lib() -> str:
    """Compile oracle/vs_index.c with gcc (a fraction of a second)."""
    import subprocess

    out = oracle_lib_path()
    src = os.path.join(HERE, "vs_index.c")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O2", "-shared", "-fPIC", "-o", out, src])
    return out


def _convert_with(fn, seqlens, v_idx, s_idx, context_size, restype_int):
    seqlens = np.ascontiguousarray(seqlens, dtype=np.int32)
    v_idx = np.ascontiguousarray(v_idx, dtype=np.int32)
    s_idx = np.ascontiguousarray(s_idx, dtype=np.int32)
    B, H, nnz_v = v_idx.shape
    nnz_s = s_idx.shape[2]
    rows = (context_size + 63) // 64
    bc = np.zeros((B, H, rows), np.int32)
    bo = np.zeros((B, H, rows, nnz_s), np.int32)
    cc = np.zeros((B, H, rows), np.int32)
    ci = np.zeros((B, H, rows, nnz_v), np.int32)
    fn.restype = ctypes.c_int if restype_int else None
    rc = fn(_ptr(seqlens), _ptr(v_idx), _ptr(s_idx), _ptr(bc), _ptr(bo), _ptr(cc), _ptr(ci),
            B, H, rows, nnz_v, nnz_s)
    return (bc, bo, cc, ci), rc


def convert_vertical_slash_indexes(seqlens, v_idx, s_idx, context_size):
    """csrc/vertical_slash_index.cu:27-99,127-167 via oracle/vs_index.c.

    ``v_idx`` ascending, ``s_idx`` descending, int32 ``[B, H, nnz]`` numpy arrays.
    Returns ``(block_count, block_offset, column_count, column_index)``.
    """
    fn = _load(build_oracle_lib(), "oracle_convert_vertical_slash_indexes")
    outs, bad = _convert_with(fn, seqlens, v_idx, s_idx, context_size, True)
    if bad:
        raise ValueError(f"{bad} row blocks have no slash offset below their end row "
                         "(the reference reads out of bounds there)")
    return outs


def convert_vertical_slash_indexes_ref_host(seqlens, v_idx, s_idx, context_size):
    """Same call through the reference kernel body compiled for the host."""
    fn = _load(ref_host_lib_path(), "ref_convert_vertical_slash_indexes_host")
    outs, _ = _convert_with(fn, seqlens, v_idx, s_idx, context_size, False)
    return outs


# ---------------------------------------------------------------------------------
# online estimator  (modules/minference_forward.py:599-614, :110-116, :41-43)
# ---------------------------------------------------------------------------------

def sum_all_diagonal_matrix(mat: torch.Tensor) -> torch.Tensor:
    """Anti-diagonal sums of a ``[1,1,n,m]`` matrix (modules/minference_forward.py:110-116).

    Entry ``j`` of the result (length ``n+m-1``) is ``sum_i mat[i, i + j + 1 - n]`` over the
    ``i`` for which the column is in range.  Written as an explicit index-add instead of
    the reference's zero-pad + ``as_strided`` view.
    """
    b, h, n, m = mat.shape
    assert b == 1 and h == 1
    out = torch.zeros(n + m - 1, dtype=mat.dtype)
    rows = torch.arange(n)[:, None]
    cols = torch.arange(m)[None, :]
    j = cols - rows + n - 1          # 0 .. n+m-2
    out.index_add_(0, j.reshape(-1), mat[0, 0].reshape(-1))
    return out[None, None]


def vertical_slash_estimate(q: torch.Tensor, k: torch.Tensor, vertical_size: int, slash_size: int,
                            return_scores: bool = False, forced_diagonals: int = 100):
    """Per-head index estimation, ``q,k`` of shape ``[1,1,N,D]`` (minference_forward.py:599-614).

    Returns ``(vertical_topk [1,1,1,v] int64, slash [1,1,s] int64 diagonal offsets)``.
    ``forced_diagonals=30`` gives the static variant (``vertical_and_slash_kernel_static``, :418-437).
    """
    q_len = q.shape[2]
    head_dim = q.shape[-1]
    vertical_size = min(q_len, max(vertical_size, 30))
    slash_size = min(q_len, max(slash_size, 50))
    last_q = min(64, q_len)
    qk = torch.einsum("bhmk,bhnk->bhmn", q[:, :, -last_q:, :], k) / math.sqrt(head_dim)
    ar = torch.arange(last_q)
    keep = ar[None, None, :, None] >= ar[None, None, None, :]
    qk[:, :, :, -last_q:] = torch.where(keep, qk[:, :, :, -last_q:], -torch.inf)
    p = torch.nn.functional.softmax(qk, dim=-1, dtype=torch.float32)
    vertical = p.sum(-2, keepdim=True)
    vertical[..., :30] = torch.inf
    vertical_topk = torch.topk(vertical, vertical_size, -1).indices
    slash = sum_all_diagonal_matrix(p)[..., : -last_q + 1]
    slash[..., -forced_diagonals:] = torch.inf
    slash_idx = (q_len - 1) - torch.topk(slash, slash_size, -1).indices
    if return_scores:
        return vertical_topk, slash_idx, vertical[0, 0, 0], slash[0, 0]
    return vertical_topk, slash_idx


def presort_indices(v_idx: torch.Tensor, s_idx: torch.Tensor, batch: int, heads: int):
    """int32 cast + sort (ops/pit_sparse_flash_attention_v2.py:218-219)."""
    v = v_idx.to(torch.int32).reshape(batch, heads, -1).sort(dim=-1, descending=False)[0]
    s = s_idx.to(torch.int32).reshape(batch, heads, -1).sort(dim=-1, descending=True)[0]
    return v, s


# ---------------------------------------------------------------------------------
# attention semantics as masked-dense fp32
# ---------------------------------------------------------------------------------

def vs_mask_for_rows(block_count, block_offset, column_count, column_index, n_ctx, row_blocks):
    """Boolean mask ``[len(row_blocks)*64, n_ctx]`` enabled by one head's index tensors.

    Follows ops/pit_sparse_flash_attention_v2.py:104-148: slash tile ``t`` of row block
    ``m`` enables ``(r, c)`` for ``c in [t, t+64)``, ``c <= r``, ``c < n_ctx``; a gathered
    column enables all 64 rows of the block (no causal test in that loop).
    """
    out = np.zeros((len(row_blocks) * 64, n_ctx), dtype=bool)
    for i, m in enumerate(row_blocks):
        rows = np.arange(m * 64, m * 64 + 64)
        sub = out[i * 64:(i + 1) * 64]
        for t in block_offset[m, : block_count[m]]:
            lo, hi = int(t), min(int(t) + 64, n_ctx)
            if lo >= n_ctx:
                continue
            cols = np.arange(lo, hi)
            sub[:, lo:hi] |= cols[None, :] <= rows[:, None]
        cols = column_index[m, : column_count[m]]
        sub[:, cols] = True
    return out


def masked_attention_rows(q, k, v, mask, row_start, sm_scale=None):
    """fp32 softmax(q k^T * scale, masked) v for a slab of rows.

    ``q`` ``[R, D]`` (rows ``row_start .. row_start+R``), ``k, v`` ``[N, D]``, ``mask`` ``[R, N]``.
    Exact softmax (the reference's torch_forward at ops/pit_sparse_flash_attention.py:596-610
    adds 1e-6 and clamps the max; the Triton kernel it is compared with does not).
    Rows with an empty mask return zeros.
    """
    q = q.float()
    k = k.float()
    v = v.float()
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    s = (q @ k.T) * sm_scale
    s = s.masked_fill(~torch.as_tensor(mask), -torch.inf)
    mx = s.max(dim=-1, keepdim=True).values
    mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    p = torch.exp(s - mx)
    denom = p.sum(-1, keepdim=True)
    o = (p @ v) / torch.where(denom == 0, torch.ones_like(denom), denom)
    return o


def vertical_slash_attention_oracle(q, k, v, v_idx, s_idx, row_blocks=None):
    """End-to-end oracle of ``vertical_slash_sparse_attention`` for ``[B,H,N,D]`` inputs
    (ops/pit_sparse_flash_attention_v2.py:195-242).  K/V may have fewer heads (GQA).

    Returns ``(out [B,H,R,D] fp32, index tensors)``; with ``row_blocks`` only those
    64-row blocks are evaluated (R = 64*len(row_blocks), rows past N dropped by caller).
    """
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    vs, ss = presort_indices(v_idx, s_idx, B, H)
    seqlens = np.full((B,), N, np.int32)
    bc, bo, cc, ci = convert_vertical_slash_indexes(seqlens, vs.numpy(), ss.numpy(), N)
    rows = (N + 63) // 64
    rbs = list(range(rows)) if row_blocks is None else list(row_blocks)
    out = torch.zeros(B, H, len(rbs) * 64, D)
    for b in range(B):
        for h in range(H):
            hk = h // (H // Hkv)
            mask = vs_mask_for_rows(bc[b, h], bo[b, h], cc[b, h], ci[b, h], N, rbs)
            for i, m in enumerate(rbs):
                r0, r1 = m * 64, min(m * 64 + 64, N)
                o = masked_attention_rows(q[b, h, r0:r1], k[b, hk], v[b, hk], mask[i * 64:i * 64 + (r1 - r0)], r0)
                out[b, h, i * 64:i * 64 + (r1 - r0)] = o
    return out, (bc, bo, cc, ci)


# ---------------------------------------------------------------------------------
# block-sparse  (ops/block_sparse_flash_attention.py:151-186, kernel :29-112)
# ---------------------------------------------------------------------------------

def build_block_index(query: torch.Tensor, key: torch.Tensor, top_k: int, block: int = 64):
    """Top-k key blocks per query block from mean-pooled Q, K (:151-166).

    Inputs are already padded to a multiple of ``block`` (the caller pads with
    ``block - (N & (block-1))`` rows, a full extra block when N is aligned, :178).
    """
    B, H, N, D = query.shape
    qp = query.reshape(B, H, -1, block, D).mean(dim=-2)
    kp = key.reshape(B, H, -1, block, D).mean(dim=-2)
    am = torch.arange(qp.shape[-2], dtype=torch.int32) * block
    an = torch.arange(kp.shape[-2], dtype=torch.int32) * block
    p = torch.einsum("bhmk,bhnk->bhmn", qp, kp)
    p = p.where(am[None, None, :, None] >= an[None, None, None, :], -torch.inf)
    top_k = min(top_k, N // block)
    return torch.topk(p, top_k, dim=-1).indices.to(torch.int32).sort(dim=-1).values


def block_sparse_pad(n: int, block: int = 64) -> int:
    return block - (n & (block - 1))


def block_sparse_mask_rows(block_index, n_ctx, row_blocks, block: int = 64):
    """Mask from the consumed prefix ``min(m+1, top_k)`` of each row (:81), causal inside tiles."""
    top_k = block_index.shape[-1]
    out = np.zeros((len(row_blocks) * block, n_ctx), dtype=bool)
    for i, m in enumerate(row_blocks):
        rows = np.arange(m * block, (m + 1) * block)
        for bidx in block_index[m, : min(m + 1, top_k)]:
            lo = int(bidx) * block
            hi = min(lo + block, n_ctx)
            if lo >= n_ctx:
                continue
            cols = np.arange(lo, hi)
            out[i * block:(i + 1) * block, lo:hi] |= cols[None, :] <= rows[:, None]
    return out


def block_sparse_attention_oracle(q, k, v, top_k, row_blocks=None):
    """``block_sparse_attention`` (:169-186) as masked-dense fp32; equal head counts or GQA."""
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    pad = block_sparse_pad(N)
    qp = torch.nn.functional.pad(q, [0, 0, 0, pad])
    kp = torch.nn.functional.pad(k, [0, 0, 0, pad])
    rep = H // Hkv
    kp_full = kp.repeat_interleave(rep, dim=1) if rep > 1 else kp
    bidx = build_block_index(qp, kp_full, top_k).numpy()
    rows = (N + 63) // 64
    rbs = list(range(rows)) if row_blocks is None else list(row_blocks)
    out = torch.zeros(B, H, len(rbs) * 64, D)
    for b in range(B):
        for h in range(H):
            hk = h // rep
            mask = block_sparse_mask_rows(bidx[b, h], N, rbs)
            for i, m in enumerate(rbs):
                r0, r1 = m * 64, min(m * 64 + 64, N)
                out[b, h, i * 64:i * 64 + (r1 - r0)] = masked_attention_rows(
                    q[b, h, r0:r1], k[b, hk], v[b, hk], mask[i * 64:i * 64 + (r1 - r0)], r0)
    return out, bidx


# ---------------------------------------------------------------------------------
# A-shape / streaming  (ops/streaming_kernel.py:611-646 and masks at :69-75)
# ---------------------------------------------------------------------------------

def a_shape_mask_rows(n_ctx, n_init, n_local, r0, r1):
    """Rows ``r0..r1``: window ``0 <= i-j < n_local`` plus, when ``n_ctx > n_local``, the
    sink part ``j < n_init and i-j >= n_local`` (streaming_kernel.py:633-643)."""
    i = np.arange(r0, r1)[:, None]
    j = np.arange(n_ctx)[None, :]
    d = i - j
    m = (d >= 0) & (d < n_local)
    if n_ctx > n_local:
        m |= (j < n_init) & (d >= n_local)
    return m


def streaming_attention_oracle(q, k, v, n_init, n_local, row_blocks=None):
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    rep = H // Hkv
    rows = (N + 63) // 64
    rbs = list(range(rows)) if row_blocks is None else list(row_blocks)
    out = torch.zeros(B, H, len(rbs) * 64, D)
    for b in range(B):
        for h in range(H):
            for i, m in enumerate(rbs):
                r0, r1 = m * 64, min(m * 64 + 64, N)
                mask = a_shape_mask_rows(N, n_init, n_local, r0, r1)
                out[b, h, i * 64:i * 64 + (r1 - r0)] = masked_attention_rows(
                    q[b, h, r0:r1], k[b, h // rep], v[b, h // rep], mask, r0)
    return out
