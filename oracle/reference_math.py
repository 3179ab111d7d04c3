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


# ---------------------------------------------------------------------------------
# FlexPrefill  (modules/flexprefill.py:880-1112)
# ---------------------------------------------------------------------------------

def flex_score_cover_topk(x: torch.Tensor, score: float) -> torch.Tensor:
    """How many of the largest entries it takes to pass ``score`` in sum (:880-883)."""
    cumsum_x = torch.cumsum(torch.sort(x, dim=-1, descending=True).values, dim=-1)
    return torch.sum(cumsum_x <= score, dim=-1) + 1


def flex_sum_pool(x: torch.Tensor, kernel: int) -> torch.Tensor:
    """Sums over consecutive groups of ``kernel`` entries of the last axis, the tail zero-padded (:866-877)."""
    n = x.shape[-1]
    x = torch.nn.functional.pad(x, (0, math.ceil(n / kernel) * kernel - n), value=0)
    return x.view(*x.shape[:-1], -1, kernel).sum(-1)


def flex_avg_pool_rows(x: torch.Tensor, kernel: int) -> torch.Tensor:
    """Mean over consecutive groups of ``kernel`` rows of ``[B,H,N,D]``, a short last group divided by its own
    length, result in the input dtype (the reference's pooling kernel, :662-727, pool type "avg")."""
    B, H, N, D = x.shape
    nb = math.ceil(N / kernel)
    xp = torch.nn.functional.pad(x.float(), (0, 0, 0, nb * kernel - N))
    cnt = torch.full((nb,), float(kernel))
    cnt[-1] = N - (nb - 1) * kernel
    return (xp.view(B, H, nb, kernel, D).sum(3) / cnt[None, None, :, None]).to(x.dtype)


def flex_sum_all_diagonal_matrix(mat: torch.Tensor) -> torch.Tensor:
    """``[b,h,n,m] -> [b,h,m]``: entry j is ``sum_i mat[i, i + j + 1 - n]`` (:893-900, the zero-pad + strided view
    written as an index-add)."""
    b, h, n, m = mat.shape
    j = torch.arange(m)[None, :] - torch.arange(n)[:, None] + n - 1          # 0 .. n+m-2
    out = torch.zeros(b, h, n + m - 1, dtype=mat.dtype)
    out.index_add_(2, j.reshape(-1), mat.reshape(b, h, n * m))
    return out[..., :m]


def flex_square_root_js_divergence(p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    m = (p + q) / 2                                                          # :946-950
    return torch.sqrt(0.5 * (p * torch.log(p / m)).sum(-1) + 0.5 * (q * torch.log(q / m)).sum(-1))


def flex_active_block_mask(q: torch.Tensor, k: torch.Tensor, block_size: int, gamma: float, min_budget: int,
                           max_budget: int, tau: float = 0.0, return_details: bool = False):
    """``get_active_blocks`` (:953-1067) for ``[B,H,N,D]`` queries and ``[B,Hkv,N,D]`` keys (query head h reads KV
    head ``h // (H/Hkv)``, the non-interleaved grouping), budgets in blocks.  Returns the block set as a boolean
    matrix ``[B,H,nb,nb]`` (entry (i, j): query block i attends key block j) instead of the reference's lists of
    flattened ids ``i*nb + j``; block (0, 0), which the reference's padding value 0 stands for, is always in the set
    because the first key block and the main block diagonal are forced.
    """
    B, H, N, D = q.shape
    Hkv = k.shape[1]
    rep = H // Hkv
    nb = math.ceil(N / block_size)
    max_budget = min(max_budget, nb)
    kk = k.repeat_interleave(rep, dim=1) if rep > 1 else k
    last_q = q[:, :, -block_size:, :] / math.sqrt(D)                         # :968 (rounds in the input dtype)
    qk = torch.einsum("bhid,bhjd->bhij", last_q, kk)                         # :969-980, product in the input dtype
    bs = last_q.shape[2]
    causal = torch.arange(bs)[:, None] >= torch.arange(bs)[None, :]
    qk[..., -bs:].masked_fill_(~causal, float("-inf"))                       # :981-988
    qk = torch.softmax(qk, dim=-1, dtype=torch.float32)                      # :990
    slash = flex_sum_all_diagonal_matrix(qk) / qk.shape[-2]                  # :992, index j <-> offset N-1-j
    vertical = qk.mean(-2)                                                   # :993
    n_vert = flex_score_cover_topk(vertical, gamma) // 128 + 1               # :995-996 (128 is a constant there)
    n_slash = flex_score_cover_topk(slash, gamma) // 128 + 1
    n_vert = n_vert.clamp(min_budget, max_budget)                            # :997-1000
    n_slash = n_slash.clamp(min_budget, max_budget)
    vertical = flex_sum_pool(vertical, block_size)                           # :1002-1003
    slash = flex_sum_pool(slash, block_size)
    avg_k = flex_avg_pool_rows(kk, block_size)                               # :1005-1008
    avg_qk = torch.einsum("bhd,bhjd->bhj", last_q.mean(2), avg_k)           # :1009-1011
    avg_qk = torch.softmax(avg_qk, dim=-1, dtype=torch.float32)
    js = flex_square_root_js_divergence(avg_qk, vertical)                    # :1013
    block_sparse = js < tau                                                  # :1014
    n_vert = torch.where(block_sparse, torch.full_like(n_vert, min_budget), n_vert)     # :1015-1016
    n_slash = torch.where(block_sparse, torch.full_like(n_slash, min_budget), n_slash)
    vertical = vertical.clone()
    slash = slash.clone()
    vertical[..., :1] = torch.inf                                            # :1018-1019
    slash[..., -1:] = torch.inf
    mask = torch.zeros(B, H, nb, nb, dtype=torch.bool)
    ii = torch.arange(nb)
    for b in range(B):
        for h in range(H):
            # slash: the n_slash best pooled entries -> block diagonals d = nb-1-index (:1021-1031, :914-917)
            ks = min(int(n_slash[b, h]), nb)
            d_sel = (nb - 1) - slash[b, h].topk(ks).indices
            for d in d_sel.tolist():
                rows = ii[ii + d < nb] + d
                mask[b, h, rows, rows - d] = True
            # vertical: the n_vert best key blocks, for the query blocks at or below them (:1033-1046, :908-913)
            kv = min(int(n_vert[b, h]), nb)
            for j in vertical[b, h].topk(kv).indices.tolist():
                mask[b, h, j:, j] = True
            if bool(block_sparse[b, h]):                                     # :1049-1066
                pad_q = nb * block_size - N
                avg_q = torch.nn.functional.pad(q[b, h], (0, 0, 0, pad_q)).view(nb, block_size, D).mean(1)
                avg_q[-1] = avg_q[-1] * block_size / (block_size - pad_q)
                attn = torch.einsum("id,jd->ij", avg_q / math.sqrt(D), avg_k[b, h])
                attn = attn.masked_fill(~torch.tril(torch.ones(nb, nb, dtype=torch.bool)), float("-inf"))
                attn = torch.softmax(attn, dim=-1, dtype=torch.float32).view(-1)
                vals, idx = torch.sort(attn, descending=True)
                keep = idx[torch.cumsum(vals, dim=-1) <= gamma * nb]         # :886-890
                mask[b, h].view(-1)[keep] = True
    if return_details:
        return mask, {"n_vertical": n_vert, "n_slash": n_slash, "block_sparse": block_sparse, "js": js,
                      "vertical_pooled": vertical, "slash_pooled": slash}
    return mask


def flex_block_mask_rows(block_mask, n_ctx: int, block_size: int, r0: int, r1: int):
    """Token-level mask of rows ``r0..r1`` from a ``[nb, nb]`` block set: the selected key blocks of the row's query
    block, causal inside (:434-436)."""
    i = np.arange(r0, r1)
    j = np.arange(n_ctx)
    sel = np.asarray(block_mask)[(i // block_size)[:, None], (j // block_size)[None, :]]
    return sel & (j[None, :] <= i[:, None])


def flexprefill_attention_oracle(q, k, v, gamma: float, tau: float = 0.0, min_budget=None, max_budget=None,
                                 block_size: int = 128, row_blocks=None, block_mask=None):
    """``flex_prefill_attention`` (:1070-1112) as masked-dense fp32 over the block set, ``[B,H,N,D]`` layout.
    Returns ``(out [B,H,len(row_blocks)*64,D], block_mask)``; sequences too short for the sparse path
    (:1087-1088) are dense causal."""
    B, H, N, D = q.shape
    rep = H // k.shape[1]
    min_budget = 1 if min_budget is None else min_budget
    max_budget = 2147483647 if max_budget is None else max_budget
    nb = math.ceil(N / block_size)
    if block_mask is None:
        if N <= max(2 * block_size, math.ceil(min_budget / block_size) * block_size):
            block_mask = torch.tril(torch.ones(nb, nb, dtype=torch.bool)).expand(B, H, nb, nb)
        else:
            block_mask = flex_active_block_mask(q, k, block_size, gamma, math.ceil(min_budget / block_size),
                                                math.ceil(max_budget / block_size), tau)
    rows = (N + 63) // 64
    rbs = list(range(rows)) if row_blocks is None else list(row_blocks)
    out = torch.zeros(B, H, len(rbs) * 64, D)
    for b in range(B):
        for h in range(H):
            bm = block_mask[b, h].numpy()
            for i, m in enumerate(rbs):
                r0, r1 = m * 64, min(m * 64 + 64, N)
                out[b, h, i * 64:i * 64 + (r1 - r0)] = masked_attention_rows(
                    q[b, h, r0:r1], k[b, h // rep], v[b, h // rep], flex_block_mask_rows(bm, N, block_size, r0, r1), r0)
    return out, block_mask
