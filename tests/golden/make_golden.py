"""Generate the golden fixtures in this folder from the reference itself.

Run where the reference tree (microsoft/MInference v0.1.6.0) is checked out: ``MINFERENCE_REFERENCE``
points at it, or it sits in a directory named ``reference`` beside this repository:

    python oracle/build_ref.py --host
    python tests/golden/make_golden.py

What is executed is the reference's own code, not this repository's restatement:

* ``vs_index_*.npz``   -- ``convert_vertical_slash_indexes_kernel`` of
  ``csrc/vertical_slash_index.cu`` compiled for the host by ``oracle/build_ref.py``.
* ``estimator_*.npz``  -- the body of ``minference_prefill_kernel`` (which contains
  ``vertical_and_slash_kernel``) and ``sum_all_diagonal_matrix`` extracted with ``ast``
  from ``minference/modules/minference_forward.py`` and executed on CPU fp32; the module
  cannot be imported as a whole (it creates CUDA tensors at import time).  The call to
  ``vertical_slash_sparse_attention`` inside is replaced by a recorder of its index
  arguments.
* ``estimator_bf16_*.npz`` -- the same function bodies executed on bf16 tensors (the dtype the
  reference runs in on the GPU: bf16 GEMM output, bf16 division by sqrt(d), fp32 softmax), with
  the score vectors it hands to ``torch.topk`` recorded beside the index lists, so that a test
  can tell a wrong selection from a near-tie at the top-k boundary.
* ``block_index_*.npz`` -- ``_build_block_index`` of
  ``minference/ops/block_sparse_flash_attention.py`` loaded by file path.
* ``flexprefill_*.npz`` -- ``get_active_blocks`` of ``minference/modules/flexprefill.py`` loaded by file
  path and run on CPU bf16 tensors, with its Triton key-pooling helper replaced by the same mean in torch.

The fixtures are small seeded cases; the tests also compare larger seeded cases through
sha256 digests stored in ``digests.json``.
"""
from __future__ import annotations

import ast
import hashlib
import importlib.util
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import reference_math as R  # noqa: E402  (only for the ctypes loader of the reference host library)

from oracle.build_ref import reference_tree  # noqa: E402

REFERENCE = reference_tree()


def index_case(seed: int, n: int, heads: int, nnz_v: int, nnz_s: int, style: str):
    g = np.random.default_rng(seed)
    v = np.sort(g.integers(0, n, size=(1, heads, nnz_v)), axis=-1).astype(np.int32)
    if style == "uniform":
        s = g.integers(0, n, size=(1, heads, nnz_s))
    elif style == "clustered":      # runs of near-equal offsets: exercises the extend-by-64 rule
        s = (g.integers(0, max(n // 48, 1), size=(1, heads, nnz_s)) * 48 + g.integers(0, 5, size=(1, heads, nnz_s))) % n
    elif style == "strided":        # gaps between 50 and 140: every branch of the range logic
        s = np.cumsum(g.integers(50, 140, size=(1, heads, nnz_s)), axis=-1) % n
    elif style == "local":          # the estimator's forced diagonals 0..nnz_s-1
        s = np.broadcast_to(np.arange(nnz_s) % n, (1, heads, nnz_s)).copy()
    else:
        raise ValueError(style)
    s = s.astype(np.int32)
    s[..., 0] = g.integers(0, 64, size=(1, heads))   # the reference needs an offset < 64 (it has no bounds check)
    s = -np.sort(-s, axis=-1)
    return v, np.ascontiguousarray(s)


INDEX_SMALL = [  # (seed, n, heads, nnz_v, nnz_s, style)
    (0, 64, 1, 1, 1, "uniform"),
    (1, 100, 2, 7, 9, "uniform"),
    (2, 1000, 2, 30, 50, "clustered"),
    (3, 1024, 1, 64, 100, "strided"),
    (4, 4096, 2, 100, 300, "uniform"),
    (5, 4100, 1, 33, 257, "local"),
]
INDEX_DIGEST = [
    (10, 8192, 2, 1000, 6096, "uniform"),
    (11, 8192, 1, 1000, 6096, "local"),
    (12, 20000, 1, 1000, 6096, "clustered"),
    (13, 65536, 1, 500, 3000, "strided"),
]


def digest(arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def make_index_fixtures(digests: dict):
    for (seed, n, heads, nv, ns, style) in INDEX_SMALL:
        v, s = index_case(seed, n, heads, nv, ns, style)
        bc, bo, cc, ci = R.convert_vertical_slash_indexes_ref_host(np.array([n], np.int32), v, s, n)
        np.savez_compressed(os.path.join(HERE, f"vs_index_{seed}.npz"), n=n, v=v, s=s, block_count=bc,
                            block_offset=bo, column_count=cc, column_index=ci)
    for (seed, n, heads, nv, ns, style) in INDEX_DIGEST:
        v, s = index_case(seed, n, heads, nv, ns, style)
        outs = R.convert_vertical_slash_indexes_ref_host(np.array([n], np.int32), v, s, n)
        digests[f"vs_index_{seed}"] = {"args": [seed, n, heads, nv, ns, style], "sha256": digest(outs),
                                       "tiles": int(outs[0].sum() + ((outs[2] + 63) // 64).sum())}


class _TorchRecordingTopk:
    """Stands in for the ``torch`` module inside the extracted functions: everything is torch's own,
    except that the inputs of ``topk`` are kept."""

    def __init__(self, sink: dict):
        self._sink = sink

    def __getattr__(self, name):
        return getattr(torch, name)

    def topk(self, x, *a, **kw):
        self._sink.setdefault("topk_inputs", []).append(x.detach().clone())
        return torch.topk(x, *a, **kw)


def load_reference_prefill_kernel(record_scores: bool = False):
    """exec the reference's estimator functions on CPU with the attention call recorded."""
    path = os.path.join(REFERENCE, "minference", "modules", "minference_forward.py")
    tree = ast.parse(open(path).read())
    wanted = {"sum_all_diagonal_matrix", "minference_prefill_kernel"}
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in wanted]
    assert {n.name for n in body} == wanted
    captured = {}

    def record(q, k, v, v_idx, s_idx):
        captured["v_idx"] = v_idx.clone()
        captured["s_idx"] = s_idx.clone()
        return torch.zeros_like(q)

    ar = torch.arange(64)
    ns = {
        "torch": _TorchRecordingTopk(captured) if record_scores else torch, "math": math,
        "LAST_Q_MASK": ar[None, None, :, None] >= ar[None, None, None, :],
        "vertical_slash_sparse_attention": record,
        "streaming_forward": None, "block_sparse_attention": None,
    }
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    return ns["minference_prefill_kernel"], captured


ESTIMATOR_CASES = [  # (seed, n, vertical_size, slash_size)
    (20, 600, 100, 200),
    (21, 1024, 30, 100),
    (22, 2048, 300, 700),
    (23, 160, 1000, 6096),   # budgets larger than the context: clamped to n
]


def make_estimator_fixtures():
    from minference_b200.synthetic import make_qkv

    kernel, captured = load_reference_prefill_kernel()
    for (seed, n, vs, ss) in ESTIMATOR_CASES:
        q, k, v = make_qkv(n, 1, 1, seed=seed, dtype=torch.float16)   # fp16-exact values keep the file small
        qf, kf = q.float(), k.float()
        cfg = {"best_pattern": [{"0": ["vertical_and_slash", vs, ss, 1.0]}]}
        kernel(qf, kf, v.float(), 0, 0, cfg)
        np.savez_compressed(os.path.join(HERE, f"estimator_{seed}.npz"), n=n, vertical_size=vs, slash_size=ss,
                            q_last=q[0, 0, -64:].numpy(), k=k[0, 0].numpy(),
                            v_idx=captured["v_idx"].numpy(), s_idx=captured["s_idx"].numpy())


ESTIMATOR_BF16_CASES = [  # (seed, n, vertical_size, slash_size)
    (40, 600, 100, 200),
    (41, 2048, 300, 700),
    (42, 4096, 1000, 3000),
    (43, 8192, 1000, 6096),
]


def make_estimator_bf16_fixtures():
    from minference_b200.synthetic import make_qkv

    kernel, captured = load_reference_prefill_kernel(record_scores=True)
    for (seed, n, vs, ss) in ESTIMATOR_BF16_CASES:
        q, k, v = make_qkv(n, 1, 1, seed=seed, dtype=torch.bfloat16)
        cfg = {"best_pattern": [{"0": ["vertical_and_slash", vs, ss, 1.0]}]}
        captured.pop("topk_inputs", None)
        kernel(q, k, v, 0, 0, cfg)
        vertical, slash = captured["topk_inputs"]           # [1,1,1,n] with the first 30 forced, [1,1,n] with the last 100 forced
        np.savez_compressed(os.path.join(HERE, f"estimator_bf16_{seed}.npz"), n=n, vertical_size=vs, slash_size=ss,
                            q_last_bits=q[0, 0, -64:].view(torch.int16).numpy(), k_bits=k[0, 0].view(torch.int16).numpy(),
                            v_idx=captured["v_idx"].numpy(), s_idx=captured["s_idx"].numpy(),
                            vertical_scores=vertical.float().reshape(-1).numpy(),
                            slash_scores_by_offset=slash.float().reshape(-1).flip(0).numpy())


BLOCK_CASES = [  # (seed, n, heads, top_k)
    (30, 512, 1, 3),
    (31, 1000, 1, 5),
    (32, 2048, 1, 100),
]


def make_block_fixtures():
    from minference_b200.synthetic import make_qkv

    path = os.path.join(REFERENCE, "minference", "ops", "block_sparse_flash_attention.py")
    spec = importlib.util.spec_from_file_location("ref_block_sparse", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for (seed, n, heads, top_k) in BLOCK_CASES:
        q, k, _ = make_qkv(n, heads, heads, seed=seed, dtype=torch.float16)
        pad = 64 - (n & 63)
        qp = torch.nn.functional.pad(q.float(), [0, 0, 0, pad])
        kp = torch.nn.functional.pad(k.float(), [0, 0, 0, pad])
        bidx = mod._build_block_index(qp, kp, top_k, 64, 64)
        np.savez_compressed(os.path.join(HERE, f"block_index_{seed}.npz"), n=n, top_k=top_k,
                            q=q.numpy(), k=k.numpy(), block_index=bidx.numpy())


FLEX_CASES = [  # (seed, n, heads, kv_heads, gamma, tau, min_budget_blocks, max_budget_blocks, planted sinks)
    (50, 1500, 4, 2, 0.9, 0.1, 1, 1 << 20, True),
    (51, 2048, 2, 1, 0.95, 0.0, 1, 1 << 20, True),
    (52, 1100, 2, 2, 0.5, 0.0, 2, 4, True),
    (53, 3000, 2, 1, 0.9, 0.1, 1, 1 << 20, False),
    (54, 2500, 2, 1, 0.9, 0.0, 1, 6, False),
]


def flex_case_inputs(seed, n, heads, kv_heads, plant):
    from minference_b200.synthetic import make_qkv

    return make_qkv(n, heads, kv_heads, seed=seed, dtype=torch.bfloat16, plant=plant)


def input_digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.int16).numpy().tobytes())
    return h.hexdigest()


def make_flexprefill_fixtures():
    """``flexprefill_*.npz``: ``get_active_blocks`` of ``minference/modules/flexprefill.py`` loaded by file path and
    executed on CPU bf16 tensors.  Its key pooling is a Triton kernel and cannot run without a GPU, so that one
    function (``triton_bnhd_pool``, average over blocks of rows, a short last block divided by its own length) is
    replaced by the same arithmetic in torch; everything else is the reference's code.  The inputs are regenerated
    from their seed by the test and checked against the stored sha256."""
    path = os.path.join(REFERENCE, "minference", "modules", "flexprefill.py")
    spec = importlib.util.spec_from_file_location("ref_flexprefill", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    def pool(x, kernel_size, pool_type="avg"):          # [b, n, h, d]
        b, n, h, d = x.shape
        m = math.ceil(n / kernel_size)
        xp = torch.nn.functional.pad(x.float(), (0, 0, 0, 0, 0, m * kernel_size - n))
        cnt = torch.full((m,), float(kernel_size))
        cnt[-1] = n - (m - 1) * kernel_size
        return (xp.view(b, m, kernel_size, h, d).sum(2) / cnt[None, :, None, None]).to(x.dtype)

    mod.triton_bnhd_pool = pool
    for (seed, n, heads, kv_heads, gamma, tau, min_b, max_b, plant) in FLEX_CASES:
        q, k, v = flex_case_inputs(seed, n, heads, kv_heads, plant)
        mod.causal_mask = None
        blocks = mod.get_active_blocks(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(),
                                       v.transpose(1, 2).contiguous(), 128, gamma, min_b, max_b, tau)
        nb = math.ceil(n / 128)
        mask = np.zeros((heads, nb * nb), dtype=bool)
        for h in range(heads):
            mask[h, blocks[0][h].numpy()] = True
        np.savez_compressed(os.path.join(HERE, f"flexprefill_{seed}.npz"), seed=seed, n=n, heads=heads, kv_heads=kv_heads,
                            gamma=gamma, tau=tau, min_budget_blocks=min_b, max_budget_blocks=max_b, plant=plant,
                            block_mask=np.packbits(mask.reshape(heads, nb, nb), axis=-1), nb=nb,
                            inputs_sha256=input_digest(q, k))


def main():
    if not os.path.isdir(REFERENCE):
        sys.exit("no reference tree: set MINFERENCE_REFERENCE to the checked-out tree")
    digests = {}
    make_index_fixtures(digests)
    make_estimator_fixtures()
    make_estimator_bf16_fixtures()
    make_block_fixtures()
    make_flexprefill_fixtures()
    with open(os.path.join(HERE, "digests.json"), "w") as f:
        json.dump(digests, f, indent=1, sort_keys=True)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
