"""The restated estimator and block-sparse index builder against fixtures produced by
executing the reference's own functions (tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import torch

from oracle import reference_math as R


def test_estimator_matches_reference_fixtures(golden_dir):
    paths = sorted(glob.glob(os.path.join(golden_dir, "estimator_[0-9]*.npz")))
    assert len(paths) >= 4
    for path in paths:
        z = np.load(path)
        n = int(z["n"])
        k = torch.from_numpy(z["k"]).float()[None, None]
        q = torch.zeros(1, 1, n, k.shape[-1])
        q[0, 0, -64:] = torch.from_numpy(z["q_last"]).float()
        v_idx, s_idx = R.vertical_slash_estimate(q, k, int(z["vertical_size"]), int(z["slash_size"]))
        assert v_idx.shape == tuple(z["v_idx"].shape) and v_idx.dim() == 4      # the 4-D quirk of the reference
        assert s_idx.shape == tuple(z["s_idx"].shape)
        assert set(v_idx.flatten().tolist()) == set(z["v_idx"].flatten().tolist()), path
        assert set(s_idx.flatten().tolist()) == set(z["s_idx"].flatten().tolist()), path
        # forced entries: first 30 columns, nearest 100 diagonals (when the budgets allow)
        if v_idx.numel() >= 30:
            assert set(range(min(30, n))) <= set(v_idx.flatten().tolist())
        if s_idx.numel() >= 100:
            assert set(range(100)) <= set(s_idx.flatten().tolist())


def test_estimator_matches_reference_run_in_bf16(golden_dir):
    """The reference's functions executed on bf16 tensors (the dtype of its GPU path): the restatement on the same
    tensors returns the same lists and the same score vectors."""
    paths = sorted(glob.glob(os.path.join(golden_dir, "estimator_bf16_*.npz")))
    assert len(paths) >= 4
    for path in paths:
        z = np.load(path)
        n = int(z["n"])
        k = torch.from_numpy(z["k_bits"]).view(torch.bfloat16)[None, None]
        q = torch.zeros(1, 1, n, 128, dtype=torch.bfloat16)
        q[0, 0, -64:] = torch.from_numpy(z["q_last_bits"]).view(torch.bfloat16)
        v_idx, s_idx, vsc, ssc = R.vertical_slash_estimate(q, k, int(z["vertical_size"]), int(z["slash_size"]), return_scores=True)
        assert set(v_idx.flatten().tolist()) == set(z["v_idx"].flatten().tolist()), path
        assert set(s_idx.flatten().tolist()) == set(z["s_idx"].flatten().tolist()), path
        assert np.array_equal(vsc.float().numpy(), z["vertical_scores"])
        got, want = ssc.float().flip(0).numpy(), z["slash_scores_by_offset"]       # the diagonal sums add in another order
        fin = np.isfinite(want)
        assert np.array_equal(np.isfinite(got), fin) and np.allclose(got[fin], want[fin], rtol=2e-6, atol=1e-9)


def test_diagonal_sum_definition():
    torch.manual_seed(0)
    n, m = 5, 11
    mat = torch.rand(1, 1, n, m)
    got = R.sum_all_diagonal_matrix(mat)[0, 0]
    for j in range(n + m - 1):
        want = sum(mat[0, 0, i, i + j + 1 - n] for i in range(n) if 0 <= i + j + 1 - n < m)
        assert abs(float(got[j]) - float(want)) < 1e-5


def test_block_index_matches_reference_fixtures(golden_dir):
    paths = sorted(glob.glob(os.path.join(golden_dir, "block_index_*.npz")))
    assert len(paths) >= 3
    for path in paths:
        z = np.load(path)
        n, top_k = int(z["n"]), int(z["top_k"])
        q = torch.from_numpy(z["q"]).float()
        k = torch.from_numpy(z["k"]).float()
        pad = R.block_sparse_pad(n)
        qp = torch.nn.functional.pad(q, [0, 0, 0, pad])
        kp = torch.nn.functional.pad(k, [0, 0, 0, pad])
        got = R.build_block_index(qp, kp, top_k).numpy()
        ref = z["block_index"]
        assert got.shape == ref.shape
        rows = got.shape[2]
        for m in range(rows):           # bit-exact on the prefix the kernel consumes
            c = min(m + 1, got.shape[-1])
            assert np.array_equal(got[..., m, :c], ref[..., m, :c]), (path, m)
