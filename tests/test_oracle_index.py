"""The CPU oracle of the index conversion against fixtures made from the reference kernel."""
import glob
import json
import os

import numpy as np
import pytest

from oracle import reference_math as R
from tests.golden.make_golden import INDEX_DIGEST, digest, index_case


def _small_cases(golden_dir):
    return sorted(glob.glob(os.path.join(golden_dir, "vs_index_*.npz")))


def test_fixtures_present(golden_dir):
    assert len(_small_cases(golden_dir)) >= 6


def test_oracle_matches_reference_fixtures(golden_dir):
    for path in _small_cases(golden_dir):
        z = np.load(path)
        n = int(z["n"])
        outs = R.convert_vertical_slash_indexes(np.array([n], np.int32), z["v"], z["s"], n)
        for name, got in zip(("block_count", "block_offset", "column_count", "column_index"), outs):
            assert np.array_equal(got, z[name]), (path, name)


def test_oracle_matches_reference_digests(golden_dir):
    digests = json.load(open(os.path.join(golden_dir, "digests.json")))
    for (seed, n, heads, nv, ns, style) in INDEX_DIGEST:
        v, s = index_case(seed, n, heads, nv, ns, style)
        outs = R.convert_vertical_slash_indexes(np.array([n], np.int32), v, s, n)
        entry = digests[f"vs_index_{seed}"]
        assert digest(outs) == entry["sha256"], seed
        assert int(outs[0].sum() + ((outs[2] + 63) // 64).sum()) == entry["tiles"]


@pytest.mark.skipif(not os.path.exists(R.ref_host_lib_path()), reason="reference host build absent")
def test_oracle_matches_reference_kernel_random():
    rng = np.random.default_rng(123)
    for trial in range(60):
        n = int(rng.integers(64, 6000))
        v, s = index_case(1000 + trial, n, int(rng.integers(1, 4)), int(rng.integers(1, 200)),
                          int(rng.integers(1, 400)), ["uniform", "clustered", "strided", "local"][trial % 4])
        a = R.convert_vertical_slash_indexes(np.array([n], np.int32), v, s, n)
        b = R.convert_vertical_slash_indexes_ref_host(np.array([n], np.int32), v, s, n)
        for x, y in zip(a, b):
            assert np.array_equal(x, y), trial


def test_oracle_reports_missing_small_offset():
    v = np.array([[[0, 5]]], np.int32)
    s = np.array([[[500, 200]]], np.int32)      # no offset below 64: row block 0 has no usable slash
    with pytest.raises(ValueError):
        R.convert_vertical_slash_indexes(np.array([1024], np.int32), v, s, 1024)


def test_index_invariants():
    """Properties of the reference index set that the attention kernel relies on."""
    for seed in range(5):
        n = 3000 + 97 * seed
        v, s = index_case(seed, n, 1, 80, 150, "uniform")
        s[..., -1] = 0      # with the main diagonal present (the estimator always forces it) the
                            # index set covers the whole fine-grained mask; without it, verticals
                            # right of the last range are dropped
        bc, bo, cc, ci = R.convert_vertical_slash_indexes(np.array([n], np.int32), v, s, n)
        rows = (n + 63) // 64
        for m in range(rows):
            tiles = bo[0, 0, m, : bc[0, 0, m]]
            cols = ci[0, 0, m, : cc[0, 0, m]]
            assert bc[0, 0, m] >= 1 and tiles[0] <= 64 * m            # first tile reaches the diagonal block or before
            assert np.all(np.diff(tiles) >= 64)                        # disjoint ascending tiles
            assert np.all(cols < 64 * m) if len(cols) else True        # gathered columns are strictly causal
            assert bc[0, 0, m] <= s.shape[2] and cc[0, 0, m] <= v.shape[2]
            # superset of the fine-grained vertical/slash mask for the rows of this block
            r = np.arange(64 * m, min(64 * m + 64, n))
            mask = R.vs_mask_for_rows(bc[0, 0], bo[0, 0], cc[0, 0], ci[0, 0], n, [m])[: len(r)]
            fine = np.zeros_like(mask)
            fine[:, v[0, 0]] = True
            for o in s[0, 0]:
                c = r - o
                ok = c >= 0
                fine[np.arange(len(r))[ok], c[ok]] = True
            fine &= np.arange(n)[None, :] <= r[:, None]
            assert not np.any(fine & ~mask)
