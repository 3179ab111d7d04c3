"""The restated FlexPrefill block selection against fixtures produced by executing the reference's own
``get_active_blocks`` on CPU (tests/golden/make_golden.py)."""
import glob
import hashlib
import os

import numpy as np
import torch

from oracle import reference_math as R


def fixture_case(path):
    """Inputs regenerated from the seed (checked against the stored digest), parameters and the reference's block set."""
    from minference_b200.synthetic import make_qkv

    z = np.load(path)
    n, heads, kv_heads = int(z["n"]), int(z["heads"]), int(z["kv_heads"])
    q, k, v = make_qkv(n, heads, kv_heads, seed=int(z["seed"]), dtype=torch.bfloat16, plant=bool(z["plant"]))
    h = hashlib.sha256()
    for t in (q, k):
        h.update(t.contiguous().view(torch.int16).numpy().tobytes())
    assert h.hexdigest() == str(z["inputs_sha256"]), "the seeded generator no longer reproduces the fixture's inputs"
    nb = int(z["nb"])
    ref = np.unpackbits(z["block_mask"], axis=-1)[..., :nb].astype(bool)
    params = dict(gamma=float(z["gamma"]), tau=float(z["tau"]), min_budget=int(z["min_budget_blocks"]),
                  max_budget=int(z["max_budget_blocks"]))
    return q, k, v, params, ref


def test_block_selection_matches_reference_fixtures(golden_dir):
    paths = sorted(glob.glob(os.path.join(golden_dir, "flexprefill_*.npz")))
    assert len(paths) >= 5
    kinds = set()
    for path in paths:
        q, k, _, p, ref = fixture_case(path)
        mask, det = R.flex_active_block_mask(q, k, 128, p["gamma"], p["min_budget"], p["max_budget"], p["tau"],
                                             return_details=True)
        assert np.array_equal(mask[0].numpy(), ref), path
        nb = ref.shape[-1]
        assert all(ref[h, i, i] for h in range(ref.shape[0]) for i in range(nb))        # main block diagonal forced
        assert ref[:, :, 0].all() and not np.triu(ref, 1).any()                          # first key block; causal
        kinds.add((bool(det["block_sparse"].any()), bool(ref.sum() < ref.shape[0] * nb * (nb + 1) // 2)))
    assert (True, True) in kinds and (False, True) in kinds       # both head kinds occur with a sparse block set


def test_attention_oracle_over_a_block_set_is_causal_inside_blocks():
    torch.manual_seed(0)
    n, bs = 300, 128
    q, k, v = torch.randn(1, 1, n, 128), torch.randn(1, 1, n, 128), torch.randn(1, 1, n, 128)
    nb = 3
    full = torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None, None]
    out, _ = R.flexprefill_attention_oracle(q, k, v, 0.9, block_size=bs, block_mask=full)
    want = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert torch.allclose(out[:, :, :n], want, atol=2e-5)
    # short sequences take the dense path
    out2, bm = R.flexprefill_attention_oracle(q[:, :, :200], k[:, :, :200], v[:, :, :200], 0.9, block_size=bs)
    assert bm.all(dim=0).all(dim=0).equal(torch.tril(torch.ones(2, 2, dtype=torch.bool)))
    assert torch.allclose(out2[:, :, :200], torch.nn.functional.scaled_dot_product_attention(
        q[:, :, :200], k[:, :, :200], v[:, :, :200], is_causal=True), atol=2e-5)


def test_host_side_block_selection_of_the_product_matches_reference_fixtures(golden_dir):
    """``select_blocks`` (budgets, pooling, Jensen-Shannon test, top-k, block-sparse fallback: the part of the product
    that is plain torch) fed with the last-block scores computed in torch on CPU: the reference's block sets, bit for bit."""
    import math

    from minference_b200.modules.flexprefill import select_blocks

    for path in sorted(glob.glob(os.path.join(golden_dir, "flexprefill_*.npz"))):
        q, k, _, p, ref = fixture_case(path)
        D = q.shape[-1]
        kk = k.repeat_interleave(q.shape[1] // k.shape[1], 1)
        last_q = q[:, :, -128:] / math.sqrt(D)
        qk = torch.einsum("bhid,bhjd->bhij", last_q, kk)
        causal = torch.arange(128)[:, None] >= torch.arange(128)[None, :]
        qk[..., -128:].masked_fill_(~causal, float("-inf"))
        pr = torch.softmax(qk, dim=-1, dtype=torch.float32)
        slash_by_offset = (R.flex_sum_all_diagonal_matrix(pr) / 128).flip(-1)
        mask = select_blocks(pr.mean(-2), slash_by_offset, last_q, q, k, 128, p["gamma"], p["min_budget"], p["max_budget"], p["tau"])
        assert np.array_equal(mask[0].numpy(), ref), path
