"""Offline pattern search scored through the kernels' log-sum-exp against the attention mass
computed from the full [N, N] probability matrix (what the reference's search materialises)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_search_scores_match_attention_mass_of_the_masks():
    from minference_b200.modules.pattern_search import CANDIDATES, search_layer_patterns, search_vertical_slash_lists
    from minference_b200.ops.block_sparse_flash_attention import _build_block_index, _rows_pad
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    n, hq, hkv = 3072, 2, 1
    q, k, v = make_qkv(n, hq, hkv, seed=11, dtype=torch.bfloat16)
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    best, table = search_layer_patterns(dq, dk, dv, return_all=True)
    assert [c[:3] for c in table] == list(CANDIDATES)

    r0 = 2500
    rbs = list(range(n // 64))
    for h in range(hq):
        s = (q[0, h].float() @ k[0, 0].float().T) * 128 ** -0.5
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
        p = torch.softmax(s, -1)[r0:]
        ref_scores = []
        for ty, vs, ss in CANDIDATES:
            if ty == "stream_llm":
                mask = R.a_shape_mask_rows(n, vs, ss + 1, 0, n)
            elif ty == "vertical_and_slash":
                v_idx, s_idx, nnz_v, nnz_s = search_vertical_slash_lists(dq, dk, vs, ss)
                assert int(nnz_v[h]) == min(n, vs) and int(nnz_s[h]) == min(n, ss)       # budgets as given, not raised
                assert set(range(30)) <= set(s_idx[0, h, : int(nnz_s[h])].tolist())         # the 30 nearest diagonals, not 100
                if ss == 100:
                    assert not set(range(100)) <= set(s_idx[0, h, :100].tolist())
                bc, bo, cc, ci = R.convert_vertical_slash_indexes(
                    np.array([n], np.int32), v_idx[:, h:h + 1, : int(nnz_v[h])].cpu().numpy(),
                    s_idx[:, h:h + 1, : int(nnz_s[h])].cpu().numpy(), n)
                mask = R.vs_mask_for_rows(bc[0, 0], bo[0, 0], cc[0, 0], ci[0, 0], n, rbs)
            else:
                bidx = _build_block_index(dq, dk, max(1, _rows_pad(n) // vs))[0, h].cpu().numpy()
                mask = R.block_sparse_mask_rows(bidx, n, rbs)
            ref_scores.append(float((p * torch.from_numpy(mask[r0:n]).float()).sum(-1).mean()))
        got = [c[3][h] for c in table]
        assert np.allclose(got, ref_scores, atol=2e-2), (got, ref_scores)
        # selection: first candidate with the best score; the reference's renaming rules applied
        i_best = int(np.argmax(got))
        ty, vs, ss = CANDIDATES[i_best]
        if ty == "stream_llm":
            ty = "vertical_and_slash"
        if ty == "block_sparse":
            ty, vs, ss = "vertical_and_slash", 1000, 6096
        assert best[h][:3] == (ty, vs, ss) and abs(best[h][3] - max(got)) < 1e-6


def test_is_search_records_one_layer_per_call_and_runs_dense(tmp_path):
    import json

    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 2600, 2, 1
    q, k, v = (t.cuda() for t in make_qkv(n, hq, hkv, seed=12, dtype=torch.bfloat16))
    path = str(tmp_path / "pattern.json")
    cfg = {"is_search": True, "config_path": path, "starting_layer": 0}
    outs = []
    for layer in range(2):
        outs.append(minference_prefill_forward(q, k, v, {"attn_forward_config": cfg, "layer_idx": layer,
                                                         "num_hidden_layers": 2, "attention_mask": None}))
    table = json.load(open(path))
    assert len(table) == 2 and set(table[0]) == {"0", "1"}
    assert all(e[0] == "vertical_and_slash" and 0.0 < e[3] <= 1.0 for e in table[0].values())
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(2, 1),
                                                           v.float().repeat_interleave(2, 1), is_causal=True)
    assert (outs[0].float() - ref).abs().max().item() < 2e-2
    with pytest.raises(RuntimeError):
        minference_prefill_forward(q, k, v, {"attn_forward_config": cfg, "layer_idx": 0, "num_hidden_layers": 2,
                                             "attention_mask": None})
