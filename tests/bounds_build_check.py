"""Run in a child process with MINFER_B200_LIB pointing at the range-checked build (see tests/test_gpu_bounds_build.py):
tiny and ragged cases through estimator -> plan -> attention with NaN-filled outputs, compared with the CPU oracle;
the status words must stay clear (bit 3 would mean an index left its array)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from minference_b200 import _cabi
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    assert "bounds" in os.path.basename(_cabi.LIB_PATH), _cabi.LIB_PATH
    dev = torch.device("cuda:0")
    for n, hq, hkv, vs, ss in [(64, 2, 1, 30, 50), (65, 2, 2, 5, 7), (200, 2, 1, 64, 128), (1000, 4, 2, 100, 200), (1024, 2, 1, 1000, 1024),
                               (777, 3, 1, 300, 700)]:
        q, k, v = make_qkv(n, hq, hkv, seed=n, dtype=torch.bfloat16)
        dq, dk, dv = q.to(dev), k.to(dev), v.to(dev)
        v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(dq, dk, vs, ss)
        plan = build_vertical_slash_plan(v_idx, s_idx, n, nnz_v, nnz_s)
        out = torch.full_like(dq, float("nan"))                   # poison: a row nobody writes stays NaN
        sparse_attention_forward(dq, dk, dv, plan, out=out)
        tables = convert_vertical_slash_indexes(torch.tensor([n], dtype=torch.int32, device=dev), v_idx, s_idx, n)
        torch.cuda.synchronize()
        assert plan.status.tolist()[:2] == [0, 0], (n, plan.status.tolist())
        assert torch.isfinite(out.float()).all(), n
        ref, _ = R.vertical_slash_attention_oracle(q.float(), k.float(), v.float(), v_idx.cpu(), s_idx.cpu())
        d = (out.float().cpu() - ref[:, :, :n]).abs()
        assert d.max().item() < 2e-2 and d.mean().item() < 2e-3, (n, d.max().item())
        assert int(tables[0].max()) <= s_idx.shape[2] and int(tables[2].max()) <= v_idx.shape[2]
    # the plan from a block mask (FlexPrefill) through the same build: ragged length, the most runs a row can have
    from minference_b200.modules.flexprefill import build_block_mask_plan, flexprefill_forward

    for n, block in [(777, 128), (1000, 64), (2048 + 5, 128)]:
        nb = -(-n // block)
        mask = torch.eye(nb, dtype=torch.bool)
        mask[::2, ::2] = True
        mask = (mask & torch.tril(torch.ones(nb, nb, dtype=torch.bool)))[None, None].expand(1, 2, nb, nb).contiguous()
        q, k, v = make_qkv(n, 2, 1, seed=n + 3, dtype=torch.bfloat16)
        plan = build_block_mask_plan(mask.to(dev), n, block)
        out = torch.full((1, 2, n, 128), float("nan"), dtype=torch.bfloat16, device=dev)
        sparse_attention_forward(q.to(dev), k.to(dev), v.to(dev), plan, out=out)
        torch.cuda.synchronize()
        assert plan.status.tolist()[:2] == [0, 0], (n, plan.status.tolist())
        assert torch.isfinite(out.float()).all(), n
        ref, _ = R.flexprefill_attention_oracle(q, k, v, 0.9, block_size=block, block_mask=mask)
        d = (out.float().cpu() - ref[:, :, :n]).abs()
        assert d.max().item() < 2e-2 and d.mean().item() < 2e-3, (n, d.max().item())
    q, k, v = (t.to(dev) for t in make_qkv(1500, 4, 2, seed=9, dtype=torch.bfloat16))
    assert torch.isfinite(flexprefill_forward(q, k, v, {"attn_forward_config": {"gamma": 0.8, "tau": 0.1}}).float()).all()
    print("BOUNDS_OK")


if __name__ == "__main__":
    main()
