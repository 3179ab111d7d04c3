"""FlexPrefill on the CUDA path (modules/flexprefill.py of the reference): the plan built from a block set, the
adaptive block selection against the reference-executed fixtures and the CPU restatement, and the operator end to end
against fp32 masked-dense attention over the identical block set."""
import glob
import math
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS = 2e-2, 2e-3


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from minference_b200 import _cabi

    _cabi.lib()
    return torch.device("cuda:0")


def _random_block_mask(nb, heads, density, seed):
    g = torch.Generator().manual_seed(seed)
    m = torch.rand(1, heads, nb, nb, generator=g) < density
    m |= torch.eye(nb, dtype=torch.bool)            # a row always sees its own block
    m[:, 0] |= torch.ones(nb, nb, dtype=torch.bool)                 # head 0: dense causal (one run per row)
    if heads > 1:
        m[:, 1] = torch.eye(nb, dtype=torch.bool)                   # head 1: main block diagonal only
        m[:, 1, ::2, ::2] |= True                                   # ... plus every other block: the most runs possible
    return m & torch.tril(torch.ones(nb, nb, dtype=torch.bool))


@pytest.mark.parametrize("n,block,heads,kv_heads", [(1500, 128, 4, 2), (4096 + 37, 128, 3, 1), (1000, 64, 2, 2), (64 * 33, 64, 2, 1)])
def test_plan_from_a_block_set_attends_exactly_that_set(dev, n, block, heads, kv_heads):
    from minference_b200.modules.flexprefill import build_block_mask_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    nb = math.ceil(n / block)
    mask = _random_block_mask(nb, heads, 0.3, seed=n)
    q, k, v = make_qkv(n, heads, kv_heads, seed=n + 1, dtype=torch.bfloat16)
    plan = build_block_mask_plan(mask.to(dev), n, block)
    out = sparse_attention_forward(q.to(dev), k.to(dev), v.to(dev), plan).float().cpu()
    assert plan.status.tolist()[:2] == [0, 0]
    rows = (n + 63) // 64
    rbs = sorted({0, 1, rows // 2, rows - 2, rows - 1} | set(range(2, rows, max(rows // 6, 1))))
    want, _ = R.flexprefill_attention_oracle(q, k, v, 0.9, block_size=block, row_blocks=rbs, block_mask=mask)
    for i, m in enumerate(rbs):
        r0, r1 = m * 64, min(m * 64 + 64, n)
        d = (out[:, :, r0:r1] - want[:, :, i * 64:i * 64 + (r1 - r0)]).abs()
        assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (m, d.max().item())
    # the tiles of the plan are the tiles of the set: every selected block, cut at the causal edge of each 64-row block
    per = block // 64
    want_tiles = 0
    mm = mask[0].numpy()
    for h in range(heads):
        for m in range(rows):
            i = m // per
            for j in np.nonzero(mm[h, i, :i + 1])[0]:
                want_tiles += (min(j * block + block, 64 * (m + 1)) - j * block) // 64
    assert plan.count_tiles() == want_tiles


def test_plan_reports_more_runs_than_it_was_sized_for(dev):
    from minference_b200 import _cabi
    from minference_b200.ops.sparse_forward import SparsePlan

    n, block, nb = 2048, 128, 16
    mask = torch.eye(nb, dtype=torch.bool)
    mask[::2, ::2] = True
    mask = (mask & torch.tril(torch.ones(nb, nb, dtype=torch.bool)))[None, None].to(torch.uint8).to(dev).contiguous()
    L = _cabi.lib()
    cap_s = 2                                   # row 14 has 8 runs
    plan = SparsePlan(plan=torch.zeros(L.minf_plan_bytes(1, 1, n, 0, cap_s), dtype=torch.uint8, device=dev), v_idx=None,
                      cap_v=0, cap_s=cap_s, context_size=n, batch=1, heads=1, status=_cabi.new_status(dev))
    _cabi.check(L.minf_block_mask_build_plan(_cabi.ptr(mask), 1, 1, n, block, cap_s, _cabi.ptr(plan.plan),
                                             _cabi.ptr(plan.status), _cabi.stream_ptr(dev)))
    torch.cuda.synchronize()
    assert plan.status.tolist()[0] & 4
    assert L.minf_block_mask_build_plan(_cabi.ptr(mask), 1, 1, n, 96, cap_s, _cabi.ptr(plan.plan),
                                        _cabi.ptr(plan.status), _cabi.stream_ptr(dev)) != 0      # not a multiple of 64


def _chosen_blocks_gate(scores_ref, scores_got, budget, chosen_got, what):
    """Blocks whose pooled score is further from the budget's boundary than the measured difference between the two
    score vectors must be decided alike; the rest are near-ties."""
    nb = scores_ref.numel()
    budget = min(int(budget), nb)
    order = torch.argsort(scores_ref, descending=True)
    fin = torch.isfinite(scores_ref)
    noise = (scores_ref[fin] - scores_got[fin]).abs().max().item()
    kth = scores_ref[order[budget - 1]].item()
    nxt = scores_ref[order[budget]].item() if budget < nb else -math.inf
    margin = 2 * noise + 1e-6 * max(abs(kth), 1e-30)
    must_in = scores_ref > (nxt + margin if math.isfinite(nxt) else -math.inf)
    must_in &= torch.zeros_like(must_in).index_fill_(0, order[:budget], True)
    must_out = scores_ref < kth - margin
    assert chosen_got[must_in].all(), what
    assert not chosen_got[must_out].any(), what
    assert int(chosen_got.sum()) == budget, what
    return noise


def test_block_selection_against_reference_fixtures_and_restatement(dev, golden_dir):
    from minference_b200.modules.flexprefill import active_block_mask
    from oracle import reference_math as R
    from tests.test_oracle_flexprefill import fixture_case

    paths = sorted(glob.glob(os.path.join(golden_dir, "flexprefill_*.npz")))
    assert len(paths) >= 5
    exact = 0
    for path in paths:
        q, k, _, p, ref = fixture_case(path)
        _, det_ref = R.flex_active_block_mask(q, k, 128, p["gamma"], p["min_budget"], p["max_budget"], p["tau"], return_details=True)
        mask, det = active_block_mask(q.to(dev), k.to(dev), 128, p["gamma"], p["min_budget"], p["max_budget"], p["tau"],
                                      return_details=True)
        got = mask[0].cpu().numpy()
        name = os.path.basename(path)
        nb = ref.shape[-1]
        # budgets and the kind of each head: integers derived from sums over thousands of tokens
        assert torch.equal(det["block_sparse"].cpu(), det_ref["block_sparse"]), name
        assert (det["n_vertical"].cpu() - det_ref["n_vertical"]).abs().max().item() <= 1, name
        assert (det["n_slash"].cpu() - det_ref["n_slash"]).abs().max().item() <= 1, name
        js_gap = (det["js"].cpu() - det_ref["js"]).abs().max().item()
        assert js_gap < 2e-3, (name, js_gap)
        same_budgets = torch.equal(det["n_vertical"].cpu(), det_ref["n_vertical"]) and torch.equal(det["n_slash"].cpu(), det_ref["n_slash"])
        sym = int((got != ref).sum())
        print(f"{name}: blocks {int(ref.sum())}, differing {sym}, budgets equal {same_budgets}, sqrt-JS gap {js_gap:.2e}")
        if same_budgets and not bool(det_ref["block_sparse"].any()):
            # vertical-slash heads: gate the two selections on the pooled scores, then the set follows from them
            tril = np.tril(np.ones((nb, nb), dtype=bool))
            for h in range(ref.shape[0]):
                _chosen_blocks_gate(det_ref["vertical_pooled"][0, h], det["vertical_pooled"][0, h].cpu(),
                                    det_ref["n_vertical"][0, h], _choice(det, "vertical", h), f"{name} head {h} vertical")
                _chosen_blocks_gate(det_ref["slash_pooled"][0, h], det["slash_pooled"][0, h].cpu(),
                                    det_ref["n_slash"][0, h], _choice(det, "slash", h), f"{name} head {h} slash")
                # the set follows from the two choices: chosen key blocks below the diagonal, chosen block diagonals
                sel_v, sel_s = _choice(det, "vertical", h).numpy(), _choice(det, "slash", h).numpy()
                want = np.zeros((nb, nb), dtype=bool)
                want[:, sel_v] = True
                for b_ in np.nonzero(sel_s)[0]:
                    d_ = nb - 1 - b_
                    want[np.arange(d_, nb), np.arange(0, nb - d_)] = True
                assert np.array_equal(got[h], want & tril), (name, h)
        assert sym <= max(2, int(0.03 * ref.sum())), (name, sym)
        exact += sym == 0
    assert exact >= 3          # most cases have no near-tie at all and reproduce the reference's set bit for bit


def _choice(det, which, h):
    """The blocks the product takes for one head: the best ``n`` pooled scores (``which``: vertical or slash)."""
    s, n = det[which + "_pooled"][0, h], int(det["n_" + which][0, h])
    sel = torch.zeros(s.numel(), dtype=torch.bool)
    sel[s.topk(min(n, s.numel())).indices.cpu()] = True
    return sel


@pytest.mark.parametrize("n,heads,kv_heads,cfg", [
    (4096 + 100, 4, 2, {"gamma": 0.9, "tau": 0.1}),
    (8192, 4, 1, {"gamma": 0.6, "tau": 0.0, "min_budget": 256, "max_budget": 1024}),
    (3000, 2, 2, {"gamma": 0.9, "tau": 0.1, "block_size": 64}),
])
def test_operator_against_masked_dense_over_its_own_block_set(dev, n, heads, kv_heads, cfg):
    from minference_b200.modules.flexprefill import active_block_mask, flexprefill_forward
    from minference_b200.patch import prefill_forwards
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    assert prefill_forwards["flexprefill"] is flexprefill_forward
    q, k, v = make_qkv(n, heads, kv_heads, seed=n, dtype=torch.bfloat16, plant=(n != 8192))
    dq, dk, dv = q.to(dev), k.to(dev), v.to(dev)
    out = flexprefill_forward(dq, dk, dv, {"attn_forward_config": cfg}).float().cpu()
    bs = cfg.get("block_size", 128)
    mask = active_block_mask(dq, dk, bs, cfg["gamma"], math.ceil(cfg.get("min_budget", 1) / bs),
                             math.ceil(cfg.get("max_budget", 2147483647) / bs), cfg["tau"]).cpu()
    nb = mask.shape[-1]
    print(f"n={n}: {int(mask.sum())} of {heads * nb * (nb + 1) // 2} causal blocks selected")
    rows = (n + 63) // 64
    rbs = sorted({0, 1, rows // 3, rows // 2, rows - 2, rows - 1})
    want, _ = R.flexprefill_attention_oracle(q, k, v, cfg["gamma"], block_size=bs, row_blocks=rbs, block_mask=mask)
    for i, m in enumerate(rbs):
        r0, r1 = m * 64, min(m * 64 + 64, n)
        d = (out[:, :, r0:r1] - want[:, :, i * 64:i * 64 + (r1 - r0)]).abs()
        assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (m, d.max().item())


def test_short_sequences_are_dense_and_the_bnhd_entry_point_matches(dev):
    from minference_b200.modules.flexprefill import flex_prefill_attention, flexprefill_forward
    from minference_b200.synthetic import make_qkv

    q, k, v = (t.to(dev) for t in make_qkv(256, 2, 1, seed=5, dtype=torch.bfloat16))
    out = flexprefill_forward(q, k, v, {"attn_forward_config": {}})
    want = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(2, 1),
                                                            v.float().repeat_interleave(2, 1), is_causal=True)
    assert (out.float() - want).abs().max().item() < MAX_ABS
    q, k, v = (t.to(dev) for t in make_qkv(2048, 2, 1, seed=6, dtype=torch.bfloat16))
    a = flexprefill_forward(q, k, v, {"attn_forward_config": {"gamma": 0.8, "tau": 0.0}})
    b = flex_prefill_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), 0.8, 0.0)
    assert b.shape == (1, 2048, 2, 128) and torch.equal(a, b.transpose(1, 2))
    with pytest.raises(Exception):
        flexprefill_forward(q, k, v, {"attn_forward_config": {"block_size": 32}})


def test_batch_of_two_sequences(dev):
    """Two sequences in one call: block sets and outputs equal the per-sequence calls."""
    from minference_b200.modules.flexprefill import active_block_mask, flexprefill_forward
    from minference_b200.synthetic import make_qkv

    n = 2048 + 64
    a = [t.to(dev) for t in make_qkv(n, 4, 2, seed=61, dtype=torch.bfloat16)]
    b = [t.to(dev) for t in make_qkv(n, 4, 2, seed=62, dtype=torch.bfloat16, plant=False)]
    both = [torch.cat((x, y), dim=0) for x, y in zip(a, b)]
    cfg = {"attn_forward_config": {"gamma": 0.7, "tau": 0.0, "max_budget": 512}}
    out = flexprefill_forward(*both, cfg)
    m_both = active_block_mask(both[0], both[1], 128, 0.7, 1, 4, 0.0)
    for i, one in enumerate((a, b)):
        assert torch.equal(m_both[i], active_block_mask(one[0], one[1], 128, 0.7, 1, 4, 0.0)[0])
        assert torch.equal(out[i], flexprefill_forward(*one, cfg)[0])


@pytest.mark.parametrize("n,heads,kv_heads", [(2048, 4, 2), (4096 + 100, 2, 1), (1500, 4, 4)])
def test_attention_over_a_block_set_matches_reference_triton_kernel_on_gpu(dev, n, heads, kv_heads):
    """The reference's own block-wise prefill kernel (modules/flexprefill.py:352-495, compiled ahead of time for
    sm_100a by oracle/build_ref.py) and this library's kernel on the same inputs and the same block set: a random one
    and the one the adaptive selection returns."""
    from minference_b200.modules.flexprefill import active_block_mask, build_block_mask_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv
    from oracle import ref_triton

    if not ref_triton.available(ref_triton.CUBIN_FLEX):
        pytest.skip("the reference kernel binary is not built (oracle/build_ref.py --triton)")
    kernel = ref_triton.ReferenceTritonKernel(ref_triton.CUBIN_FLEX)
    q, k, v = (t.to(dev) for t in make_qkv(n, heads, kv_heads, seed=n + 7, dtype=torch.bfloat16))
    nb = math.ceil(n / 128)
    masks = [_random_block_mask(nb, heads, 0.3, seed=n + 2).to(dev),
             active_block_mask(q, k, 128, 0.8, 1, 8, 0.0)]
    for mask in masks:
        plan = build_block_mask_plan(mask, n, 128)
        got = sparse_attention_forward(q, k, v, plan).float()
        want = ref_triton.reference_flex_block_attention(kernel, q, k, v, mask).float()
        d = (got - want).abs()
        assert plan.status.tolist()[:2] == [0, 0]
        assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (n, d.max().item(), d.mean().item())


def test_reference_block_wise_kernel_timing_131072(dev, capsys):
    """131072 tokens, 8 query / 2 KV heads, the block set of the adaptive selection with budgets of 64 blocks: the
    reference's block-wise kernel and this library's kernel on the same inputs, CUDA-event times of the launches alone
    (run with -s to see them)."""
    from minference_b200.modules.flexprefill import active_block_mask, build_block_mask_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv
    from oracle import ref_triton

    if not ref_triton.available(ref_triton.CUBIN_FLEX):
        pytest.skip("the reference kernel binary is not built (oracle/build_ref.py --triton)")
    n, hq, hkv = 131072, 8, 2
    q, k, v = make_qkv(n, hq, hkv, seed=0, dtype=torch.bfloat16, device=dev)
    mask = active_block_mask(q, k, 128, 0.9, 1, 64, 0.0)
    plan = build_block_mask_plan(mask, n, 128)
    # the build specialised for exactly these sizes (what the JIT does: unit strides folded, divisibility hints)
    kernel = ref_triton.ReferenceTritonKernel(ref_triton.CUBIN_FLEX_128K_8HEADS if ref_triton.available(ref_triton.CUBIN_FLEX_128K_8HEADS)
                                              else ref_triton.CUBIN_FLEX)
    launch, ref_out, keep = ref_triton.reference_flex_block_attention(kernel, q, k, v, mask, prepared_call=True)

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out

    t_ref, _ = timed(launch)
    t_new, out = timed(lambda: sparse_attention_forward(q, k, v, plan))
    tiles = plan.count_tiles()
    d = (out.float() - ref_out.float()).abs()
    with capsys.disabled():
        print(f"\n131072 tokens, {hq}/{hkv} heads, {int(mask.sum())} blocks of 128 ({tiles} 64x64 tiles): reference block-wise "
              f"kernel {t_ref:.1f} ms ({tiles * 2097152 / t_ref / 1e9:.0f} TFLOP/s), product kernel {t_new:.1f} ms "
              f"({tiles * 2097152 / t_new / 1e9:.0f} TFLOP/s), ratio {t_ref / t_new:.2f}; max-abs difference {d.max().item():.2e}")
    del keep
    assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS
    assert t_new < t_ref
