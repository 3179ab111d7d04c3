"""The benchmark configurations at their exact layer shapes (32 query / 8 KV heads), the emulated 8-rank ring at
262144 tokens, and the device-side error reporting (status words) of the C ABI.

Full recomputation is out of reach at these sizes, so the checks are (a) sampled 64-row blocks of every head against
an fp32 masked-dense recomputation over the identical index set -- on the CPU oracle where it finishes in seconds,
with the same mathematics in torch on the device otherwise -- and (b) size-independent properties.
Tolerance for bf16 attention output: max-abs 2e-2, mean-abs 2e-3."""
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


def test_config0_8192_tokens_32_heads_against_cpu_oracle(dev):
    """8192 tokens, 32/8 heads, v=1000 / s=6096: estimator -> index conversion -> attention, checked per head
    against the CPU oracle: the estimator's lists through the set gate, the reference-format tables bit-exact
    against the C restatement, and sampled row blocks of every head against fp32 masked-dense attention."""
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.modules.minference_forward import minference_prefill_forward, vertical_slash_estimate
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R
    from tests.test_gpu_parity import _topk_gate

    n, hq, hkv = 8192, 32, 8
    q, k, v = make_qkv(n, hq, hkv, seed=0, dtype=torch.bfloat16)          # CPU generator: both sides see the same bits
    dq, dk, dv = q.to(dev), k.to(dev), v.to(dev)
    cfg = {"attn_forward_config": {"best_pattern": [{}]}, "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None}
    out = minference_prefill_forward(dq, dk, dv, cfg).float().cpu()     # default pattern: vertical-slash (1000, 6096) on every head
    v_idx, s_idx, nnz_v, nnz_s, vsc, ssc = vertical_slash_estimate(dq, dk, 1000, 6096, return_scores=True)
    assert nnz_v.tolist() == [1000] * hq and nnz_s.tolist() == [6096] * hq
    seqlens = torch.tensor([n], dtype=torch.int32, device=dev)
    bc, bo, cc, ci = (t.cpu().numpy() for t in convert_vertical_slash_indexes(seqlens, v_idx, s_idx, n))
    rbc, rbo, rcc, rci = R.convert_vertical_slash_indexes(np.array([n], np.int32), v_idx.cpu().numpy(), s_idx.cpu().numpy(), n)
    assert np.array_equal(bc, rbc) and np.array_equal(bo, rbo) and np.array_equal(cc, rcc) and np.array_equal(ci, rci)
    rows = n // 64
    rep = hq // hkv
    worst = 0.0
    for h in range(hq):
        if h % 4 == 0:      # the estimator gate on one head per KV group
            rv, rs, rvs, rss = R.vertical_slash_estimate(q[:, h:h + 1], k[:, h // rep:h // rep + 1], 1000, 6096, return_scores=True)
            ref_v, ref_s = rvs.float().numpy(), rss.float().flip(0).numpy()
            got_vs, got_ss = vsc[0, h].cpu().numpy(), ssc[0, h].cpu().numpy()
            fv, fs = np.isfinite(ref_v), np.isfinite(ref_s)
            nv, ns = float(np.abs(got_vs[fv] - ref_v[fv]).max()), float(np.abs(got_ss[fs] - ref_s[fs]).max())
            _topk_gate(set(v_idx[0, h].tolist()), ref_v, 1000, 2 * nv, (h, "vertical"))
            _topk_gate(set(s_idx[0, h].tolist()), ref_s, 6096, 2 * ns, (h, "slash"))
        kc, vc = k[0, h // rep].float(), v[0, h // rep].float()
        for m in sorted({0, 1, rows - 1, (h * 37 + 5) % rows}):
            mask = R.vs_mask_for_rows(bc[0, h], bo[0, h], cc[0, h], ci[0, h], n, [m])
            ref = R.masked_attention_rows(q[0, h, m * 64:m * 64 + 64].float(), kc, vc, mask, m * 64)
            d = (out[0, h, m * 64:m * 64 + 64] - ref).abs()
            worst = max(worst, d.max().item())
            assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (h, m, d.max().item())
    assert worst > 0.0


def test_config1_131072_tokens_32_heads_sampled_row_blocks(dev):
    """131072 tokens, 32/8 heads through the public per-layer operator; sampled row blocks of all 32 heads against the
    fp32 masked-dense recomputation on the device, three of them also against the CPU oracle."""
    from minference_b200.checks import compare_row_blocks, vertical_slash_row_block
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.modules.minference_forward import minference_prefill_forward, vertical_slash_estimate
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    n, hq, hkv = 131072, 32, 8
    q, k, v = make_qkv(n, hq, hkv, seed=0, dtype=torch.bfloat16, device=dev)
    cfg = {"attn_forward_config": {"best_pattern": [{}]}, "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None}
    out = minference_prefill_forward(q, k, v, cfg)
    v_idx, s_idx, _, _ = vertical_slash_estimate(q, k, 1000, 6096)          # the same kernels on the same input: same lists
    rows, rep = n // 64, hq // hkv
    seqlens = torch.tensor([n], dtype=torch.int32, device=dev)
    worst, means = 0.0, []
    for h in range(hq):
        bc, bo, cc, ci = convert_vertical_slash_indexes(seqlens, v_idx[:, h:h + 1].contiguous(), s_idx[:, h:h + 1].contiguous(), n)
        picks = sorted({0, 1, rows - 1, rows // 2 + h, (h * 211 + 9) % rows})
        mx, mean = compare_row_blocks(lambda m: out[0, h, 64 * m:64 * m + 64], lambda m: q[0, h, 64 * m:64 * m + 64],
                                      k[0, h // rep], v[0, h // rep], n, (bc[0, 0], bo[0, 0], cc[0, 0], ci[0, 0]), picks)
        worst = max(worst, mx)
        means.append(mean)
        assert mx < MAX_ABS and mean < MEAN_ABS, (h, mx, mean)
        if h in (0, 13, 31):        # the device recomputation itself against the CPU oracle
            m = picks[-2]
            tables = tuple(t[0, 0].cpu().numpy() for t in (bc, bo, cc, ci))
            mask = R.vs_mask_for_rows(*tables, n, [m])
            ref = R.masked_attention_rows(q[0, h, m * 64:m * 64 + 64].float().cpu(), k[0, h // rep].float().cpu(),
                                          v[0, h // rep].float().cpu(), mask, m * 64)
            dev_ref = vertical_slash_row_block(q[0, h, 64 * m:64 * m + 64], k[0, h // rep], v[0, h // rep], m, n,
                                               bc[0, 0, m], bo[0, 0, m], cc[0, 0, m], ci[0, 0, m]).cpu()
            assert (dev_ref - ref).abs().max().item() < 1e-4
            assert (out[0, h, m * 64:m * 64 + 64].float().cpu() - ref).abs().max().item() < MAX_ABS
        del bc, bo, cc, ci
    assert worst > 0.0


def test_emulated_8_rank_ring_262144_tokens_at_shard_boundaries(dev):
    """262144 tokens cut into 16 zigzag chunks as on 8 ranks, every visible (query chunk, key chunk) pair through the
    windowed C ABI with the fp32 carry (the ranks run one after the other on this GPU; no kernel waits on another).
    The first and last row blocks of every chunk -- the shard boundaries -- are compared with the fp32 masked-dense
    recomputation over the global index set, and the whole output with the single-launch kernel."""
    from minference_b200.checks import compare_row_blocks
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.dist import ring
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv
    from tests.test_gpu_ring import _one_rounding_apart, _pairs_through_carry

    n, hq, hkv, world = 262144, 4, 2, 8
    q, k, v = make_qkv(n, hq, hkv, seed=5, dtype=torch.bfloat16, device=dev)
    v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q, k, 1000, 6096)
    full = sparse_attention_forward(q, k, v, build_vertical_slash_plan(v_idx, s_idx, n, nnz_v, nnz_s))
    c = ring.chunk_size(n, world)
    merged = torch.empty_like(full)
    for qc in range(2 * world):
        plan, status = ring.build_plan_window(v_idx, s_idx, nnz_v, nnz_s, n, qc * c, c)
        merged[:, :, qc * c:(qc + 1) * c] = _pairs_through_carry(ring, q, k, v, n, c, qc, plan, v_idx, s_idx.shape[2], status, world)
        assert status.tolist()[:2] == [0, 0]
    assert torch.isfinite(merged.float()).all()
    assert _one_rounding_apart(merged, full)
    seqlens = torch.tensor([n], dtype=torch.int32, device=dev)
    per = c // 64
    for h in (0, hq - 1):
        bc, bo, cc, ci = convert_vertical_slash_indexes(seqlens, v_idx[:, h:h + 1].contiguous(), s_idx[:, h:h + 1].contiguous(), n)
        picks = sorted({ch * per + o for ch in range(2 * world) for o in (0, per - 1)} | {1, 7 * per + 3})
        mx, mean = compare_row_blocks(lambda m: merged[0, h, 64 * m:64 * m + 64], lambda m: q[0, h, 64 * m:64 * m + 64],
                                      k[0, h // 2], v[0, h // 2], n, (bc[0, 0], bo[0, 0], cc[0, 0], ci[0, 0]), picks)
        assert mx < MAX_ABS and mean < MEAN_ABS, (h, mx, mean)
        del bc, bo, cc, ci


def test_bad_plans_are_reported_not_followed(dev):
    """A head in plan mode without a plan, a zeroed plan and a plan of arbitrary bytes end as status bit 2 (or an
    empty result), never as a walk through memory the plan does not own."""
    from minference_b200 import _cabi
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 1024, 2, 1
    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=3, dtype=torch.bfloat16))
    L = _cabi.lib()
    out = torch.full_like(q, float("nan"))
    cap_v, cap_s = 64, 128

    def launch(plan, head_mode, v_idx):
        status = _cabi.new_status(dev)
        param = torch.zeros((hq, 2), dtype=torch.int32, device=dev)
        rc = L.minf_sparse_attention_fwd(
            _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(out), _cabi.strides3(q), _cabi.strides3(k), _cabi.strides3(v),
            _cabi.strides3(out), 1, hq, hkv, n, 128, 128 ** -0.5, _cabi.ptr(head_mode), _cabi.ptr(param), _cabi.ptr(plan),
            _cabi.ptr(v_idx), cap_v, cap_s, _cabi.ptr(status), _cabi.stream_ptr(dev))
        _cabi.check(rc)
        torch.cuda.synchronize()
        return status.tolist()

    modes = torch.tensor([_cabi.MODE_PLAN, _cabi.MODE_ASHAPE], dtype=torch.int32, device=dev)
    st = launch(None, modes, None)                       # plan-mode head, no plan
    assert st[0] & 4 and not st[0] & 1
    nbytes = L.minf_plan_bytes(1, hq, n, cap_v, cap_s)
    st = launch(torch.zeros(nbytes, dtype=torch.uint8, device=dev), None, None)        # zeroed plan: no ranges, no columns
    assert st[0] == 0 and torch.equal(out, torch.zeros_like(out))
    g = torch.Generator(device=dev).manual_seed(1)
    junk = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev, generator=g)
    st = launch(junk, None, None)                        # arbitrary bytes: counts beyond capacity, columns without a list
    assert st[0] & 4 and not st[0] & 1
    with pytest.raises(_cabi.MInferB200Error, match="bad plan"):
        status = torch.tensor(st, dtype=torch.int32)
        _cabi.raise_on_status(status, "test")


def test_device_wait_runs_out_and_reports(dev):
    """The bounded wait the kernels rely on: a barrier nobody arrives on is abandoned after the limit and the
    kernel comes back with status bit 0; the context stays usable."""
    from minference_b200 import _cabi

    L = _cabi.lib()
    status = _cabi.new_status(dev)
    _cabi.check(L.minf_selftest_bounded_wait(1000, _cabi.ptr(status), _cabi.stream_ptr(dev)))      # 1 ms
    torch.cuda.synchronize()
    assert status.tolist()[0] & 1
    with pytest.raises(_cabi.MInferB200Error, match="abandoned wait"):
        _cabi.raise_on_status(status, "selftest")
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0        # the device still answers
