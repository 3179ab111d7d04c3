"""GPU parity tests: every call goes through the C ABI (ctypes) and is compared with the CPU
oracle on the same seeded inputs.  Tolerances for bf16 attention output: max-abs 2e-2,
mean-abs 2e-3 against an fp32 masked-dense recomputation over the identical index set;
index tensors bit-exact."""
import glob
import json
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


def _close(out, ref, what):
    d = (out.float().cpu() - ref.float()).abs()
    assert torch.isfinite(out.float()).all(), what
    assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (what, d.max().item(), d.mean().item())


# ------------------------------------------------------------------ index conversion

def test_convert_matches_reference_fixtures(dev, golden_dir):
    from minference_b200.cuda import convert_vertical_slash_indexes

    for path in sorted(glob.glob(os.path.join(golden_dir, "vs_index_*.npz"))):
        z = np.load(path)
        n = int(z["n"])
        outs = convert_vertical_slash_indexes(torch.tensor([n], dtype=torch.int32, device=dev),
                                              torch.from_numpy(z["v"]).to(dev), torch.from_numpy(z["s"]).to(dev), n)
        for name, got in zip(("block_count", "block_offset", "column_count", "column_index"), outs):
            assert np.array_equal(got.cpu().numpy(), z[name]), (path, name)


def test_convert_matches_reference_digests(dev, golden_dir):
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from tests.golden.make_golden import INDEX_DIGEST, digest, index_case

    digests = json.load(open(os.path.join(golden_dir, "digests.json")))
    for (seed, n, heads, nv, ns, style) in INDEX_DIGEST:
        v, s = index_case(seed, n, heads, nv, ns, style)
        tv, ts = torch.from_numpy(v).to(dev), torch.from_numpy(s).to(dev)
        outs = convert_vertical_slash_indexes(torch.tensor([n], dtype=torch.int32, device=dev), tv, ts, n)
        assert digest([o.cpu().numpy() for o in outs]) == digests[f"vs_index_{seed}"]["sha256"], seed
        # the compact plan holds the same index set: same number of reference tiles
        plan = build_vertical_slash_plan(tv, ts, n)
        assert plan.count_tiles() == digests[f"vs_index_{seed}"]["tiles"], seed
        assert plan.status.tolist()[:2] == [0, 0]


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(__file__), "..", "oracle", "_ref", "minference_ref_cuda.so")),
                    reason="reference CUDA extension not built")
def test_convert_matches_reference_extension_on_gpu(dev):
    """Bit-exact against the reference's own extension running on the same GPU."""
    from minference_b200.cuda import convert_vertical_slash_indexes
    from tests.golden.make_golden import index_case

    import importlib.util      # the reference builds a plain pybind module: import it by file path
    spec = importlib.util.spec_from_file_location(
        "minference_ref_cuda", os.path.join(os.path.dirname(__file__), "..", "oracle", "_ref", "minference_ref_cuda.so"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for seed, (n, heads, nv, ns, style) in enumerate([(8192, 2, 1000, 6096, "uniform"), (5000, 3, 77, 333, "clustered"),
                                                      (131072, 1, 1000, 6096, "uniform")]):
        v, s = index_case(50 + seed, n, heads, nv, ns, style)
        tv, ts = torch.from_numpy(v).to(dev), torch.from_numpy(s).to(dev)
        sl = torch.tensor([n], dtype=torch.int32, device=dev)
        ref = mod.convert_vertical_slash_indexes(sl, tv, ts, n, 64, 64)
        torch.cuda.synchronize()
        got = convert_vertical_slash_indexes(sl, tv, ts, n)
        for a, b in zip(got, ref):
            assert torch.equal(a, b), (seed,)


def test_convert_ragged_and_edge_cases(dev):
    from minference_b200 import _cabi
    from minference_b200.cuda import convert_vertical_slash_indexes
    from oracle import reference_math as R

    # single entries, context not a multiple of 64, duplicates, all offsets clamped
    cases = [
        (65, [[0]], [[0]]),
        (64, [[63]], [[63]]),
        (1000, [[0, 0, 5, 999]], [[900, 63, 63, 0]]),
        (700, [[10, 20, 650]], [[699, 640, 639, 1]]),
    ]
    for n, v, s in cases:
        v = np.array([v], np.int32)
        s = np.array([s], np.int32)
        ref = R.convert_vertical_slash_indexes(np.array([n], np.int32), v, s, n)
        got = convert_vertical_slash_indexes(torch.tensor([n], dtype=torch.int32, device=dev),
                                             torch.from_numpy(v).to(dev), torch.from_numpy(s).to(dev), n)
        for a, b in zip(got, ref):
            assert np.array_equal(a.cpu().numpy(), b), (n,)
    # seqlen shorter than the context: rows past seqlen stay zero like the reference's zero-filled outputs
    n = 1024
    v = np.array([[[1, 100, 500]]], np.int32)
    s = np.array([[[300, 70, 3]]], np.int32)
    ref = R.convert_vertical_slash_indexes(np.array([600], np.int32), v, s, n)
    got = convert_vertical_slash_indexes(torch.tensor([600], dtype=torch.int32, device=dev),
                                         torch.from_numpy(v).to(dev), torch.from_numpy(s).to(dev), n)
    for a, b in zip(got, ref):
        assert np.array_equal(a.cpu().numpy(), b)
    # no offset below 64: reported, not read out of bounds
    with pytest.raises(_cabi.MInferB200Error):
        convert_vertical_slash_indexes(torch.tensor([1024], dtype=torch.int32, device=dev),
                                       torch.tensor([[[0, 5]]], dtype=torch.int32, device=dev),
                                       torch.tensor([[[500, 200]]], dtype=torch.int32, device=dev), 1024)


# ------------------------------------------------------------------ estimator

def _topk_gate(got: set, ref_scores: np.ndarray, k: int, noise_abs: float, what, rel: float = 1e-6):
    """The gate for top-k index sets: every entry whose reference score lies further from the
    k-th / (k+1)-th boundary than 1e-6 relative plus the measured score noise of the kernel must be
    decided the same way; the remaining near-ties are reported as recall.  ``ref_scores`` holds +inf
    at forced entries.  Returns (decided entries, near-tie entries, recall over the near-ties)."""
    n = ref_scores.shape[0]
    order = np.sort(ref_scores)[::-1]
    kth = order[k - 1]
    nxt = order[k] if k < n else -np.inf
    must_have = set(np.nonzero(ref_scores > kth * (1 + rel) + noise_abs)[0].tolist())
    must_not = set(np.nonzero(ref_scores < nxt * (1 - rel) - noise_abs)[0].tolist()) if k < n else set()
    assert must_have <= got, (what, "missing decided entries", sorted(must_have - got)[:8], kth, noise_abs)
    assert not (got & must_not), (what, "took entries decidedly below the boundary", sorted(got & must_not)[:8], nxt, noise_abs)
    ties = set(range(n)) - must_have - must_not
    want_ties = k - len(must_have)
    ref_top = set(np.argsort(-ref_scores, kind="stable")[:k].tolist())
    recall = len(got & ref_top & ties) / max(want_ties, 1)
    return len(must_have) + len(must_not), len(ties), recall


def test_estimator_matches_reference_fixtures(dev, golden_dir):
    """fp32 fixtures (the reference's functions executed on fp16-exact data in fp32): the kernel sees the bf16
    rounding of those inputs, so only overlap can be asked for."""
    from minference_b200.modules.minference_forward import vertical_slash_estimate

    for path in sorted(glob.glob(os.path.join(golden_dir, "estimator_[0-9]*.npz"))):
        z = np.load(path)
        n = int(z["n"])
        k = torch.from_numpy(z["k"]).to(torch.bfloat16)
        q_last = torch.from_numpy(z["q_last"]).to(torch.bfloat16)
        q = torch.zeros(1, 1, n, 128, dtype=torch.bfloat16)
        q[0, 0, -64:] = q_last
        v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q.to(dev), k[None, None].to(dev),
                                                             int(z["vertical_size"]), int(z["slash_size"]))
        want_v, want_s = set(z["v_idx"].flatten().tolist()), set(z["s_idx"].flatten().tolist())
        got_v = set(v_idx[0, 0, : int(nnz_v[0])].tolist())
        got_s = set(s_idx[0, 0, : int(nnz_s[0])].tolist())
        assert len(got_v) == len(want_v) and len(got_s) == len(want_s)
        assert len(got_v & want_v) >= 0.9 * len(want_v), path
        assert len(got_s & want_s) >= 0.9 * len(want_s), path
        assert set(range(min(30, n))) <= got_v and set(range(min(100, len(want_s)))) <= got_s


def test_estimator_matches_reference_run_in_bf16(dev, golden_dir, capsys):
    """bf16 fixtures: the reference's own function bodies executed on the very bf16 tensors the kernel gets, with the
    score vectors they hand to torch.topk recorded.  Scores must agree to rounding noise and the selected sets must
    be equal wherever the boundary gap exceeds 1e-6 relative plus that noise."""
    from minference_b200.modules.minference_forward import vertical_slash_estimate

    paths = sorted(glob.glob(os.path.join(golden_dir, "estimator_bf16_*.npz")))
    assert len(paths) >= 4
    for path in paths:
        z = np.load(path)
        n, vs, ss = int(z["n"]), int(z["vertical_size"]), int(z["slash_size"])
        k = torch.from_numpy(z["k_bits"]).view(torch.bfloat16)
        q = torch.zeros(1, 1, n, 128, dtype=torch.bfloat16)
        q[0, 0, -64:] = torch.from_numpy(z["q_last_bits"]).view(torch.bfloat16)
        v_idx, s_idx, nnz_v, nnz_s, vsc, ssc = vertical_slash_estimate(q.to(dev), k[None, None].to(dev), vs, ss, return_scores=True)
        kv, ks = int(nnz_v[0]), int(nnz_s[0])
        assert kv == z["v_idx"].size and ks == z["s_idx"].size
        ref_v, ref_s = z["vertical_scores"].copy(), z["slash_scores_by_offset"].copy()      # +inf at forced entries
        got_vs, got_ss = vsc[0, 0].cpu().numpy(), ssc[0, 0].cpu().numpy()
        fin_v, fin_s = np.isfinite(ref_v), np.isfinite(ref_s)
        noise_v = float(np.abs(got_vs[fin_v] - ref_v[fin_v]).max()) if fin_v.any() else 0.0
        noise_s = float(np.abs(got_ss[fin_s] - ref_s[fin_s]).max()) if fin_s.any() else 0.0
        # a bf16 logit that rounds the other way moves one of 64 probabilities by under 1 %
        assert noise_v <= 2e-3 * ref_v[fin_v].max() + 1e-7 and noise_s <= 2e-3 * ref_s[fin_s].max() + 1e-7, (path, noise_v, noise_s)
        dv = _topk_gate(set(v_idx[0, 0, :kv].tolist()), ref_v, kv, 2 * noise_v, (path, "vertical"))
        ds = _topk_gate(set(s_idx[0, 0, :ks].tolist()), ref_s, ks, 2 * noise_s, (path, "slash"))
        with capsys.disabled():
            print(f"\n{os.path.basename(path)}: score noise v {noise_v:.2e} s {noise_s:.2e}; vertical decided {dv[0]} near-ties {dv[1]} "
                  f"recall {dv[2]:.3f}; slash decided {ds[0]} near-ties {ds[1]} recall {ds[2]:.3f}")
        # the lists of the reference itself, as sets, on the decided part is what the gate checked; overall overlap stays high
        assert len(set(v_idx[0, 0, :kv].tolist()) & set(z["v_idx"].flatten().tolist())) >= 0.97 * kv
        assert len(set(s_idx[0, 0, :ks].tolist()) & set(z["s_idx"].flatten().tolist())) >= 0.97 * ks


@pytest.mark.parametrize("n,hq,hkv,vs,ss", [(600, 4, 2, 100, 200), (2048, 3, 1, 300, 700), (50, 2, 2, 30, 50),
                                            (8192, 4, 2, 1000, 6096)])
def test_estimator_matches_oracle_on_same_bf16_inputs(dev, n, hq, hkv, vs, ss):
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    q, k, _ = make_qkv(n, hq, hkv, seed=4, dtype=torch.bfloat16)
    v_idx, s_idx, nnz_v, nnz_s, vsc, ssc = vertical_slash_estimate(q.to(dev), k.to(dev), vs, ss, return_scores=True)
    rep = hq // hkv
    for h in range(hq):
        rv, rs, rvs, rss = R.vertical_slash_estimate(q[:, h:h + 1], k[:, h // rep:h // rep + 1], vs, ss, return_scores=True)
        got_v = v_idx[0, h, : int(nnz_v[h])]
        got_s = s_idx[0, h, : int(nnz_s[h])]
        assert int(nnz_v[h]) == rv.numel() and int(nnz_s[h]) == rs.numel()
        assert bool((got_v.diff() > 0).all()) and bool((got_s.diff() < 0).all())     # sorted for the index conversion
        # scores agree to rounding noise of the bf16 logits
        ref_v, ref_s = rvs.float().numpy().copy(), rss.float().flip(0).numpy().copy()    # slash by diagonal offset; +inf where forced
        got_vs, got_ss = vsc[0, h].cpu().numpy(), ssc[0, h].cpu().numpy()
        fin_v, fin_s = np.isfinite(ref_v), np.isfinite(ref_s)
        noise_v = float(np.abs(got_vs[fin_v] - ref_v[fin_v]).max()) if fin_v.any() else 0.0
        noise_s = float(np.abs(got_ss[fin_s] - ref_s[fin_s]).max()) if fin_s.any() else 0.0
        assert noise_v < 1e-3 * max(ref_v[fin_v].max() if fin_v.any() else 0.0, 1e-6) + 1e-6
        assert noise_s < 1e-3 * max(ref_s[fin_s].max() if fin_s.any() else 0.0, 1e-6) + 1e-6
        # set equality wherever the boundary gap exceeds 1e-6 relative plus the measured noise
        _topk_gate(set(got_v.tolist()), ref_v, rv.numel(), 2 * noise_v, (n, h, "vertical"))
        _topk_gate(set(got_s.tolist()), ref_s, rs.numel(), 2 * noise_s, (n, h, "slash"))
        want_v, want_s = set(rv.flatten().tolist()), set(rs.flatten().tolist())
        assert len(set(got_v.tolist()) & want_v) >= 0.99 * len(want_v)
        assert len(set(got_s.tolist()) & want_s) >= 0.99 * len(want_s)


# ------------------------------------------------------------------ attention

@pytest.mark.parametrize("n,hq,hkv,nv,ns,kind", [
    (64, 2, 1, 5, 9, "rand"), (100, 2, 2, 7, 9, "rand"), (1000, 4, 2, 50, 80, "rand"),
    (1024, 4, 2, 30, 100, "local"), (4096, 4, 2, 100, 300, "rand"), (4133, 2, 1, 300, 300, "rand"),
    (8192, 4, 2, 1000, 6096, "rand"),
])
def test_vertical_slash_attention_matches_oracle(dev, n, hq, hkv, nv, ns, kind):
    from minference_b200.ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention
    from minference_b200.synthetic import local_vs_indices, make_qkv
    from oracle import reference_math as R
    from tests.golden.make_golden import index_case

    q, k, v = make_qkv(n, hq, hkv, seed=2, dtype=torch.bfloat16)
    if kind == "local":
        vi, si = local_vs_indices(n, hq, nv, ns, seed=3)
    else:
        a, b = index_case(7, n, hq, min(nv, n), min(ns, n), "uniform")
        vi, si = torch.from_numpy(a), torch.from_numpy(b)
    # unsorted int64 indices like the estimator of the reference produces: the operator sorts
    perm_v = torch.randperm(vi.shape[-1])
    out = vertical_slash_sparse_attention(q.to(dev), k.to(dev), v.to(dev), vi[..., perm_v].long().to(dev), si.long().to(dev))
    ref, _ = R.vertical_slash_attention_oracle(q.float(), k.float(), v.float(), vi, si)
    _close(out, ref[:, :, :n], (n, kind))


@pytest.mark.parametrize("n,hq,hkv,nv,ns,kind", [(2048, 4, 2, 120, 260, "uniform"), (1000, 2, 2, 64, 300, "local"),
                                                 (4096, 4, 1, 1000, 3000, "estimated")])
def test_attention_matches_reference_triton_kernel_on_gpu(dev, n, hq, hkv, nv, ns, kind):
    """The reference's own attention kernel (compiled ahead of time from the reference tree by
    oracle/build_ref.py --triton) and the product kernel on the same inputs and index tensors."""
    from oracle import ref_triton

    if not ref_triton.available():
        pytest.skip("the reference's Triton kernel was not compiled (oracle/_ref/ref_triton_vs_fwd.cubin)")
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention
    from minference_b200.synthetic import local_vs_indices, make_qkv
    from oracle import reference_math as R
    from tests.golden.make_golden import index_case

    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=31, dtype=torch.bfloat16))
    if kind == "local":
        vi, si = local_vs_indices(n, hq, nv, ns, seed=6)
    elif kind == "uniform":
        a, b = index_case(5, n, hq, nv, ns, "uniform")
        b[..., -1] = 0
        vi, si = torch.from_numpy(a), torch.from_numpy(b)
    else:
        vi, si, _, _ = vertical_slash_estimate(q, k, nv, ns)
    vs, ss = R.presort_indices(vi.cpu(), si.cpu(), 1, hq)
    vs, ss = vs.contiguous().to(dev), ss.contiguous().to(dev)
    bc, bo, cc, ci = convert_vertical_slash_indexes(torch.tensor([n], dtype=torch.int32, device=dev), vs, ss, n)
    ref = ref_triton.reference_vertical_slash_attention(ref_triton.ReferenceTritonKernel(), q, k, v, bc, bo, cc, ci).float()
    out = vertical_slash_sparse_attention(q, k, v, vs, ss).float()
    torch.cuda.synchronize()
    d = (out - ref).abs()
    assert torch.isfinite(ref).all() and ref.abs().max().item() > 0.1
    assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (d.max().item(), d.mean().item())


@pytest.mark.parametrize("n,hq,hkv,top_k", [(2048, 4, 2, 8), (1000, 2, 1, 5), (4096, 2, 2, 100)])
def test_block_sparse_matches_reference_triton_kernel_on_gpu(dev, n, hq, hkv, top_k):
    """The reference's block-sparse kernel (ahead-of-time build) on the block index of the product planner."""
    from oracle import ref_triton

    if not ref_triton.available(ref_triton.CUBIN_BLOCK_SPARSE):
        pytest.skip("the reference's block-sparse Triton kernel was not compiled (oracle/_ref/ref_triton_bs_fwd.cubin)")
    from minference_b200.ops.block_sparse_flash_attention import _build_block_index, block_sparse_attention
    from minference_b200.synthetic import make_qkv

    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=32, dtype=torch.bfloat16))
    bidx = _build_block_index(q, k, top_k)
    ref = ref_triton.reference_block_sparse_attention(ref_triton.ReferenceTritonKernel(ref_triton.CUBIN_BLOCK_SPARSE),
                                                      q, k, v, bidx).float()
    out = block_sparse_attention(q, k, v, top_k).float()
    torch.cuda.synchronize()
    d = (out - ref).abs()
    assert torch.isfinite(ref).all() and ref.abs().max().item() > 0.1
    assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (d.max().item(), d.mean().item())


@pytest.mark.parametrize("n,n_init,n_local", [(2048, 128, 512), (1000, 64, 200), (1024, 128, 4096), (3000, 128, 1000)])
def test_streaming_matches_reference_triton_kernel_on_gpu(dev, n, n_init, n_local):
    """The reference's streaming (A-shape) kernel, both of its stages, against the one-pass product kernel."""
    from oracle import ref_triton

    if not ref_triton.streaming_available():
        pytest.skip("the reference's streaming Triton kernel was not compiled (oracle/_ref/ref_triton_stream_*.cubin)")
    from minference_b200.ops.streaming_kernel import streaming_forward
    from minference_b200.synthetic import make_qkv

    q, k, v = (t.to(dev) for t in make_qkv(n, 4, 2, seed=33, dtype=torch.bfloat16))
    ref = ref_triton.reference_streaming_forward(q, k, v, n_init, n_local).float()
    out = streaming_forward(q, k, v, n_init, n_local).float()
    torch.cuda.synchronize()
    d = (out - ref).abs()
    assert torch.isfinite(ref).all() and ref.abs().max().item() > 0.1
    assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (d.max().item(), d.mean().item())


def test_reference_triton_kernel_timing_131072(dev, capsys):
    """Same 131072-token vertical-slash inputs (8 query / 2 KV heads) through the reference's own Triton
    kernel and the product kernel: outputs agree, and the CUDA-event times of both are printed
    (run with -s to see them; the reference kernel gets K/V already repeated and its dense index tables)."""
    from oracle import ref_triton

    if not ref_triton.available():
        pytest.skip("the reference's Triton kernel was not compiled (oracle/_ref/ref_triton_vs_fwd.cubin)")
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 131072, 8, 2
    q, k, v = make_qkv(n, hq, hkv, seed=0, dtype=torch.bfloat16, device=dev)
    v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q, k, 1000, 6096)
    plan = build_vertical_slash_plan(v_idx, s_idx, n, nnz_v, nnz_s)
    bc, bo, cc, ci = convert_vertical_slash_indexes(torch.tensor([n], dtype=torch.int32, device=dev), v_idx, s_idx, n)
    # the build specialised for exactly these sizes (what the JIT does: unit strides folded, divisibility hints)
    kernel = ref_triton.ReferenceTritonKernel(ref_triton.CUBIN_128K_8HEADS if ref_triton.available(ref_triton.CUBIN_128K_8HEADS)
                                              else ref_triton.CUBIN)
    kr, vr = k.repeat_interleave(hq // hkv, 1).contiguous(), v.repeat_interleave(hq // hkv, 1).contiguous()
    seqlens = torch.tensor([n], dtype=torch.int32, device=dev)

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out

    t_ref, ref = timed(lambda: kernel(q, kr, vr, seqlens, bc, bo, cc, ci, 128 ** -0.5))
    t_new, out = timed(lambda: sparse_attention_forward(q, k, v, plan))
    tiles = plan.count_tiles()
    d = (out.float() - ref.float()).abs()
    with capsys.disabled():
        print(f"\n131072 tokens, {hq}/{hkv} heads, {tiles} tiles: reference Triton kernel {t_ref:.1f} ms "
              f"({tiles * 2097152 / t_ref / 1e9:.0f} TFLOP/s), product kernel {t_new:.1f} ms "
              f"({tiles * 2097152 / t_new / 1e9:.0f} TFLOP/s), ratio {t_ref / t_new:.2f}; max-abs difference {d.max().item():.2e}")
    assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS
    assert t_new < t_ref


def test_attention_accepts_strided_layout_and_repeated_kv(dev):
    """[B,N,H,D] memory viewed as [B,H,N,D] (the layout HF projections produce) and K/V already
    repeated to the query head count, as the reference's caller passes them."""
    from minference_b200.ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention
    from minference_b200.synthetic import local_vs_indices, make_qkv
    from oracle import reference_math as R

    n, hq, hkv = 2000, 4, 2
    q, k, v = make_qkv(n, hq, hkv, seed=9, dtype=torch.bfloat16)
    vi, si = local_vs_indices(n, hq, 64, 256, seed=1)
    qs = q.transpose(1, 2).contiguous().transpose(1, 2).to(dev)
    kr = k.repeat_interleave(hq // hkv, dim=1).transpose(1, 2).contiguous().transpose(1, 2).to(dev)
    vr = v.repeat_interleave(hq // hkv, dim=1).to(dev)
    out = vertical_slash_sparse_attention(qs, kr, vr, vi.to(dev), si.to(dev))
    ref, _ = R.vertical_slash_attention_oracle(q.float(), k.float(), v.float(), vi, si)
    _close(out, ref[:, :, :n], "strided")


@pytest.mark.parametrize("n,n_init,n_local", [(64, 16, 32), (128, 0, 128), (1000, 16, 200), (3000, 128, 512), (700, 128, 4096)])
def test_streaming_attention_matches_oracle(dev, n, n_init, n_local):
    from minference_b200.ops.streaming_kernel import streaming_forward
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    q, k, v = make_qkv(n, 2, 1, seed=1, dtype=torch.bfloat16)
    out = streaming_forward(q.to(dev), k.to(dev), v.to(dev), n_init, n_local)
    ref = R.streaming_attention_oracle(q.float(), k.float(), v.float(), n_init, n_local)
    _close(out, ref[:, :, :n], (n, n_init, n_local))


@pytest.mark.parametrize("n,n_last,n_init,n_local", [(1500, 100, 64, 256), (2048, 300, 128, 512), (700, 100, 128, 4096)])
def test_tri_shape_matches_oracle(dev, n, n_last, n_init, n_local):
    """A-shape rows (on the sequence cut before the last rows) + dense last rows
    (ops/streaming_kernel.py:820-833 of the reference)."""
    from minference_b200.ops.streaming_kernel import tri_shape_kernel
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    q, k, v = make_qkv(n, 4, 2, seed=21, dtype=torch.bfloat16)
    out = tri_shape_kernel(q.to(dev), k.to(dev), v.to(dev),
                           {"attn_forward_config": {"n_init": n_init, "n_local": n_local, "n_last": n_last}}).float().cpu()
    cut = n - n_last
    ref1 = R.streaming_attention_oracle(q[:, :, :cut], k[:, :, :cut], v[:, :, :cut], n_init, n_local)[:, :, :cut]
    ref2 = torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float().repeat_interleave(2, 1), v.float().repeat_interleave(2, 1), is_causal=True)[:, :, cut:]
    d = (out - torch.cat([ref1, ref2], 2)).abs()
    assert out.shape == (1, 4, n, 128) and d.max().item() < 2e-2 and d.mean().item() < 2e-3


@pytest.mark.parametrize("kind", ["dilated1", "dilated2"])
def test_dilated_index_sets_match_oracle(dev, kind):
    from minference_b200.ops.pit_sparse_flash_attention_v2 import dilated_sparse_attention
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    n = 2500
    q, k, v = make_qkv(n, 2, 1, seed=22, dtype=torch.bfloat16)
    out = dilated_sparse_attention(q.to(dev), k.to(dev), v.to(dev), kind).float().cpu()
    pos = torch.arange(n)
    pos = pos[-8192::2] if kind == "dilated1" else torch.cat([pos[-2048:], pos[-6144:-2048:2]], 0)
    v_idx = torch.arange(min(1024, n))[None, None, :].expand(1, 2, -1)
    s_idx = ((n - 1) - pos)[None, None, :].expand(1, 2, -1)
    ref, _ = R.vertical_slash_attention_oracle(q, k, v, v_idx, s_idx)
    d = (out - ref[:, :, :n]).abs()
    assert d.max().item() < 2e-2 and d.mean().item() < 2e-3


@pytest.mark.parametrize("n,top_k", [(1000, 5), (4096, 16), (1024, 100)])
def test_block_sparse_matches_oracle(dev, n, top_k):
    from minference_b200.ops.block_sparse_flash_attention import _build_block_index, block_sparse_attention
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    hq, hkv = 4, 2
    q, k, v = make_qkv(n, hq, hkv, seed=6, dtype=torch.bfloat16)
    bidx = _build_block_index(q.to(dev), k.to(dev), top_k).cpu().numpy()
    pad = R.block_sparse_pad(n)
    qp = torch.nn.functional.pad(q, [0, 0, 0, pad])
    kp = torch.nn.functional.pad(k, [0, 0, 0, pad]).repeat_interleave(hq // hkv, dim=1)
    ref_idx = R.build_block_index(qp, kp, top_k).numpy()       # bf16 on CPU like the reference's bf16 path
    assert bidx.shape == ref_idx.shape
    tot = hit = 0
    for h in range(hq):
        for m in range(bidx.shape[2]):
            c = min(m + 1, bidx.shape[3])
            assert np.all(np.diff(bidx[0, h, m, :c]) > 0) and bidx[0, h, m, c - 1] <= m      # sorted, causal
            tot += c
            hit += len(set(bidx[0, h, m, :c].tolist()) & set(ref_idx[0, h, m, :c].tolist()))
    assert hit >= 0.95 * tot          # bf16 block scores tie often; torch.topk's tie order is unspecified
    # the gate: wherever the reference's pooled bf16 scores separate the top-k from the rest, the sets are equal
    pooled_q = qp.float().reshape(1, hq, -1, 64, 128).mean(-2).to(torch.bfloat16)
    pooled_k = kp.float().reshape(1, hq, -1, 64, 128).mean(-2).to(torch.bfloat16)
    scores = torch.einsum("bhmk,bhnk->bhmn", pooled_q, pooled_k).float().numpy()
    decided = 0
    for h in range(hq):
        for m in range(bidx.shape[2]):
            c = min(m + 1, bidx.shape[3])
            if c == m + 1:      # every causal block is taken
                assert set(bidx[0, h, m, :c].tolist()) == set(range(m + 1))
                continue
            row = scores[0, h, m, : m + 1]
            order = np.sort(row)[::-1]
            kth, nxt = order[c - 1], order[c]
            tol = 2 ** -7 * max(np.abs(row).max(), 1e-6)     # one bf16 step of the largest pooled score of the row
            must = set(np.nonzero(row > kth + tol)[0].tolist())
            never = set(np.nonzero(row < nxt - tol)[0].tolist())
            got = set(bidx[0, h, m, :c].tolist())
            assert must <= got and not (got & never), (h, m)
            decided += len(must) + len(never)
    assert decided > 0 or top_k >= bidx.shape[2]
    # attention over the kernel's own index set
    out = block_sparse_attention(q.to(dev), k.to(dev), v.to(dev), top_k)
    rows = (n + 63) // 64
    ref = torch.zeros(1, hq, rows * 64, 128)
    for h in range(hq):
        mask = R.block_sparse_mask_rows(bidx[0, h], n, list(range(rows)))
        for m in range(rows):
            r0, r1 = m * 64, min(m * 64 + 64, n)
            ref[0, h, r0:r1] = R.masked_attention_rows(q[0, h, r0:r1], k[0, h // 2], v[0, h // 2], mask[m * 64:m * 64 + (r1 - r0)], r0)
    _close(out, ref[:, :, :n], (n, top_k))


def test_block_index_matches_reference_fixtures_on_gpu(dev, golden_dir):
    """The GPU block-index builder against fixtures made by the reference's own _build_block_index (fp32 run on
    fp16-exact data): on the consumed prefix, sets are equal wherever the fixture's scores separate them by more
    than the bf16 pooling noise of the kernel."""
    from minference_b200.ops.block_sparse_flash_attention import _build_block_index

    paths = sorted(glob.glob(os.path.join(golden_dir, "block_index_*.npz")))
    assert len(paths) >= 3
    for path in paths:
        z = np.load(path)
        n, top_k = int(z["n"]), int(z["top_k"])
        q32, k32 = torch.from_numpy(z["q"]).float(), torch.from_numpy(z["k"]).float()
        q, k = q32.to(torch.bfloat16), k32.to(torch.bfloat16)
        got = _build_block_index(q.to(dev), k.to(dev), top_k).cpu().numpy()
        ref = z["block_index"]
        assert got.shape == ref.shape, path
        pad = 64 - (n & 63)
        pq = torch.nn.functional.pad(q32, [0, 0, 0, pad]).reshape(1, 1, -1, 64, 128).mean(-2)
        pk = torch.nn.functional.pad(k32, [0, 0, 0, pad]).reshape(1, 1, -1, 64, 128).mean(-2)
        scores = torch.einsum("bhmk,bhnk->bhmn", pq, pk).numpy()
        tot = hit = 0
        for m in range(got.shape[2]):
            c = min(m + 1, got.shape[3])
            g, r = set(got[0, 0, m, :c].tolist()), set(ref[0, 0, m, :c].tolist())
            tot += c
            hit += len(g & r)
            if c == m + 1:
                assert g == r == set(range(m + 1)), (path, m)
                continue
            row = scores[0, 0, m, : m + 1]
            order = np.sort(row)[::-1]
            kth, nxt = order[c - 1], order[c]
            tol = 3 * 2 ** -8 * max(np.abs(row).max(), 1e-6)      # bf16 inputs, bf16 pooled vectors, bf16 scores
            assert set(np.nonzero(row > kth + tol)[0].tolist()) <= g, (path, m)
            assert not (g & set(np.nonzero(row < nxt - tol)[0].tolist())), (path, m)
        assert hit >= 0.8 * tot, (path, hit, tot)       # a 512-token fixture has 24 consumed entries: three near-ties are 12 %


def test_mixed_pattern_prefill_forward(dev):
    """Per-head pattern table with all three pattern types, one call for the layer."""
    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.ops.block_sparse_flash_attention import block_sparse_attention
    from minference_b200.ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.ops.streaming_kernel import streaming_forward
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 3000, 6, 2
    q, k, v = make_qkv(n, hq, hkv, seed=11, dtype=torch.bfloat16)
    dq, dk, dv = q.to(dev), k.to(dev), v.to(dev)
    table = {"0": ["vertical_and_slash", 100, 400, 1.0], "1": ["stream_llm", 128, 512, 1.0], "2": ["block_sparse", 0, 0, 1.0],
             "3": ["vertical_and_slash", 30, 800, 1.0], "4": ["block_sparse", 0, 0, 1.0]}   # head 5: default pattern
    cfg = {"attn_forward_config": {"best_pattern": [table]}, "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None}
    out = minference_prefill_forward(dq, dk, dv, cfg)
    assert out.shape == q.shape and torch.isfinite(out.float()).all()
    # each head equals the single-pattern operator on that head (same kernels, same index sets)
    for h, (ty, a, b, _) in {**{str(i): ["vertical_and_slash", 1000, 6096, 1] for i in range(hq)}, **table}.items():
        h = int(h)
        hk = h // (hq // hkv)
        qh, kh, vh = dq[:, h:h + 1], dk[:, hk:hk + 1], dv[:, hk:hk + 1]
        if ty == "stream_llm":
            ref = streaming_forward(qh, kh, vh, a, b)
        elif ty == "block_sparse":
            ref = block_sparse_attention(qh.contiguous(), kh.contiguous(), vh.contiguous(), 100)
        else:
            vi, si, nv_, ns_ = vertical_slash_estimate(qh, kh, a, b)
            ref = vertical_slash_sparse_attention(qh, kh, vh, vi, si)
        assert (out[:, h:h + 1].float() - ref.float()).abs().max().item() < 1e-2, (h, ty)


def test_dense_layers_below_starting_layer(dev):
    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.synthetic import make_qkv

    n = 777
    q, k, v = make_qkv(n, 4, 2, seed=3, dtype=torch.bfloat16)
    cfg = {"attn_forward_config": {"best_pattern": [{}], "starting_layer": 1}, "layer_idx": 0, "num_hidden_layers": 2,
           "attention_mask": None}
    out = minference_prefill_forward(q.to(dev), k.to(dev), v.to(dev), cfg)
    kr, vr = k.repeat_interleave(2, dim=1).float(), v.repeat_interleave(2, dim=1).float()
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), kr, vr, is_causal=True)
    _close(out, ref, "dense")


def test_full_size_properties_131072(dev):
    """At the benchmark size the oracle cannot recompute everything: check size-independent
    properties instead.  (1) V = ones gives ones (softmax rows sum to 1 over any index set);
    (2) sampled row blocks against the fp32 oracle; (3) the plan holds as many tiles as the
    reference-format tables of one head."""
    from minference_b200.cuda import convert_vertical_slash_indexes
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    n, hq, hkv = 131072, 8, 2
    q, k, v = make_qkv(n, hq, hkv, seed=0, dtype=torch.bfloat16, device=dev)
    v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q, k, 1000, 6096)
    plan = build_vertical_slash_plan(v_idx, s_idx, n, nnz_v, nnz_s)
    ones = sparse_attention_forward(q, k, torch.ones_like(v), plan)
    assert (ones.float() - 1).abs().max().item() < 1e-2
    out = sparse_attention_forward(q, k, v, plan)
    assert plan.status.tolist()[:2] == [0, 0]
    bc, bo, cc, ci = convert_vertical_slash_indexes(torch.tensor([n], dtype=torch.int32, device=dev),
                                                    v_idx[:, :1].contiguous(), s_idx[:, :1].contiguous(), n)
    head0_tiles = int(bc.sum().item() + ((cc + 63) // 64).sum().item())
    plan0 = build_vertical_slash_plan(v_idx[:, :1].contiguous(), s_idx[:, :1].contiguous(), n)
    assert plan0.count_tiles() == head0_tiles
    bc, bo, cc, ci = (t[0, 0].cpu().numpy() for t in (bc, bo, cc, ci))
    rows = n // 64
    qc, kc, vc = q[0, 0].float().cpu(), k[0, 0].float().cpu(), v[0, 0].float().cpu()
    for m in (0, 1, 17, rows // 2, rows - 1):
        mask = R.vs_mask_for_rows(bc, bo, cc, ci, n, [m])
        ref = R.masked_attention_rows(qc[m * 64:m * 64 + 64], kc, vc, mask, m * 64)
        d = (out[0, 0, m * 64:m * 64 + 64].float().cpu() - ref).abs()
        assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, (m, d.max().item())


def test_full_size_mixed_patterns_262144(dev):
    """Mixed-pattern layer of the Qwen2.5-7B head geometry (28 query / 4 KV heads, 262144 tokens): V = 1 must give 1
    for every head pattern (each row's weights sum to one), and sampled row blocks of an A-shape
    head and a block-sparse head match the masked-dense oracle."""
    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.ops.block_sparse_flash_attention import _build_block_index
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    n, hq, hkv = 262144, 28, 4
    q, k, v = make_qkv(n, hq, hkv, seed=1, dtype=torch.bfloat16, device=dev)
    kinds = ["stream_llm", "vertical_and_slash", "block_sparse"]
    table = {str(h): ([kinds[h % 3], 128, 4096, 1.0] if h % 3 == 0 else
                      [kinds[h % 3], 1000, 6096, 1.0] if h % 3 == 1 else [kinds[h % 3], 100, 0, 1.0]) for h in range(hq)}
    kw = {"attn_forward_config": {"best_pattern": [table]}, "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None}
    ones = minference_prefill_forward(q, k, torch.ones_like(v), kw)
    assert (ones.float() - 1).abs().max().item() < 1e-2
    out = minference_prefill_forward(q, k, v, kw)
    rows = n // 64
    rep = hq // hkv
    # A-shape head 0
    kc, vc = k[0, 0].float().cpu(), v[0, 0].float().cpu()
    for m in (0, 63, 64, 65, rows // 3, rows - 1):
        mask = R.a_shape_mask_rows(n, 128, 4096, m * 64, m * 64 + 64)
        ref = R.masked_attention_rows(q[0, 0, m * 64:m * 64 + 64].float().cpu(), kc, vc, mask, m * 64)
        d = (out[0, 0, m * 64:m * 64 + 64].float().cpu() - ref).abs()
        assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, ("a_shape", m, d.max().item())
    # block-sparse head 2 (index taken from the GPU planner: ties in the pooled bf16 scores are unpinned)
    h = 2
    bidx = _build_block_index(q[:, h:h + 1], k[:, h // rep:h // rep + 1], 100)[0, 0].cpu().numpy()
    kc, vc = k[0, h // rep].float().cpu(), v[0, h // rep].float().cpu()
    for m in (0, 5, 150, rows // 2, rows - 1):
        mask = R.block_sparse_mask_rows(bidx, n, [m])
        ref = R.masked_attention_rows(q[0, h, m * 64:m * 64 + 64].float().cpu(), kc, vc, mask, m * 64)
        d = (out[0, h, m * 64:m * 64 + 64].float().cpu() - ref).abs()
        assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS, ("block_sparse", m, d.max().item())
