"""Sequence-sharded path on the GPU.

On one GPU the ranks are emulated one after the other in a single process (no kernel waits on
another): every (query chunk, key chunk) pair goes through the windowed C-ABI entry points and
the partial results are merged, then compared with the whole-sequence kernel and the oracle.
With two or more GPUs the real ring (NCCL send/recv between processes) is run as well."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _one_rounding_apart(a, b, slack: float = 2e-3):
    """Two bf16 results of the same attention computed through different chains of key chunks.  Both accumulate in
    fp32 and round the output once, but P is rounded to bf16 against each chain's own running maximum, which moves
    the fp32 sums by a few 1e-4 of their terms: the results are equal or neighbouring bf16 values, up to `slack` for
    outputs that are small because their terms cancel."""
    a, b = a.float(), b.float()
    ulp = torch.exp2(torch.floor(torch.log2(torch.maximum(a.abs(), b.abs()).clamp_min(2.0 ** -100))) - 7)
    excess = ((a - b).abs() - ulp * 1.001 - slack).max().item()
    if excess > 0:
        print(f"largest difference beyond one bf16 step + {slack}: {excess:.3e}; max abs difference {(a - b).abs().max().item():.3e}")
    return excess <= 0


def _pairs_through_carry(ring, qs, ks, vs, n, c, qc, plan, v_idx, cap_s, status, world, **kw):
    """All visible key chunks of query chunk qc through the windowed kernel with its fp32 carry; the bf16
    output is written by the last call."""
    dev = qs.device
    hq = qs.shape[1]
    acc_o = torch.empty(1, hq, c, 128, device=dev)
    acc_l = torch.full((1, hq, c), float("-inf"), device=dev)
    out = torch.full((1, hq, c, 128), float("nan"), dtype=qs.dtype, device=dev)
    visible = [kc for kc in range(2 * world) if ring.pair_is_visible(qc, kc)]
    for kc in visible:
        ring.attention_window(qs[:, :, qc * c:(qc + 1) * c], ks[:, :, kc * c:(kc + 1) * c], vs[:, :, kc * c:(kc + 1) * c],
                              n, qc * c, kc * c, plan, v_idx, cap_s, status, carry=(acc_o, acc_l),
                              out=out if kc == visible[-1] else None, **kw)
    return out


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.mark.parametrize("world,n,kind", [(2, 2048, "local"), (2, 4096, "rand"), (4, 4096, "rand")])
def test_windowed_kernel_pairs_merge_to_full_attention(dev, world, n, kind):
    from minference_b200 import _cabi
    from minference_b200.dist import ring
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import local_vs_indices, make_qkv
    from oracle import reference_math as R
    from tests.golden.make_golden import index_case

    hq, hkv = 4, 2
    q, k, v = make_qkv(n, hq, hkv, seed=8, dtype=torch.bfloat16)
    if kind == "local":
        vi, si = local_vs_indices(n, hq, 64, 300, seed=4)
    else:
        a, b = index_case(3, n, hq, 120, 260, "uniform")
        b[..., -1] = 0
        vi, si = torch.from_numpy(a), torch.from_numpy(b)
    vs, ss = R.presort_indices(vi, si, 1, hq)
    dq, dk, dv, dvs, dss = (t.to(dev) for t in (q, k, v, vs.contiguous(), ss.contiguous()))
    full = sparse_attention_forward(dq, dk, dv, build_vertical_slash_plan(dvs, dss, n))
    c = ring.chunk_size(n, world)
    parts = []
    for r in range(world):
        outs = []
        for qc in ring.owned_chunks(r, world):
            plan, status = ring.build_plan_window(dvs, dss, None, None, n, qc * c, c)
            outs.append(_pairs_through_carry(ring, dq, dk, dv, n, c, qc, plan, dvs, dss.shape[2], status, world))
            assert status.tolist()[:2] == [0, 0]       # words 2-3 count the tiles sent to the tensor pipe
        parts.append(torch.cat(outs, dim=2))
    merged = ring.zigzag_merge(parts, world).float()
    assert _one_rounding_apart(merged, full)       # merged in fp32 inside the kernel, rounded once
    ref, _ = R.vertical_slash_attention_oracle(q.float(), k.float(), v.float(), vi, si)
    d = (merged.cpu() - ref[:, :, :n]).abs()
    assert d.max().item() < 2e-2 and d.mean().item() < 2e-3


@pytest.mark.parametrize("n,world", [(4096, 2), (32768, 2), (32768, 8)])
def test_sharded_estimator_stages_match_whole_sequence(dev, n, world):
    """Score passes over key windows + combine + select == minf_vs_estimate on the whole sequence: the same
    bits when the chunks are multiples of the 2048-key statistics block, the same sets up to near-ties otherwise."""
    from minference_b200 import _cabi
    from minference_b200.dist import ring
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.synthetic import make_qkv

    hq, hkv = 4, 2
    q, k, _ = make_qkv(n, hq, hkv, seed=12, dtype=torch.bfloat16)
    dq, dk = q.to(dev), k.to(dev)
    v_ref, s_ref, nv_ref, ns_ref, vs_ref, ss_ref = vertical_slash_estimate(dq, dk, 200, 600, return_scores=True)
    L = _cabi.lib()
    c = n // (2 * world)
    bl = L.minf_vs_scores_blocks(c)
    total = 2 * world * bl
    stats = torch.empty((hq, 64, total, 2), dtype=torch.float32, device=dev)
    row_stats = torch.empty((hq, 64, 2), dtype=torch.float32, device=dev)
    scores = torch.zeros((2, 1, hq, n), dtype=torch.float32, device=dev)
    status = _cabi.new_status(dev)
    q_last = dq[:, :, -64:].contiguous()
    for pass_ in (1, 2):
        for ci in range(2 * world):
            kp = dk[:, :, ci * c:(ci + 1) * c]
            _cabi.check(L.minf_vs_scores_pass(pass_, _cabi.ptr(q_last), _cabi.ptr(kp), _cabi.strides3(q_last), _cabi.strides3(kp),
                                              1, hq, hkv, n, c, ci * c, 128, _cabi.ptr(stats), ci * bl, total, _cabi.ptr(row_stats),
                                              _cabi.ptr(scores[0]), _cabi.ptr(scores[1]), _cabi.ptr(status), _cabi.stream_ptr(dev)))
        if pass_ == 1:
            _cabi.check(L.minf_vs_scores_combine(_cabi.ptr(stats), 1, hq, total, _cabi.ptr(row_stats), _cabi.stream_ptr(dev)))
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    vsz = torch.full((hq,), 200, dtype=torch.int32, device=dev)
    ssz = torch.full((hq,), 600, dtype=torch.int32, device=dev)
    v_idx = torch.empty((1, hq, 200), dtype=torch.int32, device=dev)
    s_idx = torch.empty((1, hq, 600), dtype=torch.int32, device=dev)
    nnz_v = torch.empty(hq, dtype=torch.int32, device=dev)
    nnz_s = torch.empty(hq, dtype=torch.int32, device=dev)
    scratch = torch.empty(L.minf_vs_select_scratch_bytes(1, hq, n), dtype=torch.uint8, device=dev)
    _cabi.check(L.minf_vs_select(_cabi.ptr(scores[0]), _cabi.ptr(scores[1]), 1, hq, n, _cabi.ptr(vsz), _cabi.ptr(ssz), 200, 600,
                                 _cabi.ptr(v_idx), _cabi.ptr(s_idx), _cabi.ptr(nnz_v), _cabi.ptr(nnz_s), *_cabi.SELECT_RULES["online"],
                                 _cabi.ptr(scratch), _cabi.stream_ptr(dev)))
    if c % 2048 == 0:
        assert torch.equal(scores[0], vs_ref) and torch.equal(scores[1], ss_ref)
        assert torch.equal(v_idx, v_ref) and torch.equal(s_idx, s_ref)
    else:
        assert (scores[0] - vs_ref).abs().max().item() < 1e-4 * max(vs_ref[..., 30:].max().item(), 1e-6) + 1e-6
        assert (scores[1] - ss_ref).abs().max().item() < 1e-4 * max(ss_ref[..., 100:].max().item(), 1e-6) + 1e-6
        for h in range(hq):
            assert len(set(v_idx[0, h].tolist()) & set(v_ref[0, h].tolist())) >= 198
            assert len(set(s_idx[0, h].tolist()) & set(s_ref[0, h].tolist())) >= 594
    # the slash windows the ranks exchange cover every offset their keys reach
    for ci in range(2 * world):
        lo, hi = ring.slash_window(n, ci, c)
        own = torch.zeros((2, 1, hq, n), dtype=torch.float32, device=dev)
        kp = dk[:, :, ci * c:(ci + 1) * c]
        _cabi.check(L.minf_vs_scores_pass(2, _cabi.ptr(q_last), _cabi.ptr(kp), _cabi.strides3(q_last), _cabi.strides3(kp),
                                          1, hq, hkv, n, c, ci * c, 128, None, 0, total, _cabi.ptr(row_stats),
                                          _cabi.ptr(own[0]), _cabi.ptr(own[1]), _cabi.ptr(status), _cabi.stream_ptr(dev)))
        assert own[1][..., :lo].abs().max().item() == 0 if lo else True
        assert own[1][..., hi:].abs().max().item() == 0 if hi < n else True
        assert own[0][..., :ci * c].abs().sum().item() == 0 and own[0][..., (ci + 1) * c:].abs().sum().item() == 0
        if ci == 2 * world - 1:
            break


@pytest.mark.parametrize("n,world", [(8192, 2), (32768, 4), (65536, 8)])
def test_score_exchange_of_emulated_ranks_reproduces_whole_sequence_scores(dev, n, world):
    """The pack every rank sends (its keys' vertical scores + the diagonal offsets they reach) and the assembly of all
    packs, with the ranks emulated one after the other: bit-identical to the whole-sequence estimator, including the
    middle rank whose two chunks are neighbours."""
    from minference_b200 import _cabi
    from minference_b200.dist import ring
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.synthetic import make_qkv

    hq, hkv = 4, 2
    q, k, _ = make_qkv(n, hq, hkv, seed=13, dtype=torch.bfloat16)
    dq, dk = q.to(dev), k.to(dev)
    *_, vs_ref, ss_ref = vertical_slash_estimate(dq, dk, 200, 600, return_scores=True)
    L = _cabi.lib()
    c = ring.chunk_size(n, world)
    assert c % 2048 == 0
    bl = L.minf_vs_scores_blocks(c)
    q_last = dq[:, :, -64:].contiguous()
    status = _cabi.new_status(dev)

    def score_pass(pass_, kp, ci, stats, offset, total, row_stats, vertical, slash):
        _cabi.check(L.minf_vs_scores_pass(pass_, _cabi.ptr(q_last), _cabi.ptr(kp), _cabi.strides3(q_last), _cabi.strides3(kp),
                                          1, hq, hkv, n, c, ci * c, 128, _cabi.ptr(stats), offset, total, _cabi.ptr(row_stats),
                                          _cabi.ptr(vertical), _cabi.ptr(slash), _cabi.ptr(status), _cabi.stream_ptr(dev)))

    per_rank = []
    for r in range(world):
        stats = torch.empty((hq, 64, 2 * bl, 2), dtype=torch.float32, device=dev)
        for i, ci in enumerate(ring.owned_chunks(r, world)):
            score_pass(1, dk[:, :, ci * c:(ci + 1) * c], ci, stats, i * bl, 2 * bl, None, None, None)
        per_rank.append(stats)
    all_stats = ring._ordered_blocks(torch.stack(per_rank), world, bl)
    row_stats = torch.empty((hq, 64, 2), dtype=torch.float32, device=dev)
    _cabi.check(L.minf_vs_scores_combine(_cabi.ptr(all_stats), 1, hq, all_stats.shape[2], _cabi.ptr(row_stats), _cabi.stream_ptr(dev)))
    packs = []
    for r in range(world):
        chunks = ring.owned_chunks(r, world)
        packs.append(ring.rank_score_pack(
            lambda i, vertical, slash: score_pass(2, dk[:, :, chunks[i] * c:(chunks[i] + 1) * c], chunks[i], None, 0,
                                                  2 * world * bl, row_stats, vertical, slash),
            chunks, n, c, 1, hq, dev))
    scores = ring.assemble_scores(torch.stack(packs), n, c, world)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert torch.equal(scores[0], vs_ref) and torch.equal(scores[1], ss_ref)


@pytest.mark.parametrize("world,n,n_init,n_local", [(2, 4096, 128, 512), (4, 8192, 64, 1500)])
def test_windowed_kernel_pairs_merge_mixed_a_shape_and_vertical_slash(dev, world, n, n_init, n_local):
    """Heads 0 and 2 vertical-slash, heads 1 and 3 A-shape, in the same windowed launches."""
    from minference_b200 import _cabi
    from minference_b200.dist import ring
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import local_vs_indices, make_qkv
    from oracle import reference_math as R

    hq, hkv = 4, 2
    q, k, v = make_qkv(n, hq, hkv, seed=9, dtype=torch.bfloat16)
    vi, si = local_vs_indices(n, hq, 64, 300, seed=5)
    vs, ss = R.presort_indices(vi, si, 1, hq)
    dq, dk, dv, dvs, dss = (t.to(dev) for t in (q, k, v, vs.contiguous(), ss.contiguous()))
    mode = torch.tensor([_cabi.MODE_PLAN, _cabi.MODE_ASHAPE] * 2, dtype=torch.int32, device=dev)
    param = torch.tensor([[0, 0], [n_init, n_local]] * 2, dtype=torch.int32, device=dev)
    full = sparse_attention_forward(dq, dk, dv, build_vertical_slash_plan(dvs, dss, n), head_mode=mode, head_param=param)
    c = ring.chunk_size(n, world)
    parts = []
    for r in range(world):
        outs = []
        for qc in ring.owned_chunks(r, world):
            plan, status = ring.build_plan_window(dvs, dss, None, None, n, qc * c, c)
            outs.append(_pairs_through_carry(ring, dq, dk, dv, n, c, qc, plan, dvs, dss.shape[2], status, world,
                                             head_mode=mode, head_param=param))
            assert status.tolist()[:2] == [0, 0]
        parts.append(torch.cat(outs, dim=2))
    merged = ring.zigzag_merge(parts, world).float()
    assert _one_rounding_apart(merged, full)
    ref = R.streaming_attention_oracle(q[:, 1:2].float(), k[:, 0:1].float(), v[:, 0:1].float(), n_init, n_local)
    d = (merged[:, 1:2].cpu() - ref[:, :, :n]).abs()
    assert d.max().item() < 2e-2 and d.mean().item() < 2e-3


@pytest.mark.parametrize("world,n,top_k", [(2, 4096, 6), (4, 8192, 20)])
def test_windowed_block_sparse_planner_matches_whole_sequence(dev, world, n, top_k):
    """Pooled keys of the whole sequence + per-chunk block selection (the sequence-sharded planner)
    give the same attention as the whole-sequence block-sparse operator."""
    from minference_b200 import _cabi
    from minference_b200.dist import ring
    from minference_b200.ops.block_sparse_flash_attention import block_sparse_attention
    from minference_b200.synthetic import make_qkv

    hq, hkv = 4, 2
    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=10, dtype=torch.bfloat16))
    full = block_sparse_attention(q, k, v, top_k).float()
    L = _cabi.lib()
    c = ring.chunk_size(n, world)
    k_pool_all = torch.cat([ring._pooled_blocks(k[:, :, ch * c:(ch + 1) * c]) for ch in range(2 * world)], dim=2).contiguous()
    merged = torch.zeros(1, hq, n, 128, device=dev)
    for qc in range(2 * world):
        plan = torch.empty(L.minf_plan_bytes_window(1, hq, qc * c, c, 0, top_k), dtype=torch.uint8, device=dev)
        status = _cabi.new_status(dev)
        q_pool = ring._pooled_blocks(q[:, :, qc * c:(qc + 1) * c])
        _cabi.check(L.minf_block_sparse_select_window(_cabi.ptr(q_pool), _cabi.ptr(k_pool_all), 1, hq, hkv, n, qc * c, c, top_k,
                                                      None, 0, top_k, _cabi.ptr(plan), _cabi.stream_ptr(dev)))
        # this one keeps the unfused form: normalised partial outputs merged with torch ops
        acc_o = torch.zeros(1, hq, c, 128, device=dev)
        acc_l = torch.full((1, hq, c), float("-inf"), device=dev)
        for kc in range(qc + 1):
            o, lse = ring.attention_window(q[:, :, qc * c:(qc + 1) * c], k[:, :, kc * c:(kc + 1) * c], v[:, :, kc * c:(kc + 1) * c],
                                           n, qc * c, kc * c, plan, None, top_k, status, cap_v=0)
            ring.merge_partial(acc_o, acc_l, o, lse)
        assert status.tolist()[:2] == [0, 0]
        merged[:, :, qc * c:(qc + 1) * c] = acc_o
    assert (merged - full).abs().max().item() < 1.5e-2       # two bf16 roundings apart


def test_real_ring_on_two_gpus():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", os.path.join(ROOT, "tests", "multi_gpu_ring_check.py")]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    print(p.stdout[-2000:])
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "RING_OK" in p.stdout
