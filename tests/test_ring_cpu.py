"""The ring orchestration (zigzag layout, pair schedule, communication, log-sum-exp merge) on two
and four CPU ranks over gloo, with the CPU oracle standing in for the attention kernel."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from minference_b200.dist import ring
from oracle import reference_math as R


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_window(q, k, v, index, h_rep, n_ctx, q_pos0, kv_pos0):
    """Masked-dense partial attention of one (query chunk, key chunk) pair + base-2 log-sum-exp."""
    bc, bo, cc, ci = index
    B, H, C, D = q.shape
    out = torch.zeros(B, H, C, D)
    lse = torch.full((B, H, C), float("-inf"))
    scale = D ** -0.5
    rbs = list(range(q_pos0 // 64, (q_pos0 + C) // 64))
    for h in range(H):
        mask = R.vs_mask_for_rows(bc[0, h], bo[0, h], cc[0, h], ci[0, h], n_ctx, rbs)[:, kv_pos0:kv_pos0 + k.shape[2]]
        s = (q[0, h].float() @ k[0, h // h_rep].float().T) * scale
        s = s.masked_fill(~torch.from_numpy(mask), float("-inf"))
        mx = s.max(-1, keepdim=True).values
        mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
        p = torch.exp(s - mx)
        den = p.sum(-1, keepdim=True)
        out[0, h] = (p @ v[0, h // h_rep].float()) / torch.where(den == 0, torch.ones_like(den), den)
        lse[0, h] = torch.where(den[:, 0] == 0, torch.full_like(den[:, 0], float("-inf")),
                                (mx[:, 0] + torch.log(den[:, 0])) / np.log(2.0))
    return out, lse


def _worker(rank, world, port, n, hq, hkv, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from minference_b200.synthetic import local_vs_indices, make_qkv

        q, k, v = make_qkv(n, hq, hkv, seed=5, dtype=torch.float32)
        vi, si = local_vs_indices(n, hq, 40, 300, seed=2)
        vs, ss = R.presort_indices(vi, si, 1, hq)
        index = R.convert_vertical_slash_indexes(np.array([n], np.int32), vs.numpy(), ss.numpy(), n)
        q_loc, k_loc, v_loc = (ring.zigzag_split(t, rank, world) for t in (q, k, v))

        def attn_fn(qc, kc, vc, qi, q_pos0, kv_pos0):
            return _oracle_window(qc, kc, vc, index, hq // hkv, n, q_pos0, kv_pos0)

        out_loc = ring.ring_attention(q_loc, k_loc, v_loc, n, attn_fn)
        gathered = [torch.empty_like(out_loc) for _ in range(world)]
        dist.all_gather(gathered, out_loc)
        if rank == 0:
            full = ring.zigzag_merge(gathered, world)
            ref, _ = R.vertical_slash_attention_oracle(q, k, v, vi, si)
            result.put(float((full - ref[:, :, :n]).abs().max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ring_schedule_and_merge_on_gloo_ranks(world):
    n = 256 * 2 * world
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, 4, 2, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    assert result.get(timeout=10) < 1e-4


def test_zigzag_layout_roundtrip_and_balance():
    world, n = 4, 256 * 8
    x = torch.arange(n, dtype=torch.float32).reshape(1, 1, n, 1)
    parts = [ring.zigzag_split(x, r, world) for r in range(world)]
    assert torch.equal(ring.zigzag_merge(parts, world), x)
    # every rank owns one early and one late chunk: the causal work (sum of visible chunk pairs) is equal
    work = []
    for r in range(world):
        work.append(sum(1 for qc in ring.owned_chunks(r, world) for kc in range(2 * world) if ring.pair_is_visible(qc, kc)))
    assert len(set(work)) == 1
    with pytest.raises(ValueError):
        ring.chunk_size(1000, 2)


def test_merge_partial_matches_joint_softmax():
    torch.manual_seed(0)
    s = torch.randn(1, 2, 5, 12)
    v = torch.randn(1, 2, 12, 3)
    ref = torch.softmax(s, -1) @ v
    acc_o = torch.zeros(1, 2, 5, 3)
    acc_l = torch.full((1, 2, 5), float("-inf"))
    for lo, hi in ((0, 5), (5, 5), (5, 12)):          # includes an empty part
        if hi == lo:
            ring.merge_partial(acc_o, acc_l, torch.zeros(1, 2, 5, 3), torch.full((1, 2, 5), float("-inf")))
            continue
        part = s[..., lo:hi]
        o = torch.softmax(part, -1) @ v[..., lo:hi, :]
        lse = torch.logsumexp(part, -1) / np.log(2.0)
        ring.merge_partial(acc_o, acc_l, o, lse)
    assert (acc_o - ref).abs().max() < 1e-5


def _dense_window(q, k, v, qi, q_pos0, kv_pos0):
    """Plain causal attention of one (query chunk, key chunk) pair at global positions + base-2 lse."""
    B, H, C, D = q.shape
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, 1).float(), v.repeat_interleave(rep, 1).float()
    s = (q.float() @ kk.transpose(-1, -2)) * D ** -0.5
    rows = q_pos0 + torch.arange(C)[:, None]
    cols = kv_pos0 + torch.arange(k.shape[2])[None, :]
    s = s.masked_fill(cols > rows, float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    return (p @ vv).to(q.dtype), lse / np.log(2.0)


def _runner_worker(rank, world, port, n, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from minference_b200.prefill_runner import (LlamaPrefill, LlamaShape, dense_reference_logits,
                                                    zigzag_positions)

        shape = LlamaShape(layers=2, hidden=256, q_heads=2, kv_heads=1, head_dim=128, ffn=512, vocab=500)
        model = LlamaPrefill(shape, "cpu", seed=3, dtype=torch.float32, init_std=0.05)     # same weights on every rank
        ids = torch.randint(0, shape.vocab, (n,), generator=torch.Generator().manual_seed(4))
        pos = zigzag_positions(n, rank, world)
        logits = model.prefill(ids[pos], None, chunk=200, positions=pos,
                               attention=lambda q, k, v, li: ring.ring_attention(q, k, v, n, _dense_window))
        if rank == 0:
            result.put(float((logits - dense_reference_logits(model, ids)).abs().max()))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_whole_model_prefill_on_gloo_ranks():
    """Token-parallel dense parts + ring attention reproduce the unsharded network's last-token logits."""
    world, n = 2, 256 * 4
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_runner_worker, args=(r, world, port, n, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    assert result.get(timeout=10) < 1e-3


# ------------------------------------------------------------------ failures among the ranks (host side only)

def _failing_worker(rank, world, port, n, mode, result):
    """One rank leaves before the exchange (an exception before its send) or brings a shard of another shape: the
    others must come back with an error from their next collective instead of waiting for ever.  No GPU is
    involved; the process group has a short timeout."""
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    outcome = "finished"
    try:
        q = torch.randn(1, 2, n, 16)
        q_loc, k_loc, v_loc = (ring.zigzag_split(t, rank, world) for t in (q, q, q))
        if mode == "raise" and rank == 1:
            raise RuntimeError("rank 1 gives up before the ring")
        if mode == "shape" and rank == 1:
            k_loc, v_loc = k_loc[:, :, :-256].contiguous(), v_loc[:, :, :-256].contiguous()       # a shard that lost a block
        out = ring.ring_attention(q_loc, k_loc, v_loc, n, _dense_window)
        outcome = "finished" if torch.isfinite(out).all() else "non-finite"
    except Exception as e:       # the point of the test: an exception on the host, not a hang
        outcome = "error: " + type(e).__name__
    finally:
        result.put((rank, outcome))
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("mode", ["raise", "shape"])
def test_a_rank_that_fails_before_its_send_ends_the_ring_with_an_error(mode):
    world, n = 2, 256 * 4
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, n, mode, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode is not None, "a rank is still waiting: the failure was not detected"
    outcomes = dict(result.get(timeout=10) for _ in range(world))
    assert outcomes[1].startswith("error")
    assert outcomes[0].startswith("error"), outcomes       # the healthy rank saw the failure as an exception


def test_score_exchange_packs_each_chunk_alone_and_assembles_the_sum():
    """The exchange of the distributed estimator on CPU tensors with a stand-in score pass that *adds* into its
    window (as the kernel's boundary atomics do): every rank's pack must hold each of its chunks alone -- the middle
    rank's two chunks are neighbours and share 63 diagonal offsets -- and the assembly must be the sum over chunks."""
    import torch

    from minference_b200.dist import ring

    for world in (1, 2, 3, 4):
        c = 128
        n = 2 * world * c
        packs = []
        for rank in range(world):
            chunks = ring.owned_chunks(rank, world)

            def score_pass(i, vertical, slash, chunks=chunks):
                ci = chunks[i]
                lo, hi = ring.slash_window(n, ci, c)
                vertical[:, :, ci * c:(ci + 1) * c] = float(ci + 1)
                slash[:, :, lo:hi] += float(ci + 1)

            packs.append(ring.rank_score_pack(score_pass, chunks, n, c, 1, 2, torch.device("cpu")))
        scores = ring.assemble_scores(torch.stack(packs), n, c, world)
        want_v = torch.arange(1, 2 * world + 1, dtype=torch.float32).repeat_interleave(c)
        want_s = torch.zeros(n)
        for ci in range(2 * world):
            lo, hi = ring.slash_window(n, ci, c)
            want_s[lo:hi] += ci + 1
        assert torch.equal(scores[0], want_v.expand(1, 2, n))
        assert torch.equal(scores[1], want_s.expand(1, 2, n))
        # neighbouring windows do overlap, by 63 offsets
        if world > 1:
            (lo0, hi0), (lo1, hi1) = ring.slash_window(n, 0, c), ring.slash_window(n, 1, c)
            assert hi1 - lo0 == 63
