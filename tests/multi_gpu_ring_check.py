"""Launched by torchrun with one process per GPU (see tests/test_gpu_ring.py and bench.py):
runs the sequence-sharded vertical-slash attention, including the distributed index estimation,
and compares with the whole-sequence kernels on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from minference_b200.dist import ring
    from minference_b200.modules.minference_forward import vertical_slash_estimate
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    n, hq, hkv = 256 * 2 * world * 8, 8, 2
    q, k, v = make_qkv(n, hq, hkv, seed=3, dtype=torch.bfloat16)          # same tensors on every rank (CPU generator)
    q_loc, k_loc, v_loc = (ring.zigzag_split(t, rank, world).to(dev) for t in (q, k, v))
    stats = {}
    out_loc = ring.ring_vertical_slash_attention(q_loc, k_loc, v_loc, n, 200, 600, stats=stats)
    gathered = [torch.empty_like(out_loc) for _ in range(world)]
    dist.all_gather(gathered, out_loc)
    ok = True
    if rank == 0:
        from tests.test_gpu_ring import _one_rounding_apart

        merged = ring.zigzag_merge(gathered, world).float()
        dq, dk, dv = q.to(dev), k.to(dev), v.to(dev)
        v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(dq, dk, 200, 600)
        # chunks are multiples of the 2048-key statistics block: the distributed estimator returns the very lists
        # of the whole-sequence one, whatever the number of ranks
        same_lists = torch.equal(stats["indices"][0], v_idx) and torch.equal(stats["indices"][1], s_idx)
        full = sparse_attention_forward(dq, dk, dv, build_vertical_slash_plan(v_idx, s_idx, n, nnz_v, nnz_s)).float()
        d = (merged - full).abs()
        close = _one_rounding_apart(merged, full)       # merged in fp32 inside the kernel and rounded once
        print(f"ring vs whole-sequence on {world} ranks, {n} tokens: index lists identical {same_lists}; "
              f"max {d.max().item():.3e} mean {d.mean().item():.3e}; at most one bf16 step apart {close}")
        ok = same_lists and close and d.max().item() < 1.5e-2 and torch.isfinite(merged).all().item()
    # per-head pattern table (vertical-slash and A-shape heads) through the ring against the single-GPU operator
    from minference_b200.modules.minference_forward import LayerPattern, minference_prefill_forward

    table = {str(h): (["vertical_and_slash", 200, 600, 1.0] if h % 3 == 0 else
                      ["stream_llm", 64, 1024, 1.0] if h % 3 == 1 else ["block_sparse", 100, 0, 1.0]) for h in range(hq)}
    pat = LayerPattern(table, hq, n, None, dev)
    mixed_loc = ring.ring_prefill_attention(q_loc, k_loc, v_loc, n, pat, block_sparse_top_k=20)
    gathered = [torch.empty_like(mixed_loc) for _ in range(world)]
    dist.all_gather(gathered, mixed_loc)
    if rank == 0:
        merged = ring.zigzag_merge(gathered, world).float()
        import minference_b200.modules.minference_forward as mf

        mf.BLOCK_SPARSE_TOPK = 20          # few enough blocks that the selection matters at this length
        single = minference_prefill_forward(q.to(dev), k.to(dev), v.to(dev), {
            "attn_forward_config": {"best_pattern": [table]}, "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None}).float()
        d = (merged - single).abs()
        print(f"mixed ring vs single GPU: max {d.max().item():.3e} mean {d.mean().item():.3e}; "
              f"A-shape heads max {d[:, 1::3].max().item():.3e}, block-sparse heads max {d[:, 2::3].max().item():.3e}")
        # A-shape and block-sparse heads have no estimator noise: same index set, two bf16 roundings apart
        ok = ok and d.mean().item() < 2e-3 and d[:, 1::3].max().item() < 1.5e-2 and d[:, 2::3].max().item() < 1.5e-2 \
            and torch.isfinite(merged).all().item()
    # whole network, sequence-sharded, against the same network on one GPU (both through the CUDA kernels)
    from minference_b200.prefill_runner import LlamaPrefill, LlamaShape, seeded_pattern_tables, zigzag_positions

    shape = LlamaShape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=1000)
    model = LlamaPrefill(shape, dev, seed=1, init_std=0.05)
    ids = torch.randint(0, shape.vocab, (n,), generator=torch.Generator().manual_seed(2))
    pos = zigzag_positions(n, rank, world, dev)
    logits = model.prefill(ids[pos.cpu()], None, chunk=1024, positions=pos,
                           attention=lambda q_, k_, v_, li: ring.ring_vertical_slash_attention(q_, k_, v_, n, 200, 600))
    if rank == 0:
        tables = seeded_pattern_tables(shape, seed=0, vertical=200, slash=600, kinds=("vertical_and_slash",))
        single = model.prefill(ids, {"starting_layer": 0, "best_pattern": tables}, chunk=1024)
        dl = (logits - single).abs().max().item()
        print(f"sharded vs single-GPU logits: max {dl:.3e} (scale {single.abs().max().item():.3e})")
        ok = ok and dl <= 3e-2 * single.abs().max().item() + 1e-3 and torch.isfinite(logits).all().item()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, src=0)
    dist.destroy_process_group()
    if flag.item() != 1:
        sys.exit(1)
    if rank == 0:
        print("RING_OK")


if __name__ == "__main__":
    main()
