"""Benchmark of the dynamic sparse prefill attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One *step* is one pass of the hot path over one layer of synthetic input: online
vertical/slash index estimation -> index plan -> sparse flash-attention forward, for all
heads.  Default workload: Llama-3-8B layer shape at 131072 tokens (32 query / 8 KV heads,
head_dim 128, bf16, vertical 1000 / slash 6096 / last_q 64 on every head), seeded N(0,1)
Q/K/V with rotary embedding and planted sink columns standing in for real prompts.

Printed JSON (one line, rank 0):
  value        algorithmic TFLOP/s with inputs resident in HBM: 64x64 tiles of the reference
               index set x 4*64*64*128 flop / step time
  e2e          the same through the public operator (minference_prefill_forward) with HOST
               buffers: pinned Q/K/V copied in and the output copied out inside the timed region
  roofline     the attention kernel alone (CUDA events around its launch, same stream)
  cpu_baseline the CPU oracle (port of the reference's torch path) on a bounded sample

With N > 1 ranks (torchrun) the default workload is one 1,048,576-token sequence sharded over the
ranks with the zigzag ring (strong scaling; K/V shards travel by NCCL send/recv); a single-GPU
workload name with N > 1 runs replicas instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FLOP_PER_TILE = 4 * 64 * 64 * 128

WORKLOADS = {
    # name: (tokens, query heads, kv heads, vertical, slash)
    "llama3_8b_128k_vs": (131072, 32, 8, 1000, 6096),
    "llama3_8b_256k_vs": (262144, 32, 8, 1000, 6096),
    "llama3_8b_32k_vs": (32768, 32, 8, 1000, 6096),
    "llama3_8b_8k_vs": (8192, 32, 8, 1000, 6096),
    "llama3_8b_1m_vs": (1048576, 32, 8, 1000, 6096),
}
# per-head mix of the three patterns (seeded): A-shape(128, 4096) / vertical-slash(1000, 6096) / block-sparse top-100
MIXED_WORKLOADS = {
    "qwen25_7b_256k_mixed": (262144, 28, 4, 1000, 6096),
    "llama3_8b_512k_mixed": (524288, 32, 8, 1000, 6096),
}
WORKLOADS.update(MIXED_WORKLOADS)
A_SHAPE = (128, 4096)


def mixed_pattern_table(hq: int, vsize: int, ssize: int, seed: int = 3):
    g = torch.Generator().manual_seed(seed)
    kinds = torch.randint(0, 3, (hq,), generator=g).tolist()
    table = {}
    for h, kd in enumerate(kinds):
        table[str(h)] = (["stream_llm", A_SHAPE[0], A_SHAPE[1], 1.0] if kd == 0 else
                         ["vertical_and_slash", vsize, ssize, 1.0] if kd == 1 else ["block_sparse", 100, 0, 1.0])
    return table, kinds


def a_shape_tiles(n: int, n_init: int, n_local: int) -> int:
    """64x64 tiles the reference's two stages compute for one A-shape head: the tiles that meet the
    window of a row block, plus the sink tiles that hold a key at distance >= n_local from one of
    its rows (sink tiles masked out entirely are not counted)."""
    total = 0
    for m in range((n + 63) // 64):
        lo = max(64 * m - n_local + 1, 0) // 64
        total += m - lo + 1
        if n > n_local:
            for t in range((n_init + 63) // 64):
                if 64 * (m - t) + 63 >= n_local:
                    total += 1
    return total


# with more than one GPU the sequence is sharded over the ranks (zigzag ring); tokens in total
RING_WORKLOADS = {
    "llama3_8b_1m_vs_ring": (1048576, 32, 8, 1000, 6096),
    "llama3_8b_256k_vs_ring": (262144, 32, 8, 1000, 6096),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one sparse_attn_fwd_kernel launch, from one-pass ncu
# captures of the workload itself (the figures and commands are in profiles/); other workloads: not captured
NCU_TRAFFIC_BYTES = {"llama3_8b_128k_vs": 2.92e9 + 1.04e9, "llama3_8b_32k_vs": 0.409e9 + 0.233e9}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"burst": p["bf16_tflops"], "sustained": p["bf16_tflops_sustained"], "hbm": p["hbm_gbs"], "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i] == "Active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------ CPU arm

def cpu_sample(n, hq, hkv, vsize, ssize, seed, budget_s=12.0, max_blocks=4096):
    """Time the CPU oracle on a bounded sample of the workload: one head's estimator over the
    full context, its index conversion, and masked-dense attention for a spread of 64-row
    blocks (evaluated until `budget_s` seconds are used).  Returns (TFLOP/s, description)."""
    import numpy as np
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    q, k, v = make_qkv(n, 1, 1, seed=seed, dtype=torch.float32)
    t0 = time.perf_counter()
    v_idx, s_idx = R.vertical_slash_estimate(q, k, vsize, ssize)
    vs, ss = R.presort_indices(v_idx, s_idx, 1, 1)
    bc, bo, cc, ci = R.convert_vertical_slash_indexes(np.full((1,), n, np.int32), vs.numpy(), ss.numpy(), n)
    t_index = time.perf_counter() - t0
    rows = (n + 63) // 64
    order = [rows - 1 - (i * 7919) % rows for i in range(rows)]      # spread over the context, last block first
    tiles = 0
    done = 0
    t1 = time.perf_counter()
    for m in order[:max_blocks]:
        r0, r1 = m * 64, min(m * 64 + 64, n)
        mask = R.vs_mask_for_rows(bc[0, 0], bo[0, 0], cc[0, 0], ci[0, 0], n, [m])[: r1 - r0, :r1]
        R.masked_attention_rows(q[0, 0, r0:r1], k[0, 0, :r1], v[0, 0, :r1], mask, r0)
        tiles += int(bc[0, 0, m]) + (int(cc[0, 0, m]) + 63) // 64
        done += 1
        if time.perf_counter() - t1 > budget_s:
            break
    t_attn = time.perf_counter() - t1
    # the index work of one head is amortised over all of its row blocks
    t_total = t_attn + t_index * done / rows
    desc = (f"1 of {hq} heads, {done} of {rows} row blocks (64 query rows each, spread over the context) of masked-dense "
            f"fp32 attention + that share of the head's estimator and index conversion; {t_attn + t_index:.1f} s of CPU work")
    return tiles * FLOP_PER_TILE / t_total / 1e12, desc


def run_reference_arm(args, wl):
    n, hq, hkv, vsize, ssize = WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    vals = []
    desc = ""
    t_begin = time.perf_counter()
    for i in range(args.warmup + args.steps):
        per_step_budget = max(2.0, min(12.0, 150.0 / (args.warmup + args.steps)))
        tf, desc = cpu_sample(n, hq, hkv, vsize, ssize, seed=i, budget_s=per_step_budget)
        if i >= args.warmup:
            vals.append(tf)
    value = sum(vals) / len(vals)
    cores = torch.get_num_threads()
    out = {
        "impl": "reference", "metric": "sparse_prefill_attn_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * (time.perf_counter() - t_begin) / (args.warmup + args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl, "tokens": n, "q_heads": hq, "kv_heads": hkv, "vertical": vsize, "slash": ssize},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


# ------------------------------------------------------------------------------ GPU arm

def run_gpu_arm(args, wl):
    import torch.distributed as dist

    from minference_b200 import _cabi
    from minference_b200.cuda import set_status_checks
    from minference_b200.modules.minference_forward import (BLOCK_SPARSE_TOPK, LayerPattern, build_vertical_slash_plan_into,
                                                            minference_prefill_forward, vertical_slash_estimate)
    from minference_b200.ops.block_sparse_flash_attention import build_block_sparse_plan
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import SparsePlan
    from minference_b200.ops.sparse_forward import sparse_attention_forward
    from minference_b200.synthetic import make_qkv

    n, hq, hkv, vsize, ssize = WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _cabi.lib()     # fail loudly right here when the CUDA library is missing
    set_status_checks(False)    # status words are read once after the timed region instead

    q, k, v = make_qkv(n, hq, hkv, seed=rank, dtype=torch.bfloat16, device=dev)
    mixed = wl in MIXED_WORKLOADS
    if mixed:
        table, kinds = mixed_pattern_table(hq, vsize, ssize)
        pat = LayerPattern(table, hq, n, None, dev)
        mixed_plan = SparsePlan(plan=torch.zeros(_cabi.lib().minf_plan_bytes(1, hq, n, pat.cap_v, pat.cap_s), dtype=torch.uint8, device=dev),
                                v_idx=None, cap_v=pat.cap_v, cap_s=pat.cap_s, context_size=n, batch=1, heads=hq,
                                status=_cabi.new_status(dev))
    else:
        table = {str(h): ["vertical_and_slash", vsize, ssize, 1.0] for h in range(hq)}
    cfg = {"attn_forward_config": {"best_pattern": [table]}, "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None}

    ev = lambda: torch.cuda.Event(enable_timing=True)
    attn_events, est_events, plan_events = [], [], []
    tiles_box = {}

    def step_resident(record: bool):
        e0, e1, e2, e3 = ev(), ev(), ev(), ev()
        e0.record()
        if mixed:       # the same calls minference_prefill_forward makes, with events between them
            plan = mixed_plan
            v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q, k, pat.vertical_size, pat.slash_size,
                                                                 cap_v=pat.cap_v, cap_s=pat.cap_s)
            e1.record()
            plan.v_idx = build_vertical_slash_plan_into(plan, v_idx, s_idx, nnz_v, nnz_s)
            build_block_sparse_plan(q, k, BLOCK_SPARSE_TOPK, plan=plan, head_select=pat.block_select)
            e2.record()
            out = sparse_attention_forward(q, k, v, plan, head_mode=pat.head_mode, head_param=pat.head_param)
        else:
            v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q, k, vsize, ssize)
            e1.record()
            plan = build_vertical_slash_plan(v_idx, s_idx, n, nnz_v, nnz_s)
            e2.record()
            out = sparse_attention_forward(q, k, v, plan)
        e3.record()
        if record:
            est_events.append((e0, e1)); plan_events.append((e1, e2)); attn_events.append((e2, e3))
        tiles_box["plan"] = plan
        return out

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_resident(False)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    t0, t1 = ev(), ev()
    t0.record()
    for _ in range(args.steps):
        step_resident(True)
    t1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = t0.elapsed_time(t1)
    plan = tiles_box["plan"]
    status = plan.status.tolist()
    if status[0] != 0 or status[1] != 0:
        raise SystemExit(f"device status {status}: the kernels reported an error")
    tiles = plan.count_tiles()      # A-shape heads have empty (zeroed) plan slots
    if mixed:
        tiles += kinds.count(0) * a_shape_tiles(n, *A_SHAPE)
    attn_ms = sum(a.elapsed_time(b) for a, b in attn_events) / len(attn_events)
    est_ms = sum(a.elapsed_time(b) for a, b in est_events) / len(est_events)
    plan_ms = sum(a.elapsed_time(b) for a, b in plan_events) / len(plan_events)

    # ---- end to end through the public operator with host buffers: every step copies its Q/K/V from pinned host
    # memory and its output back; the copies of neighbouring steps run on their own streams under the compute
    hq_, hk_, hv_ = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq_).pin_memory()
    dbuf = [tuple(torch.empty_like(t) for t in (q, k, v)) for _ in range(2)]
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(steps: int):
        for i in range(steps):
            b = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(freed[b])              # the step that last read this buffer set is done
                for dst, src in zip(dbuf[b], (hq_, hk_, hv_)):
                    dst.copy_(src, non_blocking=True)
                ready[b].record(s_in)
            cur.wait_event(ready[b])
            out = minference_prefill_forward(*dbuf[b], cfg)
            freed[b].record(cur)
            s_out.wait_stream(cur)
            with torch.cuda.stream(s_out):
                ho.copy_(out, non_blocking=True)
            out.record_stream(s_out)
        cur.wait_stream(s_out)

    e2e_steps = max(1, args.steps)
    s_in.wait_stream(cur)
    e2e_run(1)
    barrier()
    s0, s1 = ev(), ev()
    s0.record()
    s_in.wait_stream(cur)
    e2e_run(e2e_steps)
    s1.record()
    barrier()
    e2e_ms = s0.elapsed_time(s1) / e2e_steps
    tiles_box["plan"].status[2:].zero_()        # the mixed workload reuses one status buffer for every launch
    parity_probe = float((ho[0, 0, -1].float() - step_resident(False)[0, 0, -1].float().cpu()).abs().max())
    st = tiles_box["plan"].status.tolist()      # words 2-3: tile equivalents the kernel sent to the tensor pipe in that launch
    issued_tiles = (st[2] & 0xFFFFFFFF) | ((st[3] & 0xFFFFFFFF) << 32)

    times = torch.tensor([total_ms, e2e_ms, attn_ms], dtype=torch.float64, device=dev)
    tile_sum = torch.tensor([float(tiles)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(tile_sum, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms, attn_ms_max = times.tolist()
    all_tiles = tile_sum.item()
    ms_per_step = total_ms / args.steps
    value = all_tiles * FLOP_PER_TILE / (ms_per_step * 1e-3) / 1e12
    e2e_value = all_tiles * FLOP_PER_TILE / (e2e_ms * 1e-3) / 1e12

    if rank == 0:
        peaks = measured_peaks()
        achieved = tiles * FLOP_PER_TILE / (attn_ms * 1e-3) / 1e12
        cpu_tf, cpu_desc = cpu_sample(n, hq, hkv, vsize, ssize, seed=0, budget_s=12.0)
        if mixed:
            cpu_desc = "vertical-slash heads only; " + cpu_desc
        rows = (n + 63) // 64
        out = {
            "metric": "sparse_prefill_attn_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl, "tokens": n, "q_heads": hq, "kv_heads": hkv, "head_dim": 128, "vertical": vsize,
                       "slash": ssize, "last_q": 64, "l2": "inputs_exceed_l2", "replicas": world,
                       **({"head_patterns": {"a_shape": kinds.count(0), "vertical_slash": kinds.count(1),
                                             "block_sparse": kinds.count(2)}} if mixed else {}),
                       "tiles_per_layer": tiles, "fraction_of_causal_tiles": tiles / (hq * rows * (rows + 1) / 2),
                       "dense_equivalent_tflops": 4.0 * (n * n / 2) * 128 * hq * world / (ms_per_step * 1e-3) / 1e12,
                       "ms_estimator": est_ms, "ms_plan": plan_ms, "ms_attention": attn_ms,
                       "issued_over_reference_tiles": issued_tiles / max(tiles, 1)},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in (q, k, v)),
                    "d2h_bytes_per_step": q.numel() * q.element_size(), "max_abs_vs_resident_last_row": parity_probe},
            "gpu_launches": (7 if mixed else 5) * args.steps,
            "roofline": {"bound": "tensor", "kernel": "sparse_attn_fwd_kernel", "achieved": achieved,
                         "peak": peaks["sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["sustained"],
                         "peak_kind": f"bf16 dense sustained, of {peaks['source']}", "frac_of_burst": achieved / peaks["burst"],
                         "traffic": NCU_TRAFFIC_BYTES.get(wl), "traffic_unit": "bytes per launch (ncu)",
                         "algorithmic_bytes": (2 * hq + 2 * hkv) * n * 128 * 2},
            "cpu_baseline": {"value": cpu_tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": cpu_desc},
            "clocks": clocks,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run_ring_arm(args, wl):
    """N > 1: one sequence sharded over the ranks, zigzag ring attention (strong scaling)."""
    import torch.distributed as dist

    from minference_b200 import _cabi
    from minference_b200.cuda import set_status_checks
    from minference_b200.dist import ring
    from minference_b200.synthetic import make_qkv_ranges

    n, hq, hkv, vsize, ssize = RING_WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    _cabi.lib()
    set_status_checks(False)
    c = ring.chunk_size(n, world)
    ranges = [(ch * c, c) for ch in ring.owned_chunks(rank, world)]
    q, k, v = make_qkv_ranges(n, ranges, hq, hkv, seed=0, dtype=torch.bfloat16, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    stats = {"count_tiles": True}
    ring.ring_vertical_slash_attention(q, k, v, n, vsize, ssize, stats=stats)       # also counts the tiles once
    tiles_local = stats["tiles"]
    for _ in range(max(args.warmup - 1, 0)):
        ring.ring_vertical_slash_attention(q, k, v, n, vsize, ssize)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    stats = {}
    t0, t1 = ev(), ev()
    t0.record()
    for _ in range(args.steps):
        ring.ring_vertical_slash_attention(q, k, v, n, vsize, ssize, stats=stats)
    t1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = t0.elapsed_time(t1)
    attn_ms = sum(a.elapsed_time(b) for a, b in stats["attn_events"]) / args.steps
    launches = len(stats["attn_events"]) // args.steps

    hq_, hk_, hv_ = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq_).pin_memory()
    # host copies of neighbouring steps run on their own streams under the ring (as in the single-GPU arm)
    dbuf = [tuple(torch.empty_like(t) for t in (q, k, v)) for _ in range(2)]
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(steps: int):
        for i in range(steps):
            b = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(freed[b])
                for dst, src in zip(dbuf[b], (hq_, hk_, hv_)):
                    dst.copy_(src, non_blocking=True)
                ready[b].record(s_in)
            cur.wait_event(ready[b])
            out = ring.ring_vertical_slash_attention(*dbuf[b], n, vsize, ssize)
            freed[b].record(cur)
            s_out.wait_stream(cur)
            with torch.cuda.stream(s_out):
                ho.copy_(out, non_blocking=True)
            out.record_stream(s_out)
        cur.wait_stream(s_out)

    e2e_steps = max(1, min(args.steps, 3))
    s_in.wait_stream(cur)
    e2e_run(1)
    barrier()
    s0, s1 = ev(), ev()
    s0.record()
    s_in.wait_stream(cur)
    e2e_run(e2e_steps)
    s1.record()
    barrier()
    e2e_ms = s0.elapsed_time(s1) / e2e_steps

    times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    sums = torch.tensor([float(tiles_local)], dtype=torch.float64, device=dev)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms = times.tolist()
    all_tiles = sums.item()
    ms_per_step = total_ms / args.steps
    if rank == 0:
        peaks = measured_peaks()
        achieved = tiles_local * FLOP_PER_TILE / (attn_ms * 1e-3) / 1e12
        rows = n // 64
        out = {
            "metric": "sparse_prefill_attn_tflops", "value": all_tiles * FLOP_PER_TILE / (ms_per_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl, "tokens": n, "tokens_per_gpu": n // world, "q_heads": hq, "kv_heads": hkv, "head_dim": 128,
                       "vertical": vsize, "slash": ssize, "last_q": 64, "l2": "inputs_exceed_l2",
                       "parallelism": f"zigzag ring over {world} ranks, K/V shards by NCCL send/recv",
                       "one_gpu_reference": "the default 1-GPU run is a different workload (131072 tokens, 98 % of the causal "
                                            "tiles); this sequence on one GPU is `--workload " + wl.replace("_ring", "") + "`",
                       "tiles_per_layer": int(all_tiles), "fraction_of_causal_tiles": all_tiles / (hq * rows * (rows + 1) / 2),
                       "dense_equivalent_tflops": 4.0 * (n * n / 2) * 128 * hq / (ms_per_step * 1e-3) / 1e12,
                       "ms_attention_kernels_rank0": attn_ms},
            "e2e": {"value": all_tiles * FLOP_PER_TILE / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": world * sum(t.numel() * t.element_size() for t in (q, k, v)),
                    "d2h_bytes_per_step": world * q.numel() * q.element_size()},
            "gpu_launches": (launches + 2 * 2 + 1 + 2) * args.steps * world,
            "roofline": {"bound": "tensor", "kernel": "sparse_attn_fwd_kernel", "achieved": achieved, "peak": peaks["sustained"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["sustained"],
                         "peak_kind": f"bf16 dense sustained per GPU, of {peaks['source']}; rank 0, summed over its {launches} launches per step",
                         "frac_of_burst": achieved / peaks["burst"], "traffic": None},
            "cpu_baseline": None,
            "clocks": clocks,
        }
        print(json.dumps(out))
    dist.destroy_process_group()


# ------------------------------------------------------------------------------ whole-model prefill (TTFT)

TTFT_WORKLOADS = {
    # name: (tokens, layers) of the Llama-3-8B architecture with seeded random weights and seeded per-head patterns
    "llama3_8b_512k_ttft": (524288, 32),
    "llama3_8b_128k_ttft": (131072, 32),
    "llama3_8b_32k_ttft_4layers": (32768, 4),
    "llama3_8b_1m_ttft": (1048576, 32),
    # vertical-slash on every head (the 1M-token ring configuration extended to the whole model)
    "llama3_8b_1m_ttft_vs": (1048576, 32),
    "llama3_8b_256k_ttft_4layers": (262144, 4),
    "llama3_8b_256k_ttft_vs_4layers": (262144, 4),
}


def run_ttft_arm(args, wl):
    """One ``use_cache=False``-style forward of the whole network over one long prompt; a step is
    one prefill, timed with CUDA events, token ids copied from pinned host memory inside the timed
    region and the last token's logits copied back.  Under torchrun the prompt is sharded over the
    ranks in zigzag chunks: dense parts are token-parallel, attention is the vertical-slash ring."""
    import torch.distributed as dist

    from minference_b200 import _cabi
    from minference_b200.cuda import set_status_checks
    from minference_b200.dist import ring
    from minference_b200.prefill_runner import LlamaPrefill, LlamaShape, seeded_pattern_tables, zigzag_positions

    n, layers = TTFT_WORKLOADS[wl]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _cabi.lib()
    set_status_checks(False)
    shape = LlamaShape(layers=layers)
    model = LlamaPrefill(shape, dev, seed=0)            # same seed: identical weights on every rank
    vs_only = wl.endswith("_vs") or "_vs_" in wl
    tables = seeded_pattern_tables(shape, seed=0, kinds=("vertical_and_slash",) if vs_only else
                                   ("stream_llm", "vertical_and_slash", "block_sparse"))
    cfg = {"starting_layer": 0, "best_pattern": tables}
    ids_all = torch.randint(0, shape.vocab, (n,), generator=torch.Generator().manual_seed(0))
    positions = zigzag_positions(n, rank, world, dev) if world > 1 else None
    ids_host = (ids_all[positions.cpu()] if world > 1 else ids_all).pin_memory()
    logits_host = torch.empty(shape.vocab, dtype=torch.float32).pin_memory()
    attention = None
    if world > 1:       # with N > 1 ranks the prompt is sequence-sharded (zigzag chunks) and attention is the ring
        from minference_b200.modules.minference_forward import LayerPattern

        patterns = [LayerPattern(t, shape.q_heads, n, None, dev) for t in tables]
        attention = lambda q, k, v, li: ring.ring_prefill_attention(q, k, v, n, patterns[li])
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step():
        ids = ids_host.to(dev, non_blocking=True)
        logits = model.prefill(ids, cfg, positions=positions, attention=attention)
        if rank == 0:       # the prompt's last token is rank 0's last token
            logits_host.copy_(logits, non_blocking=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    t0, t1 = ev(), ev()
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ttft_s = t.item() / args.steps / 1e3
    if rank == 0:
        kinds = [e[0] for layer in tables for e in layer.values()]
        dense_flop = 2.0 * n * layers * (shape.hidden * (shape.q_heads + 2 * shape.kv_heads) * 128 + shape.q_heads * 128 * shape.hidden
                                         + 3 * shape.hidden * shape.ffn)
        out = {
            "metric": "ttft_s", "value": ttft_s, "unit": "s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ttft_s * 1e3, "higher_is_better": False, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl, "tokens": n, "tokens_per_gpu": n // world, "layers": layers, "hidden": shape.hidden,
                       "q_heads": shape.q_heads, "kv_heads": shape.kv_heads, "ffn": shape.ffn, "vocab": shape.vocab,
                       "weights": "random init, seed 0",
                       "head_patterns": {kd: kinds.count(kd) for kd in sorted(set(kinds))},
                       "parallelism": f"zigzag sequence split over {world} ranks, ring attention" if world > 1 else "one GPU",
                       "dense_gemm_pflop": dense_flop / 1e15, "dense_parts": "torch.matmul (cuBLAS), chunked over 16384 tokens",
                       "tokens_per_s": n / ttft_s, "finite_logits": bool(torch.isfinite(logits_host).all())},
            "e2e": {"value": ttft_s, "unit": "s", "h2d_bytes_per_step": world * ids_host.numel() * ids_host.element_size(),
                    "d2h_bytes_per_step": logits_host.numel() * 4},
            "gpu_launches": None, "roofline": None, "cpu_baseline": None, "clocks": clocks,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + sorted(RING_WORKLOADS) + sorted(TTFT_WORKLOADS))
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload is None:
        args.workload = "llama3_8b_128k_vs" if world == 1 else "llama3_8b_1m_vs_ring"
    if args.workload in TTFT_WORKLOADS:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the whole-model prefill has no CPU arm; the attention workloads do"}))
            return
        return run_ttft_arm(args, args.workload)
    if args.impl == "reference":
        # the CPU arm times the same per-tile work; for a ring workload it uses the single-GPU shape of that length
        wl = args.workload if args.workload in WORKLOADS else args.workload.replace("_ring", "")
        run_reference_arm(args, wl)
    elif args.workload in RING_WORKLOADS:
        if world < 2:
            raise SystemExit("ring workloads need torchrun with two or more ranks")
        run_ring_arm(args, args.workload)
    else:
        run_gpu_arm(args, args.workload)


if __name__ == "__main__":
    main()
