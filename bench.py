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

  detail       what else was measured: tiles, stage times, issued over reference tiles, the parity probe of this
               very output (sampled row blocks of every head against fp32 masked-dense attention over the
               identical index set; the run exits non-zero above 2e-2 max / 2e-3 mean), and for the default
               workload the band index set at the same length and the 1,048,576-token layer on this one GPU
               (the anchor of the ring lines; --no-extras leaves these out)

Workload families (--workload): *_vs (index set estimated online), *_vs_local (prescribed band), *_vs_scattered
(prescribed scattered diagonals), *_mixed (per-head pattern table), *_flexprefill (adaptive block budgets), *_ttft*
(whole-model prefill, metric ttft_s) and *_ring (N > 1).

With N > 1 ranks (torchrun) the default workload is one 1,048,576-token sequence sharded over the
ranks with the zigzag ring (strong scaling; K/V shards travel by NCCL send/recv; the line carries ring_parity,
the band twin and issued over reference tiles); a single-GPU workload name with N > 1 runs replicas instead.
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
# The same layers with a prescribed band index set instead of the estimated one: slash offsets 0..6095 (the
# diagonals next to the main one) and 1000 seeded vertical columns per head, handed to
# vertical_slash_sparse_attention (no estimator in the step).  Seeded N(0,1) data has a nearly flat
# slash score, so its estimated diagonals scatter over the whole context; heads of real models pick bands.
LOCAL_WORKLOADS = {name + "_local": spec for name, spec in WORKLOADS.items()}
# ... and with a prescribed scattered set: the 100 nearest diagonals + diagonals drawn uniformly from the whole
# context (what the estimator returns on structureless data at a million tokens), at any length
# (the number of drawn diagonals is scaled with the length so that their density is that of 6096 in a million)
SCATTERED_WORKLOADS = {name + "_scattered": (n, hq, hkv, v, 100 + round((s - 100) * n / 1048576))
                       for name, (n, hq, hkv, v, s) in WORKLOADS.items()}
WORKLOADS.update(LOCAL_WORKLOADS)
WORKLOADS.update(SCATTERED_WORKLOADS)
LOCAL_WORKLOADS.update(SCATTERED_WORKLOADS)       # both are "prescribed index set" workloads
# per-head mix of the three patterns (seeded): A-shape(128, 4096) / vertical-slash(1000, 6096) / block-sparse top-100
MIXED_WORKLOADS = {
    "qwen25_7b_256k_mixed": (262144, 28, 4, 1000, 6096),
    "llama3_8b_512k_mixed": (524288, 32, 8, 1000, 6096),
}
WORKLOADS.update(MIXED_WORKLOADS)
A_SHAPE = (128, 4096)
# FlexPrefill layers (adaptive block budgets from the last 128 queries): the reference's defaults, and a variant with
# the Jensen-Shannon fallback off and the budgets capped at 8192 tokens, which gives a sparse vertical/slash block set
FLEX_WORKLOADS = {
    "llama3_8b_128k_flexprefill": (131072, 32, 8, 0, 0),
    "llama3_8b_128k_flexprefill_b8k": (131072, 32, 8, 0, 0),
}
FLEX_PARAMS = {
    "llama3_8b_128k_flexprefill": {"gamma": 0.9, "tau": 0.1, "block_size": 128},
    "llama3_8b_128k_flexprefill_b8k": {"gamma": 0.9, "tau": 0.0, "max_budget": 8192, "block_size": 128},
}
WORKLOADS.update(FLEX_WORKLOADS)


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
RING_WORKLOADS.update({name.replace("_ring", "_local_ring"): spec for name, spec in RING_WORKLOADS.items()})


def workload_config(wl: str, world: int) -> dict:
    """What is computed, the same in both arms (measured figures go into ``detail``)."""
    ring = wl in RING_WORKLOADS
    n, hq, hkv, vsize, ssize = (RING_WORKLOADS if ring else WORKLOADS)[wl]
    cfg = {"workload": wl, "tokens": n, "q_heads": hq, "kv_heads": hkv, "head_dim": 128, "vertical": vsize, "slash": ssize,
           "last_q": 64, "l2": "inputs_exceed_l2",
           "index_set": "band: slash offsets 0..s-1 + seeded vertical columns, given to the operator" if "_local" in wl
           else "scattered: 100 nearest + uniformly drawn diagonals and columns, given to the operator" if "_scattered" in wl
           else f"FlexPrefill block set, estimated online from the last 128 queries, {FLEX_PARAMS[wl]}" if wl in FLEX_PARAMS
           else "estimated online from the last 64 queries"}
    if ring:
        cfg["parallelism"] = f"one sequence, zigzag ring over {world} ranks, K/V shards by NCCL send/recv"
    else:
        cfg["replicas"] = world
    return cfg


# dram__bytes_read.sum + dram__bytes_write.sum of one sparse_attn_fwd_kernel launch, from one-pass ncu
# captures of the workload itself (the figures and commands are in profiles/); other workloads: not captured
NCU_TRAFFIC_BYTES = {"llama3_8b_128k_vs": 2.991e9 + 1.038e9, "llama3_8b_32k_vs": 0.409e9 + 0.233e9}


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

def cpu_sample(n, hq, hkv, vsize, ssize, seed, budget_s=12.0, max_blocks=4096, local=False):
    """Time the CPU oracle on a bounded sample of the workload: one head's estimator over the
    full context (skipped for a prescribed band index set), its index conversion, and masked-dense
    attention for a spread of 64-row blocks (evaluated until `budget_s` seconds are used).
    Returns (TFLOP/s, description)."""
    import numpy as np
    from minference_b200.synthetic import local_vs_indices, make_qkv
    from oracle import reference_math as R

    q, k, v = make_qkv(n, 1, 1, seed=seed, dtype=torch.float32)
    t0 = time.perf_counter()
    if local:
        v_idx, s_idx = local_vs_indices(n, 1, vsize, ssize, seed=seed)
    else:
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
            f"fp32 attention + that share of the head's {'index conversion' if local else 'estimator and index conversion'}; "
            f"{t_attn + t_index:.1f} s of CPU work")
    return tiles * FLOP_PER_TILE / t_total / 1e12, desc


def run_reference_arm(args, wl):
    # the CPU arm times the same per-tile work; for a ring workload it uses the layer shape of that length
    n, hq, hkv, vsize, ssize = (RING_WORKLOADS if wl in RING_WORKLOADS else WORKLOADS)[wl]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    if wl in FLEX_PARAMS:
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm times the vertical-slash, band and mixed workloads; "
                          "FlexPrefill workloads carry no CPU baseline"}))
        return
    torch.set_num_threads(os.cpu_count() or 1)
    vals = []
    desc = ""
    t_begin = time.perf_counter()
    for i in range(args.warmup + args.steps):
        per_step_budget = max(2.0, min(12.0, 150.0 / (args.warmup + args.steps)))
        tf, desc = cpu_sample(n, hq, hkv, vsize, ssize, seed=i, budget_s=per_step_budget, local="_local" in wl)
        if i >= args.warmup:
            vals.append(tf)
    value = sum(vals) / len(vals)
    cores = torch.get_num_threads()
    out = {
        "impl": "reference", "metric": "sparse_prefill_attn_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * (time.perf_counter() - t_begin) / (args.warmup + args.steps),
        "higher_is_better": True, "scaling": "strong" if wl in RING_WORKLOADS else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(wl, world),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


# ------------------------------------------------------------------------------ GPU arm

# kernels of this library per step: estimator (2 score passes, combine, 3 histogram levels, count, write) = 8,
# plan 1, attention 1; the mixed workload adds the block-sparse pooling and selection
LAUNCHES_VS, LAUNCHES_BAND, LAUNCHES_MIXED = 10, 2, 12
LAUNCHES_FLEX = 8          # two groups of 64 queries x (pass 1, combine, pass 2), plan from the block mask, attention


def layer_runner(n, hq, hkv, vsize, ssize, dev, seed, kind, q=None, k=None, v=None, flex=None):
    """Returns ``step(record) -> out`` for one layer workload with inputs resident in HBM, the event lists it
    fills and a box holding the last plan.  kind: "vs" (estimator -> plan -> attention), "band"
    (prescribed band index set -> plan -> attention) or "mixed" (per-head pattern table)."""
    from minference_b200 import _cabi
    from minference_b200.modules.flexprefill import active_block_mask, build_block_mask_plan
    from minference_b200.modules.minference_forward import (BLOCK_SPARSE_TOPK, LayerPattern, build_vertical_slash_plan_into,
                                                            vertical_slash_estimate)
    from minference_b200.ops.block_sparse_flash_attention import build_block_sparse_plan
    from minference_b200.ops.pit_sparse_flash_attention_v2 import build_vertical_slash_plan
    from minference_b200.ops.sparse_forward import SparsePlan, sparse_attention_forward
    from minference_b200.synthetic import local_vs_indices, make_qkv, make_qkv_ranges, scattered_vs_indices

    if q is None and seed == 0 and any(spec[0] == n for spec in RING_WORKLOADS.values()):
        # the sequence the ring workloads shard (the generator keyed by fixed blocks): the one-GPU anchor of those
        # lines computes on the same values, so tiles_per_layer can be compared across GPU counts
        q, k, v = make_qkv_ranges(n, [(0, n)], hq, hkv, seed=0, dtype=torch.bfloat16, device=dev)
    elif q is None:
        q, k, v = make_qkv(n, hq, hkv, seed=seed, dtype=torch.bfloat16, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    events = {"est": [], "plan": [], "attn": []}
    box = {"kinds": None}
    if kind == "mixed":
        table, kinds = mixed_pattern_table(hq, vsize, ssize)
        box["kinds"], box["table"] = kinds, table
        pat = LayerPattern(table, hq, n, None, dev)
        mixed_plan = SparsePlan(plan=torch.zeros(_cabi.lib().minf_plan_bytes(1, hq, n, pat.cap_v, pat.cap_s), dtype=torch.uint8, device=dev),
                                v_idx=None, cap_v=pat.cap_v, cap_s=pat.cap_s, context_size=n, batch=1, heads=hq,
                                status=_cabi.new_status(dev))
    elif kind in ("band", "scattered"):
        bv, bs = (scattered_vs_indices if kind == "scattered" else local_vs_indices)(n, hq, vsize, ssize, seed=seed, device=dev)
        kind = "band"
        box["indices"] = (bv.contiguous(), bs.contiguous())

    def step(record: bool):
        e0, e1, e2, e3 = ev(), ev(), ev(), ev()
        e0.record()
        if kind == "mixed":     # the same calls minference_prefill_forward makes, with events between them
            plan = mixed_plan
            v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q, k, pat.vertical_size, pat.slash_size,
                                                                 cap_v=pat.cap_v, cap_s=pat.cap_s)
            e1.record()
            plan.v_idx = build_vertical_slash_plan_into(plan, v_idx, s_idx, nnz_v, nnz_s)
            build_block_sparse_plan(q, k, BLOCK_SPARSE_TOPK, plan=plan, head_select=pat.block_select)
            e2.record()
            out = sparse_attention_forward(q, k, v, plan, head_mode=pat.head_mode, head_param=pat.head_param)
        elif kind == "band":
            e1.record()
            plan = build_vertical_slash_plan(*box["indices"], n)
            e2.record()
            out = sparse_attention_forward(q, k, v, plan)
        elif kind == "flex":     # the calls flexprefill_forward makes
            bs = flex.get("block_size", 128)
            box["block_mask"] = active_block_mask(q, k, bs, flex["gamma"], -(-flex.get("min_budget", 1) // bs),
                                                  -(-flex.get("max_budget", 2147483647) // bs), flex["tau"])
            e1.record()
            plan = build_block_mask_plan(box["block_mask"], n, bs)
            e2.record()
            out = sparse_attention_forward(q, k, v, plan)
        else:
            v_idx, s_idx, nnz_v, nnz_s = vertical_slash_estimate(q, k, vsize, ssize)
            e1.record()
            plan = build_vertical_slash_plan(v_idx, s_idx, n, nnz_v, nnz_s)
            e2.record()
            out = sparse_attention_forward(q, k, v, plan)
        e3.record()
        if record:
            events["est"].append((e0, e1)); events["plan"].append((e1, e2)); events["attn"].append((e2, e3))
        box["plan"] = plan
        return out

    return step, events, box, (q, k, v)


def issued_tiles_of(status) -> int:
    st = status.tolist()
    return (st[2] & 0xFFFFFFFF) | ((st[3] & 0xFFFFFFFF) << 32)


def side_measurement(name, dev, steps=2, warmup=1):
    """A short measurement of another single-GPU workload, reported inside ``detail`` of the headline line."""
    n, hq, hkv, vsize, ssize = WORKLOADS[name]
    kind = "scattered" if name in SCATTERED_WORKLOADS else "band" if name in LOCAL_WORKLOADS else "vs"
    step, events, box, _ = layer_runner(n, hq, hkv, vsize, ssize, dev, 0, kind)
    for _ in range(warmup):
        step(False)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step(True)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    plan = box["plan"]
    st = plan.status.tolist()
    if st[0] or st[1]:
        raise SystemExit(f"{name}: device status {st}")
    tiles = plan.count_tiles()
    step(False)
    torch.cuda.synchronize()
    issued = issued_tiles_of(box["plan"].status)          # the plan (and status words) of that one step
    attn_ms = sum(a.elapsed_time(b) for a, b in events["attn"]) / steps
    peaks = measured_peaks()
    rows = (n + 63) // 64
    return {"workload": name, "tokens": n, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "value": tiles * FLOP_PER_TILE / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "tiles_per_layer": tiles,
            "fraction_of_causal_tiles": tiles / (hq * rows * (rows + 1) / 2), "ms_attention": attn_ms,
            "attention_frac_of_sustained_peak": tiles * FLOP_PER_TILE / (attn_ms * 1e-3) / 1e12 / peaks["sustained"],
            "issued_over_reference_tiles": issued / max(tiles, 1)}


def run_gpu_arm(args, wl):
    import torch.distributed as dist

    from minference_b200 import _cabi
    from minference_b200.cuda import set_status_checks
    from minference_b200.modules.flexprefill import flexprefill_forward
    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention

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

    mixed = wl in MIXED_WORKLOADS
    band = wl in LOCAL_WORKLOADS
    flex = FLEX_PARAMS.get(wl)
    step_resident, events, box, (q, k, v) = layer_runner(n, hq, hkv, vsize, ssize, dev, rank,
                                                         "mixed" if mixed else "scattered" if wl in SCATTERED_WORKLOADS
                                                         else "band" if band else "flex" if flex else "vs", flex=flex)
    kinds = box["kinds"]
    table = box["table"] if mixed else {str(h): ["vertical_and_slash", vsize, ssize, 1.0] for h in range(hq)}
    cfg = {"attn_forward_config": {"best_pattern": [table]}, "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None}
    ev = lambda: torch.cuda.Event(enable_timing=True)

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
    plan = box["plan"]
    status = plan.status.tolist()
    if status[0] != 0 or status[1] != 0:
        raise SystemExit(f"device status {status}: the kernels reported an error")
    tiles = plan.count_tiles()      # A-shape heads have empty (zeroed) plan slots
    if mixed:
        tiles += kinds.count(0) * a_shape_tiles(n, *A_SHAPE)
    mean_ms = lambda evs: sum(a.elapsed_time(b) for a, b in evs) / len(evs)
    attn_ms, est_ms, plan_ms = mean_ms(events["attn"]), mean_ms(events["est"]), mean_ms(events["plan"])

    # ---- end to end through the public operator with host buffers: every step copies its Q/K/V from pinned host
    # memory and its output back; the copies of neighbouring steps run on their own streams under the compute
    hq_, hk_, hv_ = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty_like(hq_).pin_memory()
    dbuf = [tuple(torch.empty_like(t) for t in (q, k, v)) for _ in range(2)]
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]

    def public_call(qd, kd, vd):
        if flex:
            return flexprefill_forward(qd, kd, vd, {"attn_forward_config": flex})
        if band:
            return vertical_slash_sparse_attention(qd, kd, vd, *box["indices"])
        return minference_prefill_forward(qd, kd, vd, cfg)

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
            out = public_call(*dbuf[b])
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
    box["plan"].status[2:].zero_()        # the mixed workload reuses one status buffer for every launch
    out_res = step_resident(False)
    parity_probe = float((ho[0, 0, -1].float() - out_res[0, 0, -1].float().cpu()).abs().max())
    issued_tiles = issued_tiles_of(box["plan"].status)   # tile equivalents the kernel sent to the tensor pipe in that launch

    # ---- parity of this very output at the benchmark's size: sampled row blocks of every head against an fp32
    # masked-dense recomputation over the identical index set (vertical-slash workloads)
    parity = None
    if flex:
        parity = flex_parity_probe(q, k, v, out_res, box["block_mask"], flex.get("block_size", 128), n, hq, hkv)
    elif not mixed:
        parity = vs_parity_probe(q, k, v, out_res, box["plan"], n, hq, hkv, dev)
    if parity is not None and (parity["max_abs"] > 2e-2 or parity["mean_abs"] > 2e-3):
        raise SystemExit(f"parity probe failed: {parity}")

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
        rows = (n + 63) // 64
        detail = {"tiles_per_layer": tiles, "fraction_of_causal_tiles": tiles / (hq * rows * (rows + 1) / 2),
                  "dense_equivalent_tflops": 4.0 * (n * n / 2) * 128 * hq * world / (ms_per_step * 1e-3) / 1e12,
                  "ms_estimator": est_ms, "ms_plan": plan_ms, "ms_attention": attn_ms,
                  "issued_over_reference_tiles": issued_tiles / max(tiles, 1), "parity_vs_fp32_masked_dense": parity}
        if mixed:
            detail["head_patterns"] = {"a_shape": kinds.count(0), "vertical_slash": kinds.count(1), "block_sparse": kinds.count(2)}
        if world == 1 and wl == "llama3_8b_128k_vs" and not args.no_extras:
            # beside the headline: the band index set at this length, and the 1,048,576-token layer (the sequence the
            # ring workload shards over 2/4/8 GPUs) on this one GPU with the estimated and the band index set
            del q, k, v, out_res, dbuf, hq_, hk_, hv_, ho
            box.clear()
            torch.cuda.empty_cache()
            detail["band_index_set"] = side_measurement("llama3_8b_128k_vs_local", dev, steps=3, warmup=2)
            torch.cuda.empty_cache()
            detail["one_gpu_1m"] = side_measurement("llama3_8b_1m_vs", dev, steps=2, warmup=1)
            torch.cuda.empty_cache()
            detail["one_gpu_1m_band"] = side_measurement("llama3_8b_1m_vs_local", dev, steps=3, warmup=3)   # short steps: settle the allocator first
        if flex:
            detail["blocks_selected_of_causal"] = float(box["block_mask"].sum().item()) / (hq * (n // 128) * (n // 128 + 1) / 2)
            cpu_tf, cpu_desc = None, "not timed for this workload (the default workload carries the CPU baseline)"
        else:
            cpu_tf, cpu_desc = cpu_sample(n, hq, hkv, vsize, ssize, seed=0, budget_s=12.0, local=band)
        if mixed:
            cpu_desc = "vertical-slash heads only; " + cpu_desc
        out = {
            "metric": "sparse_prefill_attn_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(wl, world), "detail": detail,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (hq + 2 * hkv) * n * 128 * 2,
                    "d2h_bytes_per_step": hq * n * 128 * 2, "max_abs_vs_resident_last_row": parity_probe},
            "gpu_launches": (LAUNCHES_MIXED if mixed else LAUNCHES_BAND if band else LAUNCHES_FLEX if flex else LAUNCHES_VS) * args.steps,
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


def sample_row_blocks(first: int, count: int, want: int):
    """``want`` row blocks of [first, first + count) including the first two and the last two."""
    want = max(4, min(want, count))
    picks = {first, first + 1, first + count - 2, first + count - 1}
    i = 0
    while len(picks) < want:
        picks.add(first + (i * 7919 + 13) % count)
        i += 1
    return sorted(p for p in picks if first <= p < first + count)


def vs_parity_probe(q, k, v, out, plan, n, hq, hkv, dev, blocks_per_head=4):
    """Kernel output against the fp32 masked-dense recomputation over the identical index set: reference-format
    tables are built from the plan's index lists one head at a time (they are 0.5 GB per head at 1M tokens)."""
    from minference_b200.checks import compare_row_blocks
    from minference_b200.cuda import convert_vertical_slash_indexes

    rows = (n + 63) // 64
    group = hq // hkv
    v_idx = plan.v_idx
    worst, mean_sum, cnt = 0.0, 0.0, 0
    s_idx = plan_slash_lists(plan)
    seqlens = torch.tensor([n], dtype=torch.int32, device=dev)
    for h in range(hq):
        bc, bo, cc, ci = convert_vertical_slash_indexes(seqlens, v_idx[:, h:h + 1].contiguous(), s_idx[:, h:h + 1].contiguous(), n)
        picks = sample_row_blocks(0, rows, blocks_per_head) if rows >= 4 else list(range(rows))
        picks = sorted(set(picks) | {(h * 131 + 7) % rows})
        mx, mean = compare_row_blocks(lambda m: out[0, h, 64 * m:64 * m + 64], lambda m: q[0, h, 64 * m:64 * m + 64],
                                      k[0, h // group], v[0, h // group], n, (bc[0, 0], bo[0, 0], cc[0, 0], ci[0, 0]), picks)
        worst = max(worst, mx)
        mean_sum += mean * len(picks)
        cnt += len(picks)
        del bc, bo, cc, ci
    return {"max_abs": worst, "mean_abs": mean_sum / max(cnt, 1), "row_blocks": cnt, "heads": hq}


def flex_parity_probe(q, k, v, out, block_mask, block, n, hq, hkv, blocks_per_head=3):
    """Kernel output against fp32 masked-dense attention over the identical block set, sampled row blocks of every head."""
    from minference_b200.checks import block_mask_row_block

    rows = (n + 63) // 64
    group = hq // hkv
    worst, mean_sum, cnt = 0.0, 0.0, 0
    for h in range(hq):
        picks = sorted(set(sample_row_blocks(0, rows, blocks_per_head)) | {(h * 131 + 7) % rows})
        for m in picks:
            want = block_mask_row_block(q[0, h, 64 * m:64 * m + 64], k[0, h // group], v[0, h // group], block_mask[0, h], m, block)
            d = (out[0, h, 64 * m:64 * m + 64].float() - want).abs()
            worst = max(worst, d.max().item())
            mean_sum += d.mean().item()
            cnt += 1
    return {"max_abs": worst, "mean_abs": mean_sum / max(cnt, 1), "row_blocks": cnt, "heads": hq}


def plan_slash_lists(plan):
    """The slash lists a plan was built from (kept by the plan builders for checks like the one above)."""
    if getattr(plan, "s_idx", None) is None:
        raise SystemExit("the plan does not carry its slash lists")
    return plan.s_idx


def run_ring_arm(args, wl):
    """N > 1: one sequence sharded over the ranks, zigzag ring attention (strong scaling)."""
    import torch.distributed as dist

    from minference_b200 import _cabi
    from minference_b200.checks import compare_row_blocks
    from minference_b200.cuda import convert_vertical_slash_indexes, set_status_checks
    from minference_b200.dist import ring
    from minference_b200.synthetic import local_vs_indices, make_qkv_ranges

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
    my_chunks = ring.owned_chunks(rank, world)
    ranges = [(ch * c, c) for ch in my_chunks]
    q, k, v = make_qkv_ranges(n, ranges, hq, hkv, seed=0, dtype=torch.bfloat16, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    band_idx = None

    def band_indices():
        bv, bs = local_vs_indices(n, hq, vsize, ssize, seed=0, device=dev)
        full = lambda x: torch.full((hq,), x, dtype=torch.int32, device=dev)
        return bv.contiguous(), bs.contiguous(), full(bv.shape[2]), full(bs.shape[2])

    if "_local" in wl:
        band_idx = band_indices()

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def measure(indices, steps, warmup):
        """(ms per step, attention ms on this rank, launches, tiles, issued, last output, index lists)"""
        stats = {"count_tiles": True}
        out = ring.ring_vertical_slash_attention(q, k, v, n, vsize, ssize, indices=indices, stats=stats)   # also counts the tiles
        tiles_local, issued_local = stats["tiles"], stats["issued"]
        for _ in range(max(warmup - 1, 0)):
            ring.ring_vertical_slash_attention(q, k, v, n, vsize, ssize, indices=indices)
        barrier()
        stats = {}
        t0, t1 = ev(), ev()
        t0.record()
        for _ in range(steps):
            out = ring.ring_vertical_slash_attention(q, k, v, n, vsize, ssize, indices=indices, stats=stats)
        t1.record()
        barrier()
        attn_ms = sum(a.elapsed_time(b) for a, b in stats["attn_events"]) / steps
        return (t0.elapsed_time(t1) / steps, attn_ms, len(stats["attn_events"]) // steps, tiles_local, issued_local, out,
                stats["indices"])

    sampler = ClockSampler(local) if rank == 0 else None
    step_ms, attn_ms, launches, tiles_local, issued_local, out, indices = measure(band_idx, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None

    # ---- parity of the timed output: sampled row blocks of this rank's two chunks (their first and last two row
    # blocks included) for two query heads of different KV groups, against the fp32 masked-dense recomputation over
    # the identical global index set; the KV heads' keys and values are gathered from all ranks for it
    v_idx, s_idx = indices[0], indices[1]
    heads = sorted({0, hq - 1})
    group = hq // hkv
    per_chunk = max(4, -(-64 // (2 * world)))
    seqlens = torch.tensor([n], dtype=torch.int32, device=dev)
    worst, mean_sum, cnt = 0.0, 0.0, 0
    for h in heads:
        hk = h // group
        kv_loc = torch.stack((k[0, hk], v[0, hk])).contiguous()             # [2, 2c, 128]
        gathered = [torch.empty_like(kv_loc) for _ in range(world)]
        dist.all_gather(gathered, kv_loc)
        k_full = ring.zigzag_merge([g[0] for g in gathered], world)
        v_full = ring.zigzag_merge([g[1] for g in gathered], world)
        del gathered
        bc, bo, cc, ci = convert_vertical_slash_indexes(seqlens, v_idx[:, h:h + 1].contiguous(), s_idx[:, h:h + 1].contiguous(), n)
        for li, ch in enumerate(my_chunks):
            picks = sample_row_blocks(ch * c // 64, c // 64, per_chunk)
            to_local = lambda m, li=li, ch=ch: li * c + (64 * m - ch * c)
            mx, mean = compare_row_blocks(lambda m: out[0, h, to_local(m):to_local(m) + 64], lambda m: q[0, h, to_local(m):to_local(m) + 64],
                                          k_full, v_full, n, (bc[0, 0], bo[0, 0], cc[0, 0], ci[0, 0]), picks)
            worst = max(worst, mx)
            mean_sum += mean * len(picks)
            cnt += len(picks)
        del bc, bo, cc, ci, k_full, v_full
    par = torch.tensor([worst, mean_sum, float(cnt)], dtype=torch.float64, device=dev)
    par_max = par.clone()
    dist.all_reduce(par_max, op=dist.ReduceOp.MAX)
    dist.all_reduce(par, op=dist.ReduceOp.SUM)
    ring_parity = {"max_abs": par_max[0].item(), "mean_abs": par[1].item() / max(par[2].item(), 1.0),
                   "row_blocks": int(par[2].item()), "heads": heads,
                   "against": "fp32 masked-dense over the identical global index set, rows of every rank's two chunks"}
    torch.cuda.empty_cache()

    # ---- the band index set on the same tensors (three steps), beside the headline
    band = None
    if band_idx is None and not args.no_extras:
        b_ms, b_attn, _, b_tiles, b_issued, _, _ = measure(band_indices(), 3, 2)
        bt = torch.tensor([b_ms, float(b_tiles), float(b_issued)], dtype=torch.float64, device=dev)
        bmax = bt.clone()
        dist.all_reduce(bmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(bt, op=dist.ReduceOp.SUM)
        band = {"workload": wl.replace("_ring", "_local_ring"), "steps": 3, "ms_per_step": bmax[0].item(),
                "value": bt[1].item() * FLOP_PER_TILE / (bmax[0].item() * 1e-3) / 1e12, "unit": "TFLOP/s",
                "tiles_per_layer": int(bt[1].item()), "issued_over_reference_tiles": bt[2].item() / max(bt[1].item(), 1.0),
                "attention_frac_of_sustained_peak_rank0": b_tiles * FLOP_PER_TILE / (b_attn * 1e-3) / 1e12 / measured_peaks()["sustained"]}

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
            o = ring.ring_vertical_slash_attention(*dbuf[b], n, vsize, ssize, indices=band_idx)
            freed[b].record(cur)
            s_out.wait_stream(cur)
            with torch.cuda.stream(s_out):
                ho.copy_(o, non_blocking=True)
            o.record_stream(s_out)
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

    times = torch.tensor([step_ms, e2e_ms], dtype=torch.float64, device=dev)
    sums = torch.tensor([float(tiles_local), float(issued_local)], dtype=torch.float64, device=dev)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    ms_per_step, e2e_ms = times.tolist()
    all_tiles, all_issued = sums.tolist()
    if rank == 0:
        peaks = measured_peaks()
        achieved = tiles_local * FLOP_PER_TILE / (attn_ms * 1e-3) / 1e12
        rows = n // 64
        est_launches = 0 if band_idx is not None else 10      # 2+2 score passes, combine, 3 histogram levels, count, write
        out_line = {
            "metric": "sparse_prefill_attn_tflops", "value": all_tiles * FLOP_PER_TILE / (ms_per_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(wl, world),
            "detail": {"tokens_per_gpu": n // world, "tiles_per_layer": int(all_tiles),
                       "fraction_of_causal_tiles": all_tiles / (hq * rows * (rows + 1) / 2),
                       "dense_equivalent_tflops": 4.0 * (n * n / 2) * 128 * hq / (ms_per_step * 1e-3) / 1e12,
                       "ms_attention_kernels_rank0": attn_ms, "non_kernel_share_rank0": 1.0 - attn_ms / ms_per_step,
                       "issued_over_reference_tiles": all_issued / max(all_tiles, 1.0),
                       "ring_parity": ring_parity, "band_index_set": band,
                       "one_gpu_anchor": "the 1-GPU line of the default workload carries detail.one_gpu_1m: this sequence on one GPU"},
            "e2e": {"value": all_tiles * FLOP_PER_TILE / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": world * sum(t.numel() * t.element_size() for t in (q, k, v)),
                    "d2h_bytes_per_step": world * q.numel() * q.element_size()},
            "gpu_launches": (launches + est_launches + 2) * args.steps * world,
            "roofline": {"bound": "tensor", "kernel": "sparse_attn_fwd_kernel", "achieved": achieved, "peak": peaks["sustained"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["sustained"],
                         "peak_kind": f"bf16 dense sustained per GPU, of {peaks['source']}; rank 0, summed over its {launches} launches per step",
                         "frac_of_burst": achieved / peaks["burst"], "traffic": None},
            "cpu_baseline": None,
            "clocks": clocks,
        }
        print(json.dumps(out_line))
    ok = ring_parity["max_abs"] <= 2e-2 and ring_parity["mean_abs"] <= 2e-3
    dist.destroy_process_group()
    if not ok:
        raise SystemExit(f"ring parity probe failed: {ring_parity}")


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
    from minference_b200.modules.minference_forward import LayerPattern
    from minference_b200.prefill_runner import LlamaPrefill, LlamaShape, seeded_pattern_tables, split_times, zigzag_positions

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
        patterns = [LayerPattern(t, shape.q_heads, n, None, dev) for t in tables]
        attention = lambda q, k, v, li: ring.ring_prefill_attention(q, k, v, n, patterns[li])
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def step(timing=None):
        ids = ids_host.to(dev, non_blocking=True)
        logits = model.prefill(ids, cfg, positions=positions, attention=attention, timing=timing)
        if rank == 0:       # the prompt's last token is rank 0's last token
            logits_host.copy_(logits, non_blocking=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if args.short_warmup and args.warmup > 0:
        # warm-up on a 32768-token prompt through the same code (kernels loaded, cuBLAS and NCCL initialised): a
        # full-length warm-up step of a million-token prompt costs minutes of GPU time
        n_short = 32768
        ids_s = ids_all[:n_short]
        pos_s = zigzag_positions(n_short, rank, world, dev) if world > 1 else None
        att_s = None
        if world > 1:
            pats_s = [LayerPattern(t, shape.q_heads, n_short, None, dev) for t in tables[:2]]
            att_s = lambda q, k, v, li: ring.ring_prefill_attention(q, k, v, n_short, pats_s[li % 2])
        for _ in range(args.warmup):
            model.prefill((ids_s[pos_s.cpu()] if world > 1 else ids_s).to(dev), cfg, positions=pos_s, attention=att_s)
    else:
        for _ in range(args.warmup):
            step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    timing = {}
    t0, t1 = ev(), ev()
    t0.record()
    for _ in range(args.steps):
        step(timing)
    t1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = t0.elapsed_time(t1)
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
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
                       "warmup_kind": "32768-token prompt" if args.short_warmup else "full prompt"},
            "detail": {"tokens_per_s": n / ttft_s, "finite_logits": bool(torch.isfinite(logits_host).all()),
                       "split_rank0": split_times(timing, total_ms / args.steps, layers)},
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
    ap.add_argument("--short-warmup", action="store_true",
                    help="whole-model workloads: warm up on a 32768-token prompt instead of the full one")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the side measurements reported beside the headline (band index set, the 1M-token layer on one GPU)")
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
        run_reference_arm(args, args.workload)
    elif args.workload in RING_WORKLOADS:
        if world < 2:
            raise SystemExit("ring workloads need torchrun with two or more ranks")
        run_ring_arm(args, args.workload)
    else:
        run_gpu_arm(args, args.workload)


if __name__ == "__main__":
    main()
