"""Seeded synthetic Q/K/V with the shapes and value distributions of a long-context prefill layer.

Stands in for the prompts and model weights the reference measures on (they are
downloaded at run time by experiments/benchmarks/benchmark_e2e.py:14-25 and are not
redistributable here).  Q, K, V ~ N(0,1), rotary position embedding on Q and K in the
half-rotation convention the patched attention uses (minference/patch.py:110-113,
minference/modules/minference_forward.py:495), then a fixed unit vector is added to a few
K rows (attention sinks at positions 0-3 plus 48 seeded positions) and to every Q row so
that vertical lines exist for the estimator to find.
"""
from __future__ import annotations

import torch


def rope_cos_sin(n: int, dim: int, theta: float, device, dtype=torch.float32, start: int = 0):
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    pos = torch.arange(start, start + n, device=device, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    return x * cos + rotate_half(x) * sin


def planted_positions(n: int, seed: int, extra: int = 48) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 7919)
    extra = min(extra, max(n - 4, 0))
    rest = 4 + torch.randperm(max(n - 4, 0), generator=g)[:extra]
    return torch.cat((torch.arange(min(4, n)), rest)).sort().values


def make_qkv(n: int, hq: int, hkv: int, d: int = 128, seed: int = 0, dtype=torch.bfloat16,
             device="cpu", theta: float = 5e5, plant: bool = True, chunk: int = 1 << 16):
    """Return ``q [1,hq,n,d]``, ``k, v [1,hkv,n,d]`` in ``dtype`` on ``device``.

    Generated chunk by chunk along the sequence so million-token cases never hold fp32
    copies of the whole tensor.  The CPU generator and the CUDA generator produce
    different streams; parity tests always feed the same tensors to both sides.
    """
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    gu = torch.Generator().manual_seed(seed + 104729)
    u = torch.nn.functional.normalize(torch.randn(d, generator=gu), dim=0).to(dev)
    q = torch.empty(1, hq, n, d, dtype=dtype, device=dev)
    k = torch.empty(1, hkv, n, d, dtype=dtype, device=dev)
    v = torch.empty(1, hkv, n, d, dtype=dtype, device=dev)
    planted = planted_positions(n, seed).to(dev) if plant else None
    for s in range(0, n, chunk):
        e = min(s + chunk, n)
        cos, sin = rope_cos_sin(e - s, d, theta, dev, start=s)
        qc = apply_rope(torch.randn(1, hq, e - s, d, generator=g, device=dev), cos, sin)
        kc = apply_rope(torch.randn(1, hkv, e - s, d, generator=g, device=dev), cos, sin)
        vc = torch.randn(1, hkv, e - s, d, generator=g, device=dev)
        if plant:
            qc = qc + u
            sel = planted[(planted >= s) & (planted < e)] - s
            kc[:, :, sel] += 3.0 * u
        q[:, :, s:e] = qc.to(dtype)
        k[:, :, s:e] = kc.to(dtype)
        v[:, :, s:e] = vc.to(dtype)
    return q, k, v


STREAM_BLOCK = 1 << 16


def make_qkv_ranges(n: int, ranges, hq: int, hkv: int, d: int = 128, seed: int = 0, dtype=torch.bfloat16,
                    device="cpu", theta: float = 5e5, plant: bool = True):
    """Token ranges ``[(start, length), ...]`` (concatenated in that order) of one fixed sequence of ``n`` tokens:
    the shard a rank owns under sequence parallelism, or with ``[(0, n)]`` the whole sequence.  Positions, and
    therefore the rotary phases and the planted columns, are those of the whole sequence, and the random stream is
    keyed by (seed, 65536-token block), so every split of the sequence sees the same values.  (``make_qkv`` draws one
    stream from token 0 on and gives a different sequence.)"""
    dev = torch.device(device)
    gu = torch.Generator().manual_seed(seed + 104729)
    u = torch.nn.functional.normalize(torch.randn(d, generator=gu), dim=0).to(dev)
    planted = planted_positions(n, seed).to(dev) if plant else None
    qs, ks, vs = [], [], []
    for start, length in ranges:
        q = torch.empty(1, hq, length, d, dtype=dtype, device=dev)
        k = torch.empty(1, hkv, length, d, dtype=dtype, device=dev)
        v = torch.empty(1, hkv, length, d, dtype=dtype, device=dev)
        for blk in range(start // STREAM_BLOCK, (start + length - 1) // STREAM_BLOCK + 1):
            b0 = blk * STREAM_BLOCK
            bl = min(STREAM_BLOCK, n - b0)
            g = torch.Generator(device=dev).manual_seed(seed * 1000003 + blk)
            cos, sin = rope_cos_sin(bl, d, theta, dev, start=b0)
            qc = apply_rope(torch.randn(1, hq, bl, d, generator=g, device=dev), cos, sin)
            kc = apply_rope(torch.randn(1, hkv, bl, d, generator=g, device=dev), cos, sin)
            vc = torch.randn(1, hkv, bl, d, generator=g, device=dev)
            if plant:
                qc = qc + u
                sel = planted[(planted >= b0) & (planted < b0 + bl)] - b0
                kc[:, :, sel] += 3.0 * u
            lo, hi = max(start, b0), min(start + length, b0 + bl)          # the part of the block inside the range
            q[:, :, lo - start:hi - start] = qc[:, :, lo - b0:hi - b0].to(dtype)
            k[:, :, lo - start:hi - start] = kc[:, :, lo - b0:hi - b0].to(dtype)
            v[:, :, lo - start:hi - start] = vc[:, :, lo - b0:hi - b0].to(dtype)
        qs.append(q); ks.append(k); vs.append(v)
    if len(qs) == 1:
        return qs[0], ks[0], vs[0]
    return torch.cat(qs, dim=2), torch.cat(ks, dim=2), torch.cat(vs, dim=2)


def local_vs_indices(n: int, heads: int, vertical_size: int, slash_size: int, seed: int = 0,
                     device="cpu"):
    """A "local" vertical-slash index set: slash offsets 0..s-1 (a band along the diagonal)
    and ``v`` vertical columns (first 30 plus seeded positions), per head.

    This is the regime real long-context heads live in (the shipped pattern tables pick
    a few thousand diagonals next to the main one); i.i.d. Gaussian data gives a nearly
    flat slash score instead, whose top-k spreads over the whole context.
    """
    s = min(n, max(slash_size, 50))
    v = min(n, max(vertical_size, 30))
    g = torch.Generator().manual_seed(seed + 15485863)
    s_idx = torch.arange(s - 1, -1, -1, dtype=torch.int32).repeat(1, heads, 1)
    v_rows = []
    for _ in range(heads):
        rest = 30 + torch.randperm(max(n - 30, 0), generator=g)[: max(v - 30, 0)]
        v_rows.append(torch.cat((torch.arange(min(30, n)), rest))[:v].sort().values)
    v_idx = torch.stack(v_rows)[None].to(torch.int32)
    return v_idx.to(device), s_idx.to(device)


def scattered_vs_indices(n: int, heads: int, vertical_size: int, slash_size: int, seed: int = 0, device="cpu"):
    """A "scattered" vertical-slash index set: the 100 nearest diagonals plus ``s - 100`` diagonals drawn uniformly
    from the whole context, and ``v`` uniformly drawn vertical columns, per head.  This is what the estimator returns
    on data without diagonal structure (seeded N(0,1) at a million tokens): nearly every selected diagonal stands
    alone, the regime in which a 128-row MMA tile does twice the work of the two 64x64 tiles it serves."""
    s = min(n, max(slash_size, 50))
    v = min(n, max(vertical_size, 30))
    g = torch.Generator().manual_seed(seed + 32452843)
    v_rows, s_rows = [], []
    for _ in range(heads):
        near = min(100, s)
        far = near + torch.randperm(max(n - near, 0), generator=g)[: s - near]
        s_rows.append(torch.cat((torch.arange(near), far)).sort(descending=True).values)
        rest = 30 + torch.randperm(max(n - 30, 0), generator=g)[: max(v - 30, 0)]
        v_rows.append(torch.cat((torch.arange(min(30, n)), rest))[:v].sort().values)
    return torch.stack(v_rows)[None].to(torch.int32).to(device), torch.stack(s_rows)[None].to(torch.int32).to(device)
