"""Whole-model long-context prefill with the sparse attention path: time to first token.

Plays the role of the reference's patched Hugging Face forward for a single long prompt
(minference/patch.py:500-558: layer norm, projections and MLP applied chunk by chunk so that no
[N, ffn] activation is ever resident; patch.py:787-790: logits of the last token only) and of its
timing script (experiments/benchmarks/benchmark_e2e.py:33-38: one ``use_cache=False`` forward).
The weights are random (there are no checkpoints here); the architecture is Llama: RMSNorm,
rotary embedding in the half-rotation convention, grouped-query attention, SwiGLU MLP.

Dense projections and the MLP are library GEMMs (``torch.matmul``); attention of every layer goes
through ``minference_prefill_forward`` with the per-head pattern table, exactly as the patched model
would call it.  Under a process group the prompt is sequence-sharded in zigzag chunks: the dense
parts are token-parallel and need no exchange, attention runs as the vertical-slash ring.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .modules.minference_forward import minference_prefill_forward
from .synthetic import apply_rope, rope_cos_sin


@dataclass
class LlamaShape:
    layers: int = 32
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 5e5
    rms_eps: float = 1e-5


class LlamaPrefill:
    """Random-init Llama-architecture weights and a chunked prefill forward."""

    def __init__(self, shape: LlamaShape, device, seed: int = 0, dtype=torch.bfloat16, init_std: float = 0.02):
        self.shape, self.device, self.dtype = shape, torch.device(device), dtype
        g = torch.Generator(device=self.device).manual_seed(seed)
        s = shape
        if s.head_dim != 128:
            raise ValueError("the attention kernel is built for head_dim 128")

        def w(rows, cols):
            return (torch.randn(rows, cols, generator=g, device=self.device, dtype=torch.float32) * init_std).to(dtype)

        self.embed = w(s.vocab, s.hidden)
        self.lm_head = w(s.hidden, s.vocab)
        self.final_norm = torch.ones(s.hidden, device=self.device, dtype=dtype)
        self.layers = []
        for _ in range(s.layers):
            self.layers.append({
                "attn_norm": torch.ones(s.hidden, device=self.device, dtype=dtype),
                "wqkv": w(s.hidden, (s.q_heads + 2 * s.kv_heads) * s.head_dim),
                "wo": w(s.q_heads * s.head_dim, s.hidden),
                "mlp_norm": torch.ones(s.hidden, device=self.device, dtype=dtype),
                "w_gate_up": w(s.hidden, 2 * s.ffn),
                "w_down": w(s.ffn, s.hidden),
            })

    def _rms(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.shape.rms_eps)).to(x.dtype) * weight

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, attn_forward_config: dict, chunk: int = 16384,
                positions: torch.Tensor | None = None, attention=None, timing: dict | None = None) -> torch.Tensor:
        """``ids [N]`` (this rank's tokens) -> fp32 logits ``[vocab]`` of the last local token.

        ``positions [N]`` are the tokens' positions in the whole prompt (default 0..N-1).
        ``attention(q, k, v, layer_idx)`` replaces the single-GPU operator (the ring passes one).
        ``timing``: a dict that receives CUDA-event pairs, ``"gemm"`` around every projection / MLP product and
        ``"attention"`` around every layer's attention (see ``split_times``).
        """
        s = self.shape
        n = ids.numel()
        dev, dt = self.device, self.dtype

        def timed(kind, fn):
            if timing is None:
                return fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn()
            e1.record()
            timing.setdefault(kind, []).append((e0, e1))
            return r

        x = self.embed[ids.to(dev)]                                   # [N, hidden]
        q = torch.empty(1, s.q_heads, n, s.head_dim, device=dev, dtype=dt)
        k = torch.empty(1, s.kv_heads, n, s.head_dim, device=dev, dtype=dt)
        v = torch.empty(1, s.kv_heads, n, s.head_dim, device=dev, dtype=dt)
        nq, nk = s.q_heads * s.head_dim, s.kv_heads * s.head_dim
        for li, L in enumerate(self.layers):
            for c0 in range(0, n, chunk):
                c1 = min(c0 + chunk, n)
                h_in = self._rms(x[c0:c1], L["attn_norm"])
                qkv = timed("gemm", lambda: h_in @ L["wqkv"])
                if positions is None:
                    cos, sin = rope_cos_sin(c1 - c0, s.head_dim, s.rope_theta, dev, start=c0)
                else:
                    cos, sin = _rope_at(positions[c0:c1], s.head_dim, s.rope_theta)
                cos, sin = cos[:, None, :], sin[:, None, :]
                qc = apply_rope(qkv[:, :nq].view(c1 - c0, s.q_heads, s.head_dim).float(), cos, sin)
                kc = apply_rope(qkv[:, nq:nq + nk].view(c1 - c0, s.kv_heads, s.head_dim).float(), cos, sin)
                q[0, :, c0:c1] = qc.transpose(0, 1)
                k[0, :, c0:c1] = kc.transpose(0, 1)
                v[0, :, c0:c1] = qkv[:, nq + nk:].view(c1 - c0, s.kv_heads, s.head_dim).transpose(0, 1)
            if attention is not None:
                o = timed("attention", lambda: attention(q, k, v, li))
            else:
                o = timed("attention", lambda: minference_prefill_forward(
                    q, k, v, {"attention_mask": None, "layer_idx": li, "num_hidden_layers": s.layers,
                              "attn_forward_config": attn_forward_config}))
            for c0 in range(0, n, chunk):
                c1 = min(c0 + chunk, n)
                o_rows = o[0, :, c0:c1].transpose(0, 1).reshape(c1 - c0, nq)
                x[c0:c1] += timed("gemm", lambda: o_rows @ L["wo"])
                h_mlp = self._rms(x[c0:c1], L["mlp_norm"])
                gu = timed("gemm", lambda: h_mlp @ L["w_gate_up"])
                act = torch.nn.functional.silu(gu[:, :s.ffn]) * gu[:, s.ffn:]
                x[c0:c1] += timed("gemm", lambda: act @ L["w_down"])
            del o
        return (self._rms(x[-1:], self.final_norm) @ self.lm_head)[0].float()


def split_times(timing: dict, total_ms: float, layers: int) -> dict:
    """Milliseconds per layer of attention, of the dense products and of everything else (norms, rotary embedding,
    activation, residual adds, copies) from the event pairs ``prefill(timing=...)`` recorded; synchronise first."""
    gemm = sum(a.elapsed_time(b) for a, b in timing.get("gemm", []))
    attn = sum(a.elapsed_time(b) for a, b in timing.get("attention", []))
    return {"attention_ms_per_layer": attn / layers, "dense_gemm_ms_per_layer": gemm / layers,
            "rest_ms_per_layer": max(total_ms - gemm - attn, 0.0) / layers}


def zigzag_positions(n_ctx: int, rank: int, world: int, device=None) -> torch.Tensor:
    """Positions in the prompt of the tokens rank ``rank`` owns under the zigzag sequence split
    (chunks ``rank`` and ``2*world-1-rank``); the prompt's last token is the last one of rank 0."""
    from .dist.ring import chunk_size, owned_chunks

    c = chunk_size(n_ctx, world)
    return torch.cat([torch.arange(ch * c, (ch + 1) * c, device=device) for ch in owned_chunks(rank, world)])


def _rope_at(positions: torch.Tensor, dim: int, theta: float):
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim))
    freqs = torch.outer(positions.float(), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def seeded_pattern_tables(shape: LlamaShape, seed: int = 0, vertical: int = 1000, slash: int = 6096,
                          a_shape=(128, 4096), kinds=("stream_llm", "vertical_and_slash", "block_sparse")):
    """One pattern table per layer in the schema of the reference's configs/*.json, each head drawn
    from ``kinds`` by the seed."""
    g = torch.Generator().manual_seed(seed)
    tables = []
    for _ in range(shape.layers):
        pick = torch.randint(0, len(kinds), (shape.q_heads,), generator=g).tolist()
        t = {}
        for h, p in enumerate(pick):
            ty = kinds[p]
            t[str(h)] = ([ty, a_shape[0], a_shape[1], 1.0] if ty == "stream_llm" else
                         [ty, vertical, slash, 1.0] if ty == "vertical_and_slash" else [ty, 100, 0, 1.0])
        tables.append(t)
    return tables


@torch.no_grad()
def dense_reference_logits(model: LlamaPrefill, ids: torch.Tensor) -> torch.Tensor:
    """The same network evaluated without chunking and with the stock causal attention of torch
    (checker for tests; fp32 softmax inside ``scaled_dot_product_attention``)."""
    s = model.shape
    n = ids.numel()
    x = model.embed[ids.to(model.device)]
    cos, sin = rope_cos_sin(n, s.head_dim, s.rope_theta, model.device)
    cos, sin = cos[:, None, :], sin[:, None, :]
    nq, nk = s.q_heads * s.head_dim, s.kv_heads * s.head_dim
    for L in model.layers:
        qkv = model._rms(x, L["attn_norm"]) @ L["wqkv"]
        q = apply_rope(qkv[:, :nq].view(n, s.q_heads, s.head_dim).float(), cos, sin).to(x.dtype).transpose(0, 1)
        k = apply_rope(qkv[:, nq:nq + nk].view(n, s.kv_heads, s.head_dim).float(), cos, sin).to(x.dtype).transpose(0, 1)
        v = qkv[:, nq + nk:].view(n, s.kv_heads, s.head_dim).transpose(0, 1)
        rep = s.q_heads // s.kv_heads
        o = torch.nn.functional.scaled_dot_product_attention(
            q[None], k.repeat_interleave(rep, 0)[None], v.repeat_interleave(rep, 0)[None], is_causal=True)
        x = x + o[0].transpose(0, 1).reshape(n, nq) @ L["wo"]
        gu = model._rms(x, L["mlp_norm"]) @ L["w_gate_up"]
        x = x + (torch.nn.functional.silu(gu[:, :s.ffn]) * gu[:, s.ffn:]) @ L["w_down"]
    return (model._rms(x[-1:], model.final_norm) @ model.lm_head)[0].float()
