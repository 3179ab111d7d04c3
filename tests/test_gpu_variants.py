"""Variants of the prefill path built on the same kernels: the static vertical-slash lists, the TriangleMix layer
policies and the vLLM attention hook with its tensor-parallel head offset."""
import types

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


def test_static_variant_estimates_once_per_layer_and_shares_the_lists(dev):
    """modules/minference_forward.py:418-437 of the reference: head 0's lists (30 forced diagonals), cached, used by
    every head and by the next prompt."""
    from minference_b200.modules.minference_forward import static_prefill_forward
    from minference_b200.ops.pit_sparse_flash_attention_v2 import vertical_slash_sparse_attention
    from minference_b200.synthetic import make_qkv
    from oracle import reference_math as R

    n, hq, hkv = 2048, 4, 2
    q, k, v = make_qkv(n, hq, hkv, seed=14, dtype=torch.bfloat16)
    cfg = {"best_pattern": [{}, {"0": ["vertical_and_slash", 100, 300, 1.0], "1": ["vertical_and_slash", 500, 700, 1.0]}]}
    kw = {"attn_forward_config": cfg, "layer_idx": 1, "num_hidden_layers": 2, "attention_mask": None}
    out = static_prefill_forward(q.to(dev), k.to(dev), v.to(dev), kw)
    n_cached, v_idx, s_idx = cfg["_static_vs"][1]
    assert n_cached == n and v_idx.shape == (1, hq, 100) and s_idx.shape == (1, hq, 300)        # head 0's budgets for every head
    assert all(torch.equal(v_idx[0, h], v_idx[0, 0]) and torch.equal(s_idx[0, h], s_idx[0, 0]) for h in range(hq))
    # the oracle's static lists for head 0: same sets up to near-ties, 30 nearest diagonals forced (not 100)
    rv, rs = R.vertical_slash_estimate(q[:, :1], k[:, :1], 100, 300, forced_diagonals=30)
    got_v, got_s = set(v_idx[0, 0].tolist()), set(s_idx[0, 0].tolist())
    assert len(got_v & set(rv.flatten().tolist())) >= 98 and len(got_s & set(rs.flatten().tolist())) >= 294
    assert set(range(30)) <= got_s and not set(range(30, 100)) <= got_s
    # every head attends through those lists
    ref, _ = R.vertical_slash_attention_oracle(q.float(), k.float(), v.float(), v_idx.cpu(), s_idx.cpu())
    d = (out.float().cpu() - ref[:, :, :n]).abs()
    assert d.max().item() < MAX_ABS and d.mean().item() < MEAN_ABS
    # a second prompt of the same length reuses them (no estimation from its own queries)
    q2, k2, v2 = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=15, dtype=torch.bfloat16))
    out2 = static_prefill_forward(q2, k2, v2, kw)
    assert cfg["_static_vs"][1][1] is v_idx
    want2 = vertical_slash_sparse_attention(q2, k2, v2, v_idx, s_idx)
    assert torch.equal(out2, want2)


def test_tri_mix_policies_switch_at_the_starting_layer(dev):
    """modules/tri_mix.py:19-53 of the reference."""
    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.modules.tri_mix import tri_mix_forward, tri_mix_minference_forward
    from minference_b200.ops.streaming_kernel import tri_shape_kernel
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 1500, 4, 2
    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=16, dtype=torch.bfloat16))
    table = [{str(h): ["vertical_and_slash", 100, 300, 1.0] for h in range(hq)}] * 4
    cfg = {"starting_layer": 2, "n_init": 8, "n_local": 512, "n_last": 128, "best_pattern": table}
    kw = lambda layer: {"attn_forward_config": cfg, "layer_idx": layer, "num_hidden_layers": 4, "attention_mask": None}
    dense = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(2, 1),
                                                             v.float().repeat_interleave(2, 1), is_causal=True)
    shallow = tri_mix_forward(q, k, v, kw(1)).float()
    assert (shallow - dense).abs().max().item() < MAX_ABS
    deep = tri_mix_forward(q, k, v, kw(2))
    assert torch.equal(deep, tri_shape_kernel(q, k, v, kw(2)))
    assert (deep.float() - dense).abs().max().item() > 0.05              # the middle rows do lose keys
    assert (deep[:, :, -128:].float() - dense[:, :, -128:]).abs().max().item() < MAX_ABS     # the last rows see everything
    shallow_sparse = tri_mix_minference_forward(q, k, v, kw(0))
    want = minference_prefill_forward(q, k, v, {"attn_forward_config": {"best_pattern": table, "starting_layer": 0},
                                               "layer_idx": 0, "num_hidden_layers": 4, "attention_mask": None})
    assert torch.equal(shallow_sparse, want)
    assert cfg["starting_layer"] == 2                                    # the caller's config is left as it was
    assert torch.equal(tri_mix_minference_forward(q, k, v, kw(3)), tri_shape_kernel(q, k, v, kw(3)))


def test_vllm_hook_runs_the_sparse_prefill_with_the_tensor_parallel_head_offset(dev):
    """The wrapped AttentionImpl.forward on vLLM's own tensor layout ([tokens, heads, head_size]): a single-sequence
    prefill takes the sparse path, anything else the stock method; two emulated tensor-parallel ranks, each holding
    half of the heads and reading the pattern table at its head offset, reproduce the unsharded layer."""
    from minference_b200 import vllm_hook as V
    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 3000, 8, 4
    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=17, dtype=torch.bfloat16))
    table = [{}, {"0": ["vertical_and_slash", 100, 400, 1.0], "1": ["stream_llm", 64, 512, 1.0], "2": ["block_sparse", 0, 0, 1.0],
                  "4": ["stream_llm", 32, 256, 1.0], "5": ["vertical_and_slash", 30, 800, 1.0], "7": ["block_sparse", 0, 0, 1.0]}]
    attn_config = {"best_pattern": table, "starting_layer": 0}
    want = minference_prefill_forward(q, k, v, {"attn_forward_config": dict(attn_config), "layer_idx": 1,
                                               "num_hidden_layers": 2, "attention_mask": None})
    tok = lambda x: x[0].transpose(0, 1).contiguous()                    # [tokens, heads, 128] as vLLM passes them
    md = types.SimpleNamespace(num_actual_tokens=n, query_start_loc=torch.tensor([0, n], dtype=torch.int32, device=dev),
                               max_query_len=n, max_seq_len=n, use_cascade=False, causal=True)
    layer = types.SimpleNamespace(layer_name="model.layers.1.self_attn.attn")
    calls = []

    class Impl:         # the attributes of vllm.v1.attention.backends.flash_attn.FlashAttentionImpl the hook reads
        def __init__(self, heads, kv_heads):
            self.num_heads, self.num_kv_heads, self.head_size, self.scale = heads, kv_heads, 128, 128 ** -0.5
            self.alibi_slopes, self.sliding_window, self.logits_soft_cap, self.sinks = None, (-1, -1), 0, None

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None):
            calls.append(attn_metadata.num_actual_tokens)
            return output.fill_(7)

    parts = []
    for rank in range(2):          # tensor parallel size 2: four query heads and two KV heads per rank
        impl = V.wrap_impl(Impl(hq // 2, hkv // 2), dict(attn_config), head_offset=rank * (hq // 2))
        hs, ks = slice(rank * 4, rank * 4 + 4), slice(rank * 2, rank * 2 + 2)
        out = torch.empty(n + 8, 4 * 128, dtype=torch.bfloat16, device=dev)        # padded like vLLM's buffers
        pad = lambda x: torch.cat([x, torch.zeros(8, *x.shape[1:], dtype=x.dtype, device=dev)])
        impl.forward(layer, pad(tok(q[:, hs])), pad(tok(k[:, ks])), pad(tok(v[:, ks])), None, md, out)
        parts.append(out[:n].view(n, 4, 128).transpose(0, 1))
    got = torch.cat(parts, dim=0)[None]
    assert not calls and torch.equal(got, want)
    # a decode step and a two-request batch go to the stock method
    impl = V.wrap_impl(Impl(hq, hkv), dict(attn_config), 0)
    step = types.SimpleNamespace(num_actual_tokens=1, query_start_loc=torch.tensor([0, 1], device=dev), max_query_len=1,
                                 max_seq_len=n + 1, use_cascade=False, causal=True)
    two = types.SimpleNamespace(num_actual_tokens=n, query_start_loc=torch.tensor([0, 1000, n], device=dev), max_query_len=2000,
                                max_seq_len=2000, use_cascade=False, causal=True)
    for meta in (step, two):
        buf = torch.empty(n, hq * 128, dtype=torch.bfloat16, device=dev)
        impl.forward(layer, tok(q), tok(k), tok(v), None, meta, buf)
    assert calls == [1, n]


def test_install_on_model_wraps_every_attention_layer():
    from minference_b200 import vllm_hook as V

    class Impl:
        num_heads, num_kv_heads, head_size, scale = 4, 2, 128, 128 ** -0.5

        def forward(self, *a, **kw):
            return "stock"

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.impl = Impl()

    model = torch.nn.Sequential(Attn(), torch.nn.Linear(2, 2), Attn())
    assert V.install_on_model(model, {"best_pattern": [{}, {}], "starting_layer": 0}) == 2
    assert all(m.impl._minference_b200_wrapped for m in model if isinstance(m, Attn))
    assert model[0].impl.forward(None, None, None, None, None, None, None) == "stock"       # no metadata: profiling run


def test_vllm_hook_on_the_installed_vllm_implementation_and_metadata_classes(dev):
    """The same single-sequence prefill through an object of the installed vLLM's own ``FlashAttentionImpl`` with its
    own ``FlashAttentionMetadata`` (no engine, no KV cache: the wrapped method takes the sparse path before the stock
    code would touch either)."""
    import inspect

    try:
        from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl, FlashAttentionMetadata
    except Exception as e:
        pytest.skip(f"vLLM cannot be imported here: {type(e).__name__}")
    from minference_b200 import vllm_hook as V
    from minference_b200.modules.minference_forward import minference_prefill_forward
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 2048 + 40, 4, 2
    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=18, dtype=torch.bfloat16))
    table = [{"0": ["vertical_and_slash", 100, 400, 1.0], "1": ["stream_llm", 64, 512, 1.0], "2": ["block_sparse", 0, 0, 1.0]}]
    attn_config = {"best_pattern": table, "starting_layer": 0}
    want = minference_prefill_forward(q, k, v, {"attn_forward_config": dict(attn_config), "layer_idx": 0,
                                               "num_hidden_layers": 1, "attention_mask": None})
    try:
        kwargs = dict(num_heads=hq, head_size=128, scale=128 ** -0.5, num_kv_heads=hkv, alibi_slopes=None, sliding_window=None,
                      kv_cache_dtype="auto")
        accepted = inspect.signature(FlashAttentionImpl.__init__).parameters
        impl = FlashAttentionImpl(**{a: b for a, b in kwargs.items() if a in accepted})
        md = FlashAttentionMetadata(
            num_actual_tokens=n, max_query_len=n, query_start_loc=torch.tensor([0, n], dtype=torch.int32, device=dev),
            max_seq_len=n, seq_lens=torch.tensor([n], dtype=torch.int32, device=dev),
            block_table=torch.zeros(1, 1, dtype=torch.int32, device=dev), slot_mapping=torch.zeros(n, dtype=torch.int64, device=dev),
            use_cascade=False, common_prefix_len=0, cu_prefix_query_lens=None, prefix_kv_lens=None, suffix_kv_lens=None)
    except Exception as e:           # constructor arguments of another vLLM version, or a missing engine context
        pytest.skip(f"the installed vLLM's classes cannot be built stand-alone: {type(e).__name__}: {e}")
    assert V.is_single_sequence_prefill(md) and V.supports(impl, q)
    V.wrap_impl(impl, dict(attn_config), head_offset=0)
    layer = types.SimpleNamespace(layer_name="model.layers.0.self_attn.attn")
    tok = lambda x: x[0].transpose(0, 1).contiguous()
    out = torch.empty(n, hq * 128, dtype=torch.bfloat16, device=dev)
    impl.forward(layer, tok(q), tok(k), tok(v), None, md, out)
    assert torch.equal(out.view(n, hq, 128).transpose(0, 1)[None], want)


def test_vllm_hook_runs_the_other_operators_by_name(dev):
    """``vllm_a_shape`` and ``vllm_flexprefill``: the wrapped forward hands the tokens to the operator of that name."""
    from minference_b200 import vllm_hook as V
    from minference_b200.modules.flexprefill import flexprefill_forward
    from minference_b200.ops.streaming_kernel import a_shape_kernel
    from minference_b200.synthetic import make_qkv

    n, hq, hkv = 2500, 4, 2
    q, k, v = (t.to(dev) for t in make_qkv(n, hq, hkv, seed=19, dtype=torch.bfloat16))
    md = types.SimpleNamespace(num_actual_tokens=n, num_prefills=1, num_decodes=0, num_prefill_tokens=n, use_cascade=False)
    layer = types.SimpleNamespace(layer_name="model.layers.0.self_attn.attn")
    tok = lambda x: x[0].transpose(0, 1).contiguous()

    class Impl:
        def __init__(self):
            self.num_heads, self.num_kv_heads, self.head_size, self.scale = hq, hkv, 128, 128 ** -0.5
            self.alibi_slopes, self.sliding_window, self.logits_soft_cap, self.sinks = None, (-1, -1), 0, None

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None):
            raise AssertionError("the stock method must not run for a single-sequence prefill")

    for cfg, op in (({"prefill_operator": "a_shape", "n_local": 512, "n_init": 64}, a_shape_kernel),
                    ({"prefill_operator": "flexprefill", "gamma": 0.8, "tau": 0.0}, flexprefill_forward)):
        want = op(q, k, v, {"attn_forward_config": dict(cfg), "layer_idx": 0, "num_hidden_layers": 1, "attention_mask": None})
        impl = V.wrap_impl(Impl(), dict(cfg), 0)
        out = torch.empty(n, hq * 128, dtype=torch.bfloat16, device=dev)
        impl.forward(layer, tok(q), tok(k), tok(v), None, md, out)
        assert torch.equal(out.view(n, hq, 128).transpose(0, 1)[None], want)
