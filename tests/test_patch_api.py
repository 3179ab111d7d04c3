"""The patch / configuration API that mirrors the reference's MInference(...)(model)."""
import json

import pytest
import torch


def test_config_mirrors_reference_fields(tmp_path):
    from minference_b200 import MInferenceConfig
    from minference_b200.configs.model2path import register_model, get_support_models, synthetic_pattern_table, save_pattern_table

    table = synthetic_pattern_table(2, 4, seed=3, mix=("vertical_and_slash", "stream_llm", "block_sparse"))
    assert len(table) == 2 and set(table[0]) == {"0", "1", "2", "3"}
    for entry in table[0].values():
        assert entry[0] in ("vertical_and_slash", "stream_llm", "block_sparse") and len(entry) == 4
    path = tmp_path / "pattern.json"
    save_pattern_table(table, str(path))
    assert json.load(open(path)) == table
    cfg = MInferenceConfig(attn_type="minference", config_path=str(path), starting_layer=1)
    assert cfg.config_path == str(path) and cfg.attn_kwargs["starting_layer"] == 1 and cfg.kv_type == "dense"
    assert "minference" in MInferenceConfig.get_available_attn_types()
    register_model("unit/test-model", str(path))
    assert "unit/test-model" in get_support_models()
    assert MInferenceConfig(attn_type="minference", model_name="unit/test-model").config_path == str(path)
    with pytest.raises(ValueError):
        MInferenceConfig(attn_type="minference", model_name="no/such-model")
    with pytest.raises(ValueError):
        MInferenceConfig(attn_type="inf_llm")
    with pytest.raises(ValueError):
        MInferenceConfig(kv_type="snapkv", config_path=str(path))
    for ty in ("static", "tri_mix", "dilated1", "dilated2", "a_shape", "tri_shape", "dense"):       # no table needed
        assert MInferenceConfig(attn_type=ty).attn_type == ty
    assert MInferenceConfig(attn_type="tri_mix_minference", config_path=str(path)).config_path == str(path)
    with pytest.raises(ValueError):
        MInferenceConfig(attn_type="tri_mix_minference", model_name="no/such-model")


def test_register_config_dir_maps_the_reference_model_names(tmp_path):
    """MInference("minference", model_name) needs the model-name -> table-file mapping of the reference."""
    from minference_b200 import MInferenceConfig
    from minference_b200.configs import model2path as P

    assert len(P.TABLE_FILE_OF_MODEL) == 18
    fname = P.TABLE_FILE_OF_MODEL["gradientai/Llama-3-8B-Instruct-Gradient-1048k"]
    assert fname == P.TABLE_FILE_OF_MODEL["gradientai/Llama-3-8B-Instruct-262k"] and fname.endswith("best_pattern.json")
    (tmp_path / fname).write_text(json.dumps([{"0": ["vertical_and_slash", 30, 800, 0.9]}]))
    saved = dict(P.MODEL2PATH)
    try:
        names = P.register_config_dir(str(tmp_path))
        assert sorted(names) == sorted(m for m, f in P.TABLE_FILE_OF_MODEL.items() if f == fname)
        cfg = MInferenceConfig("minference", model_name="gradientai/Llama-3-8B-Instruct-Gradient-1048k")
        assert cfg.config_path == str(tmp_path / fname)
        with pytest.raises(ValueError):
            MInferenceConfig("minference", model_name="Qwen/Qwen2.5-7B-Instruct")       # its file is not in the directory
        assert len(P.register_config_dir(str(tmp_path), require_files=False)) == 18
    finally:
        P.MODEL2PATH.clear()
        P.MODEL2PATH.update(saved)


def test_patch_defaults_follow_the_reference(tmp_path, monkeypatch):
    """Per-type defaults injected by MInference.patch_model (models_patch.py:98-128 of the reference)."""
    import types

    from minference_b200 import MInference, models_patch

    monkeypatch.setattr(models_patch, "new_patch", lambda model, cfg: cfg)
    model = types.SimpleNamespace(config=types.SimpleNamespace())
    path = tmp_path / "t.json"
    path.write_text(json.dumps([{"0": ["vertical_and_slash", 30, 800, 0.9]}]))
    kw = MInference("tri_mix")(model).attn_kwargs
    assert (kw["n_local"], kw["n_init"], kw["n_last"], kw["starting_layer"]) == (512, 8, 128, 16)
    kw = MInference("tri_mix_minference", config_path=str(path), starting_layer=3)(model).attn_kwargs
    assert kw["starting_layer"] == 3 and kw["best_pattern"][0]["0"][1] == 30
    kw = MInference("tri_shape")(model).attn_kwargs
    assert (kw["n_local"], kw["n_init"], kw["n_last"]) == (3968, 128, 100)
    kw = MInference("static", config_path=str(path))(model).attn_kwargs
    assert kw["best_pattern"][0]["0"][2] == 800
    assert "best_pattern" not in MInference("static")(model).attn_kwargs


def test_layer_pattern_cache_is_bounded_and_tied_to_its_config():
    from minference_b200.modules import minference_forward as mf

    table = [{"0": ["stream_llm", 64, 256, 1.0]}]
    cfg_a = {"best_pattern": table}
    pa = mf._layer_pattern(cfg_a, 0, 2, 1024, "cpu")
    assert mf._layer_pattern(cfg_a, 0, 2, 1024, "cpu") is pa            # same config, same key: reused
    cfg_b = {"best_pattern": [{"0": ["stream_llm", 8, 16, 1.0]}]}        # another model's table, same layer / heads / length
    pb = mf._layer_pattern(cfg_b, 0, 2, 1024, "cpu")
    assert pb is not pa and pb.head_param.tolist()[0] == [8, 16] and pa.head_param.tolist()[0] == [64, 256]
    for n in range(mf._PATTERN_CACHE_ENTRIES + 40):                      # many prompt lengths: the cache stays bounded
        mf._layer_pattern(cfg_a, 0, 2, 2048 + 64 * n, "cpu")
    assert len(cfg_a["_layer_patterns"]) <= mf._PATTERN_CACHE_ENTRIES
    off = mf.LayerPattern({"0": ["stream_llm", 1, 2, 1], "3": ["stream_llm", 5, 6, 1]}, 2, 1024, None, "cpu", head_offset=2)
    assert off.head_param.tolist() == [[0, 0], [5, 6]] and off.vertical_size.tolist()[0] == 1000     # heads 2 and 3 of the table


def test_stock_attention_is_used_when_the_sparse_kernels_do_not_apply():
    """Another logit scale, sliding-window layers, batch above 1, another dtype: the registered attention function
    must hand the call to the stock implementation instead of computing with 1/sqrt(d)."""
    from minference_b200.patch import _sparse_path_refusal

    q = torch.zeros(1, 4, 512, 128, dtype=torch.bfloat16, device="meta")
    ok = lambda **kw: _sparse_path_refusal(kw.pop("q", q), kw.pop("k", q), kw.pop("scaling", None), kw)
    cuda_like = type("T", (), {"shape": q.shape, "dtype": torch.bfloat16, "is_cuda": True, "device": torch.device("cuda")})()
    assert _sparse_path_refusal(cuda_like, cuda_like, None, {}) is None
    assert _sparse_path_refusal(cuda_like, cuda_like, 128 ** -0.5, {}) is None
    assert "scales" in _sparse_path_refusal(cuda_like, cuda_like, 0.0078125, {})              # Granite-style multiplier
    assert "sliding" in _sparse_path_refusal(cuda_like, cuda_like, None, {"sliding_window": 4096})
    assert "soft" in _sparse_path_refusal(cuda_like, cuda_like, None, {"softcap": 50.0})
    assert "bf16" in ok()                                                                      # not a CUDA tensor
    one = type("T", (), {"shape": (1, 4, 1, 128), "dtype": torch.bfloat16, "is_cuda": True, "device": torch.device("cuda")})()
    assert _sparse_path_refusal(one, cuda_like, None, {}) == "decode"
    two = type("T", (), {"shape": (2, 4, 512, 128), "dtype": torch.bfloat16, "is_cuda": True, "device": torch.device("cuda")})()
    assert "batch" in _sparse_path_refusal(two, two, None, {})


def test_vllm_hook_recognises_a_single_sequence_prefill():
    import types

    from minference_b200 import vllm_hook as V

    assert V.layer_index_of("model.layers.17.self_attn.attn") == 17 and V.layer_index_of("3.attn") == 3
    md = lambda n, seqs, max_q, max_s, **kw: types.SimpleNamespace(
        num_actual_tokens=n, query_start_loc=torch.zeros(seqs + 1, dtype=torch.int32), max_query_len=max_q, max_seq_len=max_s,
        use_cascade=kw.get("cascade", False), causal=kw.get("causal", True))
    assert V.is_single_sequence_prefill(md(4096, 1, 4096, 4096))
    assert not V.is_single_sequence_prefill(md(4096, 2, 2048, 2048))        # two requests
    assert not V.is_single_sequence_prefill(md(1024, 1, 1024, 5120))        # a later chunk: cached context
    assert not V.is_single_sequence_prefill(md(1, 1, 1, 900))               # decode
    assert not V.is_single_sequence_prefill(md(4096, 1, 4096, 4096, cascade=True))
    assert not V.is_single_sequence_prefill(None)
    impl = types.SimpleNamespace(head_size=128, scale=128 ** -0.5, alibi_slopes=None, sliding_window=(-1, -1),
                                 logits_soft_cap=0, sinks=None)
    q = types.SimpleNamespace(dtype=torch.bfloat16, is_cuda=True)
    assert V.supports(impl, q)
    impl.sliding_window = (4095, 0)
    assert not V.supports(impl, q)


def test_layer_pattern_parsing():
    from minference_b200 import _cabi
    from minference_b200.modules.minference_forward import LayerPattern, clamp_budgets

    assert clamp_budgets(8192, 1000, 6096) == (1000, 6096)
    assert clamp_budgets(100, 1000, 6096) == (100, 100)
    assert clamp_budgets(8192, 5, 5) == (30, 50)
    layer = {"0": ["vertical_and_slash", 30, 800, 1], "1": ["stream_llm", 128, 512, 1], "2": ["block_sparse", 0, 0, 1]}
    pat = LayerPattern(layer, 4, 8192, None, "cpu")        # head 3 falls back to the default pattern
    assert pat.head_mode.tolist() == [_cabi.MODE_PLAN, _cabi.MODE_ASHAPE, _cabi.MODE_PLAN, _cabi.MODE_PLAN]
    assert pat.head_param.tolist()[1] == [128, 512]
    assert pat.vertical_size.tolist() == [30, -1, -1, 1000] and pat.slash_size.tolist() == [800, -1, -1, 6096]
    assert pat.block_select.tolist() == [0, 0, 1, 0]
    assert pat.cap_v == 1000 and pat.cap_s == 6096 and pat.any_vs and pat.any_bs
    half = LayerPattern(layer, 4, 8192, 0.5, "cpu")        # minference_ratio scales the budgets
    assert half.vertical_size.tolist()[3] == 500 and half.slash_size.tolist()[3] == 3048


@pytest.mark.gpu
def test_patched_llama_matches_dense_when_budgets_cover_everything(tmp_path):
    """With vertical/slash budgets >= the sequence the sparse pattern is the full causal mask, so a
    patched random-init Llama must reproduce the stock attention's logits."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from transformers import LlamaConfig, LlamaForCausalLM

    from minference_b200 import MInference
    from minference_b200.configs.model2path import save_pattern_table, synthetic_pattern_table

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=1000, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      rope_theta=5e5, attn_implementation="sdpa")
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 1000, (1, 700), device="cuda")
    with torch.no_grad():
        ref = model(ids, use_cache=False).logits.float()
    path = tmp_path / "full.json"
    save_pattern_table(synthetic_pattern_table(2, 4, vertical=4096, slash=4096), str(path))
    model = MInference("minference", config_path=str(path))(model)
    with torch.no_grad():
        out = model(ids, use_cache=False).logits.float()
    assert torch.isfinite(out).all()
    assert (out - ref).abs().max().item() < 0.15 and (out - ref).abs().mean().item() < 0.02
    # a sparse table runs too and stays close on this short input
    save_pattern_table(synthetic_pattern_table(2, 4, seed=1, mix=("vertical_and_slash", "stream_llm", "block_sparse"),
                                               vertical=100, slash=300, n_init=64, n_local=256), str(path))
    model = MInference("minference", config_path=str(path))(model)
    with torch.no_grad():
        out2 = model(ids, use_cache=False).logits.float()
    assert torch.isfinite(out2).all()


def test_search_and_record_appends_one_layer_per_call(tmp_path, monkeypatch):
    """Bookkeeping of the offline search (the JSON file grows by one layer per call, a finished
    file is refused like modules/minference_forward.py:646-650 of the reference); the scoring
    itself needs the GPU and is tested there."""
    import json

    from minference_b200.modules import pattern_search

    calls = []

    def fake_search(q, k, v, **kw):
        calls.append(1)
        return {0: ("vertical_and_slash", 100, 750, 0.9), 1: ("vertical_and_slash", 1000, 6096, 0.8)}

    monkeypatch.setattr(pattern_search, "search_layer_patterns", fake_search)
    path = str(tmp_path / "table.json")
    for layer in range(2):
        got = pattern_search.search_and_record(None, None, None, layer, 2, path)
        assert got == {"0": ["vertical_and_slash", 100, 750, 0.9], "1": ["vertical_and_slash", 1000, 6096, 0.8]}
    assert len(json.load(open(path))) == 2 and len(calls) == 2
    with pytest.raises(RuntimeError):
        pattern_search.search_and_record(None, None, None, 0, 2, path)
    # a layer that is already in an unfinished file is not searched again
    path2 = str(tmp_path / "partial.json")
    pattern_search.search_and_record(None, None, None, 0, 3, path2)
    pattern_search.search_and_record(None, None, None, 0, 3, path2)
    assert len(json.load(open(path2))) == 1 and len(calls) == 3


def test_configuration_accepts_search_and_tri_shape(tmp_path):
    from minference_b200 import MInferenceConfig

    cfg = MInferenceConfig(attn_type="minference", is_search=True, config_path=str(tmp_path / "t.json"))
    assert cfg.attn_kwargs["is_search"] is True and cfg.attn_kwargs["config_path"].endswith("t.json")
    with pytest.raises(ValueError):
        MInferenceConfig(attn_type="minference", is_search=True, model_name="unregistered-model")
    assert MInferenceConfig(attn_type="tri_shape").attn_type == "tri_shape"
    assert "tri_shape" in MInferenceConfig.get_available_attn_types()


def test_bench_tile_formulas_match_the_oracle_masks():
    import numpy as np

    import bench
    from oracle import reference_math as R

    for n, n_init, n_local in ((2048, 128, 512), (1500, 100, 300), (600, 128, 4096)):
        tiles = 0
        i = np.arange(n)[:, None]
        j = np.arange(n)[None, :]
        window = ((i - j) >= 0) & ((i - j) < n_local)                       # stage 1 of the reference
        sinks = (j < n_init) & ((i - j) >= n_local) if n > n_local else np.zeros((n, n), bool)    # stage 2
        pad = (-n) % 64
        for mask in (window, sinks):
            mp = np.pad(mask, ((0, pad), (0, pad)))
            tiles += int(np.any(mp.reshape((n + pad) // 64, 64, (n + pad) // 64, 64), axis=(1, 3)).sum())
        assert bench.a_shape_tiles(n, n_init, n_local) == tiles, (n, n_init, n_local)
        assert np.array_equal(window | sinks, R.a_shape_mask_rows(n, n_init, n_local, 0, n))
    t1, k1 = bench.mixed_pattern_table(28, 1000, 6096)
    t2, k2 = bench.mixed_pattern_table(28, 1000, 6096)
    assert t1 == t2 and set(k1) == {0, 1, 2}


def test_zigzag_positions_cover_the_sequence():
    import torch

    from minference_b200.prefill_runner import zigzag_positions

    n, world = 256 * 8, 4
    allpos = torch.cat([zigzag_positions(n, r, world) for r in range(world)])
    assert sorted(allpos.tolist()) == list(range(n))
    assert zigzag_positions(n, 0, world)[-1].item() == n - 1      # the last token is rank 0's last token


def test_vllm_hook_assumptions_hold_for_the_installed_vllm():
    """The hook wraps ``impl.forward`` of every attention layer and reads a few host-side metadata fields: the installed
    vLLM's FlashAttention implementation, its metadata and its attention layer are inspected (no GPU, no engine) for
    exactly the names the hook relies on."""
    import dataclasses
    import inspect

    import pytest

    try:
        from vllm.model_executor.layers.attention import Attention
        from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl, FlashAttentionMetadata
    except Exception as e:           # vLLM absent or not importable on this machine
        pytest.skip(f"vLLM cannot be imported here: {type(e).__name__}")
    params = list(inspect.signature(FlashAttentionImpl.forward).parameters)
    assert params[:8] == ["self", "layer", "query", "key", "value", "kv_cache", "attn_metadata", "output"]
    fields = {f.name for f in dataclasses.fields(FlashAttentionMetadata)}
    assert {"num_actual_tokens", "max_query_len", "query_start_loc", "max_seq_len", "use_cascade", "causal"} <= fields
    init_src = inspect.getsource(FlashAttentionImpl.__init__)
    for attr in ("num_heads", "num_kv_heads", "head_size", "scale", "sliding_window", "logits_soft_cap", "alibi_slopes"):
        assert f"self.{attr}" in init_src, attr
    layer_src = inspect.getsource(Attention.__init__)
    assert "self.impl" in layer_src and "self.layer_name" in layer_src
    # the FlashInfer backend (the default on Blackwell): same forward signature, its own metadata layout
    from vllm.v1.attention.backends.flashinfer import FlashInferBackend, FlashInferImpl, FlashInferMetadata
    from vllm.v1.attention.backends.flash_attn import FlashAttentionBackend

    assert list(inspect.signature(FlashInferImpl.forward).parameters)[:8] == params[:8]
    fi = {f.name for f in dataclasses.fields(FlashInferMetadata)}
    assert {"num_actual_tokens", "num_prefills", "num_decodes", "num_prefill_tokens", "use_cascade"} <= fi
    # the layer, not impl.forward, writes the KV cache: a wrapped forward that skips the stock code leaves it filled
    assert FlashAttentionBackend.forward_includes_kv_cache_update is False
    assert FlashInferBackend.forward_includes_kv_cache_update is False


def test_vllm_hook_recognises_both_metadata_layouts_and_refuses_unsuitable_engines():
    import types

    import pytest
    import torch

    from minference_b200 import vllm_hook as V

    fa = types.SimpleNamespace(num_actual_tokens=100, query_start_loc=torch.tensor([0, 100]), max_query_len=100, max_seq_len=100,
                               use_cascade=False, causal=True)
    assert V.is_single_sequence_prefill(fa)
    assert not V.is_single_sequence_prefill(types.SimpleNamespace(**{**vars(fa), "max_seq_len": 300}))       # cached context
    fi = types.SimpleNamespace(num_actual_tokens=100, num_prefills=1, num_decodes=0, num_prefill_tokens=100, use_cascade=False)
    assert V.is_single_sequence_prefill(fi)
    assert not V.is_single_sequence_prefill(types.SimpleNamespace(**{**vars(fi), "num_decodes": 2, "num_prefill_tokens": 98}))
    assert not V.is_single_sequence_prefill(types.SimpleNamespace(**{**vars(fi), "num_prefills": 2}))
    assert not V.is_single_sequence_prefill(types.SimpleNamespace(num_actual_tokens=100))                     # unknown layout
    assert not V.is_single_sequence_prefill(None)

    def engine(prefix, chunked, budget, longest):
        cfg = types.SimpleNamespace(cache_config=types.SimpleNamespace(enable_prefix_caching=prefix),
                                    scheduler_config=types.SimpleNamespace(enable_chunked_prefill=chunked, max_num_batched_tokens=budget),
                                    model_config=types.SimpleNamespace(max_model_len=longest))
        return types.SimpleNamespace(llm_engine=types.SimpleNamespace(vllm_config=cfg))

    V.check_engine_settings(engine(False, False, 8192, 8192))
    V.check_engine_settings(engine(False, True, 8192, 8192))
    V.check_engine_settings(types.SimpleNamespace())                   # unknown engine object: let through
    with pytest.raises(ValueError):
        V.check_engine_settings(engine(True, False, 8192, 8192))
    with pytest.raises(ValueError):
        V.check_engine_settings(engine(False, True, 2048, 8192))


def test_other_vllm_attention_types_are_routed_through_the_hook_with_their_defaults():
    """``MInference("vllm_a_shape")(llm)`` and its siblings (minference_configuration.py:24-28 of the reference): the hook
    is installed with the operator of that name and the defaults of the Hugging Face type (no pattern table)."""
    import types

    import torch

    from minference_b200 import MInference

    class Impl:
        num_heads, num_kv_heads, head_size, scale = 4, 2, 128, 128 ** -0.5

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None):
            return output

    for ty, want in (("vllm_a_shape", {"n_local": 3968, "n_init": 128}), ("vllm_tri_shape", {"n_last": 100}),
                     ("vllm_flexprefill", {})):
        model = torch.nn.Module()
        model.attn = torch.nn.Module()
        model.attn.impl = Impl()
        def apply_model(fn, model=model):
            return [fn(model)]

        llm = types.SimpleNamespace(apply_model=apply_model)
        assert MInference(ty)(llm) is llm
        assert getattr(model.attn.impl, "_minference_b200_wrapped", False)
        cfg = model.attn.impl.forward.__func__.__closure__
        attn_config = next(c.cell_contents for c in cfg if isinstance(c.cell_contents, dict))
        assert attn_config["prefill_operator"] == ty[len("vllm_"):]
        for key, val in want.items():
            assert attn_config[key] == val
