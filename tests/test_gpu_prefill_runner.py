"""Whole-model prefill runner on the GPU against the same network with stock dense attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    from minference_b200.prefill_runner import LlamaPrefill, LlamaShape

    shape = LlamaShape(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=1000)
    model = LlamaPrefill(shape, "cuda", seed=1, init_std=0.05)
    ids = torch.randint(0, shape.vocab, (1000,), generator=torch.Generator().manual_seed(2))
    return shape, model, ids


def _close(a, b):
    scale = b.abs().max().item()
    assert torch.isfinite(a).all()
    assert (a - b).abs().max().item() <= 3e-2 * scale + 1e-3, ((a - b).abs().max().item(), scale)


def test_runner_dense_layers_match_stock_attention(tiny):
    from minference_b200.prefill_runner import dense_reference_logits

    shape, model, ids = tiny
    ref = dense_reference_logits(model, ids)
    # every layer below starting_layer runs dense causal attention; chunking must not change the result
    out = model.prefill(ids, {"starting_layer": 1 << 30, "best_pattern": []}, chunk=256)
    _close(out, ref)


def test_runner_mixed_patterns_cover_everything_at_short_length(tiny):
    """At 1000 tokens the default budgets (1000 verticals, 6096 slashes, top-100 blocks, a
    4096-token window) select every causal key, so all three head patterns must reproduce dense
    attention through the whole network."""
    from minference_b200.prefill_runner import dense_reference_logits, seeded_pattern_tables

    shape, model, ids = tiny
    tables = seeded_pattern_tables(shape, seed=5)
    kinds = {t[0] for layer in tables for t in layer.values()}
    assert kinds == {"stream_llm", "vertical_and_slash", "block_sparse"}
    out = model.prefill(ids, {"starting_layer": 0, "best_pattern": tables}, chunk=384)
    _close(out, dense_reference_logits(model, ids))
