"""Run in a child process by tests/test_gpu_vllm_engine.py: a vLLM engine (in-process V1 core) on a two-layer
Llama-architecture model with dummy weights generates four tokens from a 4096-token prompt, first as it is and then
with the sparse prefill hook installed through ``MInference("vllm_minference", config_path=...)(llm)``.  The pattern
table gives every head budgets that select every diagonal at this length, so the sparse path is dense attention and
the tokens must come out the same; the decode steps after the prefill show that the KV cache was filled."""
import json
import os
import sys
import tempfile
import time

os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
os.environ.setdefault("VLLM_ALLOW_INSECURE_SERIALIZATION", "1")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def main():
    from vllm import LLM, SamplingParams
    d = tempfile.mkdtemp()
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 512, "num_attention_heads": 4,
           "num_key_value_heads": 2, "head_dim": 128, "num_hidden_layers": 2, "intermediate_size": 1024, "vocab_size": 1000,
           "max_position_embeddings": 32768, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "torch_dtype": "bfloat16",
           "hidden_act": "silu", "tie_word_embeddings": False, "bos_token_id": 1, "eos_token_id": 2}
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    n = 4096
    t0 = time.time()
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, enforce_eager=True, gpu_memory_utilization=0.2,
              max_model_len=8192, max_num_batched_tokens=8192, enable_chunked_prefill=False, enable_prefix_caching=False,
              dtype="bfloat16", seed=0)
    print("engine up in", round(time.time() - t0, 1), "s", flush=True)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 1000, (n,), generator=g).tolist()
    sp = SamplingParams(max_tokens=4, temperature=0.0, logprobs=5, detokenize=False)
    ref = llm.generate([{"prompt_token_ids": ids}], sp)[0].outputs[0]
    print("stock tokens", list(ref.token_ids), flush=True)
    from minference_b200 import MInference, vllm_hook
    table = [{str(h): ["vertical_and_slash", 1000, 6096, 1.0] for h in range(4)} for _ in range(2)]
    path = os.path.join(d, "table.json")
    json.dump(table, open(path, "w"))
    calls = {"n": 0}
    orig = vllm_hook.sparse_prefill_forward
    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)
    vllm_hook.sparse_prefill_forward = counted
    llm = MInference("vllm_minference", config_path=path)(llm)
    out = llm.generate([{"prompt_token_ids": ids}], sp)[0].outputs[0]
    print("hooked tokens", list(out.token_ids), "sparse prefill calls", calls["n"], flush=True)
    lp_ref = {k: v.logprob for k, v in ref.logprobs[0].items()}
    lp_out = {k: v.logprob for k, v in out.logprobs[0].items()}
    common = set(lp_ref) & set(lp_out)
    print("first-token logprob differences", {k: round(abs(lp_ref[k] - lp_out[k]), 4) for k in common})
    print("ENGINE_OK" if calls["n"] == 2 and list(out.token_ids)[:1] == list(ref.token_ids)[:1] else "ENGINE_MISMATCH")

if __name__ == "__main__":
    main()
