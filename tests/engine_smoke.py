"""End-to-end smoke of the attention backend inside a real vLLM engine, without weights. An
opt-in engine test (it needs a GPU and an installed vLLM, and takes minutes): pytest does not
collect it; run it by hand.

    python tests/engine_smoke.py [--graphs] [--kv fp8] [--dtype float16] [--route [--shadow]]

Builds a two-layer Llama-shaped model with random ("dummy") weights from a config written to
a temporary directory, runs the same token prompts greedily through vLLM twice in one process
-- once on vLLM's own attention backend, once on this build's backend registered through the
plugin's own code path (`HK_VLLM_BACKEND=1`, `_vllm_plugin.register()`) -- and compares the
log-probabilities the two engines assign to the tokens they generate. It exercises, inside the
engine: the metadata builder (work list for prefill steps), the cache write, paged prefill,
paged decode and, with --graphs, decode steps captured by vLLM into CUDA graphs.

With --route the second engine keeps vLLM's own TRITON_ATTN backend and the test covers the
in-place route instead (`HK_VLLM_PREFILL=1`: vLLM's unified_attention rebound to the stand-in).

The engine core runs in this process (VLLM_ENABLE_V1_MULTIPROCESSING=0) so that the backend
registered here is the one it resolves; in a served deployment the `vllm.general_plugins`
entry point does the same in every worker process.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def tiny_config(path: str, heads: int = 8, kv_heads: int = 2) -> None:
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": heads * 128, "head_dim": 128,
        "intermediate_size": 2048, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
        "num_hidden_layers": 2, "vocab_size": 2048, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5,
        "rope_theta": 10000.0, "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16",
        "bos_token_id": 1, "eos_token_id": 2,
    }
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)


def run(model_dir: str, backend, prompts, max_tokens: int, graphs: bool, kv: str, dtype: str = "bfloat16"):
    from vllm import LLM, SamplingParams

    kw = dict(model=model_dir, load_format="dummy", skip_tokenizer_init=True, dtype=dtype, max_model_len=4096,
              gpu_memory_utilization=0.25, enforce_eager=not graphs, seed=0, block_size=16, kv_cache_dtype=kv,
              enable_prefix_caching=False)
    if backend:
        kw["attention_backend"] = backend
    llm = LLM(**kw)
    params = SamplingParams(temperature=0.0, max_tokens=max_tokens, logprobs=1, ignore_eos=True, detokenize=False)
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts], params)
    res = []
    for o in outs:
        c = o.outputs[0]
        res.append((list(c.token_ids), [next(iter(lp.values())).logprob for lp in c.logprobs]))
    del llm
    import gc

    import torch

    gc.collect()
    torch.cuda.empty_cache()
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--graphs", action="store_true", help="let vLLM capture decode steps into CUDA graphs")
    ap.add_argument("--kv", default="auto", help="kv_cache_dtype: auto | fp8")
    ap.add_argument("--max-tokens", type=int, default=24)
    ap.add_argument("--dtype", default="bfloat16", help="the model's dtype: bfloat16 | float16")
    ap.add_argument("--route", action="store_true",
                    help="test the in-place route instead: vLLM keeps its TRITON_ATTN backend and cache, and its "
                         "unified_attention calls are rebound to this build's stand-in (HK_VLLM_PREFILL=1)")
    ap.add_argument("--shadow", action="store_true",
                    help="with --route: HK_VLLM_PREFILL_SHADOW=1, vLLM's own kernel runs beside every taken call "
                         "and the rows are compared in bf16 ulps (eager only)")
    args = ap.parse_args(argv)
    if args.shadow:
        os.environ["HK_VLLM_PREFILL_SHADOW"] = "1"
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ["HK_VLLM_BACKEND"] = "0" if args.route else "1"
    os.environ["HK_VLLM_PREFILL"] = "1" if args.route else "0"

    import torch

    from hk_dsl_b200.integration import _vllm_plugin, vllm_backend, vllm_prefill

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 2000, (n,), generator=g).tolist() for n in (5, 37, 300, 1, 1025, 64)]
    with tempfile.TemporaryDirectory() as d:
        tiny_config(d)
        base = run(d, "TRITON_ATTN" if args.route else None, prompts, args.max_tokens, args.graphs, args.kv, args.dtype)
        _vllm_plugin.register()
        patch = vllm_prefill.PATCH if args.route else vllm_backend.PATCH
        patch.reset()
        ours = run(d, "TRITON_ATTN" if args.route else vllm_backend.SLOT, prompts, args.max_tokens, args.graphs, args.kv, args.dtype)
    stats = dict(patch.stats), dict(patch.captured)
    worst, same = 0.0, 0
    for (tb, lb), (to, lo) in zip(base, ours):
        n = 0
        while n < len(tb) and n < len(to) and tb[n] == to[n]:
            n += 1
        same += n
        for a, b in zip(lb[:max(n, 1)], lo[:max(n, 1)]):
            worst = max(worst, abs(a - b))
    total = sum(len(t) for t, _ in base)
    print(json.dumps({"prompts": len(prompts), "tokens_generated": total, "tokens_identical_prefix": same,
                      "worst_logprob_gap_on_shared_prefix": round(worst, 4), "eager_calls": stats[0],
                      "captured_calls": stats[1], "graphs": args.graphs, "kv_cache_dtype": args.kv, "dtype": args.dtype,
                      "surface": "in-place route (vLLM's TRITON_ATTN backend and cache)" if args.route else "backend",
                      "shadow": dict(vllm_prefill.SHADOW_STATS) if args.shadow else None}))
    ok = stats[0].get("decode", 0) + stats[1].get("decode", 0) > 0 and stats[0].get("prefill", 0) > 0 and worst < 0.1
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
