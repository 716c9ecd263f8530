"""In-engine A/B: the same requests through vLLM as it ships and through vLLM with this build's
attention backend, on the same GPU, in alternating fresh processes.

    python -m hk_dsl_b200.integration.ab [--arms stock,hk] [--context 1024,4096] [--batch 16,64]
                                         [--layers 8] [--graphs] [--kv fp8] [--json verdicts.json]

What the reference's `python -m hk.integration ab` measures (python/hk/integration/ab.py:1-29):
whether the *request* got faster, not the kernel. Each arm is a fresh engine in a child process
(a backend is chosen when the engine is built and cannot be swapped); arms alternate round by
round and every point is the best of its rounds; a shape gives three times -- the whole batch
for `--tokens` output tokens, for `--short`, and for one (= prefill) -- and steady-state decode
is the slope between the first two, a step at the full batch. The first request's greedy tokens
are compared with stock's. A verdict is `win`, `loss`, `tie` or `noise` against a band taken
from the rounds themselves, never less than 2 %.

There is no network here, so the model is a Llama-3-8B-shaped stack with random ("dummy")
weights and `--layers` layers (attention and GEMM shapes a layer as in the real model; fewer
layers only shorten the run) and the prompts are random token ids.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path
from typing import Dict, List

ROOT = str(Path(__file__).resolve().parents[2])

SHAPES = {
    # hidden, q heads, kv heads, head_dim, intermediate, vocab
    "llama3-8b": (4096, 32, 8, 128, 14336, 128256),
    "qwen3-30b-a3b-attn": (2048, 32, 4, 128, 6144, 151936),       # its attention shape on a dense MLP
    "llama3-70b-attn": (8192, 64, 8, 128, 28672, 128256),
}


def write_config(path: str, shape: str, layers: int, max_len: int) -> None:
    hidden, hq, hkv, d, inter, vocab = SHAPES[shape]
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": hidden, "head_dim": d,
           "intermediate_size": inter, "num_attention_heads": hq, "num_key_value_heads": hkv,
           "num_hidden_layers": layers, "vocab_size": vocab, "max_position_embeddings": max_len,
           "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "hidden_act": "silu", "tie_word_embeddings": False,
           "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)


def one_arm(args) -> Dict:
    """One engine, one arm: its timings for every shape."""
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")     # the backend registered here must be the one used
    os.environ["HK_VLLM_PREFILL"] = "0"
    os.environ["HK_VLLM_BACKEND"] = "1" if args.arm == "hk" else "0"
    import torch
    from vllm import LLM, SamplingParams

    from . import _vllm_plugin, vllm_backend

    backend = None                      # stock: the platform's own choice, not a name
    if args.arm == "hk":
        _vllm_plugin.register()
        backend = vllm_backend.SLOT
    elif args.arm != "stock":
        backend = args.arm              # a vLLM backend's name
    ctxs = [int(x) for x in args.context.split(",")]
    batches = [int(x) for x in args.batch.split(",")]
    out: Dict = {}
    with tempfile.TemporaryDirectory() as d:
        write_config(d, args.shape, args.layers, max(ctxs) + args.tokens + 64)
        t0 = time.perf_counter()
        kw = dict(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
                  max_model_len=max(ctxs) + args.tokens + 64, max_num_seqs=max(batches),
                  gpu_memory_utilization=args.gpu_util, enforce_eager=not args.graphs, seed=0, block_size=16,
                  kv_cache_dtype=args.kv, enable_prefix_caching=False)
        if backend:
            kw["attention_backend"] = backend
        llm = LLM(**kw)
        out["_startup_s"] = round(time.perf_counter() - t0, 1)
        g = torch.Generator().manual_seed(1)
        vocab = SHAPES[args.shape][5]

        def params(n):
            return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True, detokenize=False)

        for n_ctx in ctxs:
            for n_req in batches:
                reqs = [{"prompt_token_ids": torch.randint(3, vocab - 1, (n_ctx,), generator=g).tolist()}
                        for _ in range(n_req)]
                warm = llm.generate(reqs, params(args.tokens), use_tqdm=False)
                got = {"total": [], "short": [], "prefill": []}
                for _ in range(args.reps):
                    for name, n in (("total", args.tokens), ("short", args.short), ("prefill", 1)):
                        t = time.perf_counter()
                        llm.generate(reqs, params(n), use_tqdm=False)
                        got[name].append(time.perf_counter() - t)
                out[f"{n_ctx}x{n_req}"] = {**{k: min(v) for k, v in got.items()}, "reps": got,
                                           "tokens": list(warm[0].outputs[0].token_ids)}
                print(f"  [{args.arm}] ctx {n_ctx} batch {n_req}: {min(got['total']) * 1e3:8.1f} ms total, "
                      f"{min(got['short']) * 1e3:8.1f} ms short, {min(got['prefill']) * 1e3:8.1f} ms prefill", flush=True)
        if args.arm == "hk":
            out["_calls"] = {"eager": dict(vllm_backend.PATCH.stats), "captured": dict(vllm_backend.PATCH.captured)}
    return out


def verdict(ratio: float, band: float) -> str:
    """`ratio` = stock time / arm time. Inside the band nothing was shown: a narrow band makes it a
    tie, a wide one noise."""
    if ratio > 1 + band:
        return "win"
    if ratio < 1 - band:
        return "loss"
    return "tie" if band <= 0.05 else "noise"


def judge(rounds: Dict[str, List[Dict]], tokens: int, short: int) -> List[Dict]:
    """One row a (shape, metric, arm): best-of-rounds times, the ratio to stock, the band, the verdict.
    `rounds[arm]` = that arm's per-round results. The band of a (shape, metric) is the widest
    relative spread between rounds that any arm showed for it, and never under 2 %."""
    def metrics(r):
        return {"total": r["total"], "prefill": r["prefill"], "decode": (r["total"] - r["short"]) / (tokens - short)}

    shapes = [k for k in rounds["stock"][0] if not k.startswith("_")]
    rows = []
    for shape in shapes:
        per = {arm: [metrics(r[shape]) for r in rs if shape in r] for arm, rs in rounds.items()}
        for m in ("total", "prefill", "decode"):
            best = {arm: min(x[m] for x in xs) for arm, xs in per.items() if xs}
            band = 0.02
            for xs in per.values():
                v = [x[m] for x in xs]
                if len(v) > 1 and min(v) > 0:
                    band = max(band, (max(v) - min(v)) / min(v))
            for arm, t in best.items():
                if arm == "stock":
                    continue
                ratio = best["stock"] / t if t > 0 else float("inf")
                rows.append({"shape": shape, "metric": m, "arm": arm, "ms": t * 1e3, "stock_ms": best["stock"] * 1e3,
                             "ratio": ratio, "band": band, "verdict": verdict(ratio, band)})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m hk_dsl_b200.integration.ab", description=__doc__.splitlines()[0])
    ap.add_argument("--arms", default="stock,hk", help="stock is always run; hk = this build's backend; or a vLLM backend name")
    ap.add_argument("--shape", default="llama3-8b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--context", default="1024,4096")
    ap.add_argument("--batch", default="16,64")
    ap.add_argument("--tokens", type=int, default=96)
    ap.add_argument("--short", type=int, default=32)
    ap.add_argument("--reps", type=int, default=2, help="repeats inside an engine")
    ap.add_argument("--rounds", type=int, default=2, help="fresh engines an arm")
    ap.add_argument("--graphs", action="store_true", help="vLLM's CUDA graphs on (enforce_eager off)")
    ap.add_argument("--kv", default="auto", help="kv_cache_dtype: auto | fp8")
    ap.add_argument("--gpu-util", type=float, default=0.6)
    ap.add_argument("--json", default="", help="write the verdict rows here")
    ap.add_argument("--arm", default="", help=argparse.SUPPRESS)
    ap.add_argument("--out", default="", help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if not args.short < args.tokens:
        ap.error("need --short < --tokens for the decode slope")

    if args.arm:                                     # child: one engine
        res = one_arm(args)
        Path(args.out).write_text(json.dumps(res))
        return 0

    arms = ["stock"] + [a for a in args.arms.split(",") if a and a != "stock"]
    base = [sys.executable, "-m", "hk_dsl_b200.integration.ab", "--shape", args.shape, "--layers", str(args.layers),
            "--context", args.context, "--batch", args.batch, "--tokens", str(args.tokens), "--short", str(args.short),
            "--reps", str(args.reps), "--kv", args.kv, "--gpu-util", str(args.gpu_util)] + (["--graphs"] if args.graphs else [])
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join(p for p in (ROOT, env.get("PYTHONPATH", "")) if p)
    rounds: Dict[str, List[Dict]] = {}
    failed: Dict[str, int] = {}
    with tempfile.TemporaryDirectory() as tmp:
        for rnd in range(args.rounds):
            order = arms[rnd % len(arms):] + arms[:rnd % len(arms)]      # no arm always first
            for arm in order:
                f = os.path.join(tmp, f"{arm}_{rnd}.json")
                print(f"--- {arm}, round {rnd}", flush=True)
                r = subprocess.run(base + ["--arm", arm, "--out", f], env=env)
                if r.returncode or not os.path.exists(f):
                    failed[arm] = failed.get(arm, 0) + 1               # a result too; the others still run
                    print(f"--- {arm}, round {rnd}: FAILED, exit {r.returncode}", flush=True)
                    continue
                rounds.setdefault(arm, []).append(json.loads(Path(f).read_text()))
    if "stock" not in rounds:
        print("stock failed every round: nothing to compare against")
        return 1
    rows = judge(rounds, args.tokens, args.short)
    print(f"\n{args.shape}, {args.layers} layers, dummy weights, kv {args.kv}, CUDA graphs {'on' if args.graphs else 'off'}; "
          f"stock = vLLM's own backend = 1.00x; decode = (T({args.tokens}) - T({args.short})) / {args.tokens - args.short} "
          f"a step at the full batch")
    print(f"{'ctx x batch':>12} {'metric':>8} {'arm':>12} {'stock ms':>10} {'arm ms':>10} {'ratio':>7} {'band':>6}  verdict")
    for r in rows:
        print(f"{r['shape']:>12} {r['metric']:>8} {r['arm']:>12} {r['stock_ms']:10.2f} {r['ms']:10.2f} {r['ratio']:6.3f}x "
              f"{r['band'] * 100:5.1f}%  {r['verdict']}")
    same = []
    for arm, rs in rounds.items():
        if arm == "stock":
            continue
        for shape in (k for k in rounds["stock"][0] if not k.startswith("_")):
            ref, got = rounds["stock"][0][shape]["tokens"], rs[0].get(shape, {}).get("tokens", [])
            n = next((i for i, (x, y) in enumerate(zip(ref, got)) if x != y), min(len(ref), len(got)))
            same.append({"arm": arm, "shape": shape, "identical_leading_tokens": n, "of": len(ref)})
    print("leading greedy tokens of the first request identical to stock: "
          + ", ".join(f"{s['arm']} {s['shape']} {s['identical_leading_tokens']}/{s['of']}" for s in same))
    for arm, n in failed.items():
        print(f"{arm}: {n} of {args.rounds} rounds failed")
    calls = {arm: rs[-1].get("_calls") for arm, rs in rounds.items() if rs and rs[-1].get("_calls")}
    if calls:
        print(f"backend calls in the last round: {calls}")
    if args.json:
        Path(args.json).write_text(json.dumps({"rows": rows, "tokens": same, "failed": failed, "calls": calls,
                                               "startup_s": {a: [r.get("_startup_s") for r in rs] for a, rs in rounds.items()}},
                                              indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
