"""Generate the golden fixtures that pin the oracle to the reference's own code.

Run where a checkout of the reference (hk-dsl) is available; its path is the first argument or
the HK_DSL_REFERENCE environment variable. The fixtures travel, the reference does not:

    python tests/golden/make_golden.py /path/to/hk-dsl

What is executed from the reference, unmodified:
  * tests/hk/gpu/_attn_ref.py, loaded by path: `softmax_v64`, `rel`, `ulps` (the float64
    attention reference and the tolerance functions every decode test applies);
  * python/hk/ops/paged.py: the source text of `merge_splits` alone (the module itself needs
    the MLIR bindings to import), executed in an empty namespace;
  * python/hk/integration/switches.py, loaded by path stand-alone (stdlib only): `decide`
    over a grid of environments for the two routes of this path.
Outputs: attn_golden.pt, merge_golden.pt, switches_golden.json beside this script.
"""

from __future__ import annotations

import ast
import importlib.util
import itertools
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HK_DSL_REFERENCE", "")
if not REF or not os.path.isdir(REF):
    sys.exit("usage: python tests/golden/make_golden.py /path/to/hk-dsl")


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def attn_golden():
    ref = load_by_path("_attn_ref_reference", os.path.join(REF, "tests/hk/gpu/_attn_ref.py"))
    g = torch.Generator().manual_seed(20261125)
    page, hkv, group, d = 16, 2, 4, 64
    lens = [1, 17, 40, 16]
    pages = [-(-n // page) for n in lens]
    nb = sum(pages) + 3
    k = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16)
    v = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nb, generator=g)
    table = torch.zeros(len(lens), max(pages), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages):
        table[i, :n] = perm[at:at + n].to(torch.int32)
        at += n
    q = torch.randn(len(lens), hkv * group, d, generator=g).to(torch.bfloat16)
    # the gather of tests/hk/gpu/test_paged_decode.py:89-101, with the reference's own softmax_v64
    out = torch.zeros(len(lens), hkv * group, d, dtype=torch.float32)
    for i, s in enumerate(lens):
        pg = table[i, : -(-s // page)].tolist()
        for hh in range(hkv * group):
            kk = torch.cat([k[p, hh // group] for p in pg])[:s]
            vv = torch.cat([v[p, hh // group] for p in pg])[:s]
            out[i, hh] = ref.softmax_v64(q[i, hh][None], kk, vv, d ** -0.5)[0]
    # causal prefill with a cached prefix, as tests/hk/gpu/test_paged_prefill.py:54-70 builds it:
    # request i's last q_len tokens are the queries, row j at position ctx + j keeps keys <= it
    q_lens = [1, 5, 40, 16]
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    qp = torch.randn(starts[-1], hkv * group, d, generator=g).to(torch.bfloat16)
    outp = torch.zeros(starts[-1], hkv * group, d, dtype=torch.float32)
    for i, s in enumerate(lens):
        n, q0 = q_lens[i], starts[i]
        ctx = s - n
        pg = table[i, : -(-s // page)].tolist()
        keep = torch.arange(s)[None, :] <= (ctx + torch.arange(n))[:, None]
        for hh in range(hkv * group):
            kk = torch.cat([k[p, hh // group] for p in pg])[:s]
            vv = torch.cat([v[p, hh // group] for p in pg])[:s]
            outp[q0:q0 + n, hh] = ref.softmax_v64(qp[q0:q0 + n, hh], kk, vv, d ** -0.5, keep)
    noisy = (out + 3e-3 * torch.randn(out.shape, generator=g)).to(torch.bfloat16)
    torch.save({"q": q, "k": k, "v": v, "table": table, "lens": torch.tensor(lens, dtype=torch.int32),
                "out": out, "noisy": noisy, "prefill_q": qp, "prefill_q_start": torch.tensor(starts, dtype=torch.int32),
                "prefill_out": outp, "rel": ref.rel(noisy, out), "ulps": ref.ulps(noisy, out),
                "ULPS": ref.ULPS, "TOL": ref.TOL}, os.path.join(HERE, "attn_golden.pt"))


def merge_golden():
    src = open(os.path.join(REF, "python/hk/ops/paged.py")).read()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "merge_splits")
    ns = {}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "reference:merge_splits", "exec"), ns)  # noqa: S102
    g = torch.Generator().manual_seed(7)
    reqs, splits, hkv, tile, d = 3, 4, 2, 16, 32
    o = torch.randn(reqs * splits, hkv, tile, d, generator=g)
    ml = torch.empty(reqs * splits, hkv, 2, tile)
    ml[:, :, 0] = 4.0 * torch.randn(reqs * splits, hkv, tile, generator=g)
    ml[:, :, 1] = torch.rand(reqs * splits, hkv, tile, generator=g) * 50 + 0.5
    # one split of request 1 saw nothing: m = -inf, l = 0, numerators 0
    ml[1 * splits + 2, :, 0] = float("-inf")
    ml[1 * splits + 2, :, 1] = 0.0
    o[1 * splits + 2] = 0.0
    out = torch.empty(reqs, hkv, tile, d)
    ns["merge_splits"](o, ml, splits, out)
    torch.save({"o_part": o, "ml_part": ml, "splits": splits, "out": out}, os.path.join(HERE, "merge_golden.pt"))


def switches_golden():
    ref = load_by_path("switches_reference", os.path.join(REF, "python/hk/integration/switches.py"))
    values = ["", "0", "1", "off", "TRUE", "no", "slotname"]
    rows = []
    for dis, master, route in itertools.product(["", "0", "1", "yes"], ["", "0", "1", "false"], values):
        for name in ("vllm_backend", "vllm_prefill"):
            env = {}
            if dis:
                env["HK_DISABLE"] = dis
            if master:
                env["HK_PATCH_VLLM"] = master
            if route:
                env[ref.ROUTES[name].env] = route
            for gpu in ("gfx1100", None):       # a validated arch of the reference, and no GPU
                d = ref.decide(name, env, gpu=gpu)
                rows.append({"route": name, "env": env, "validated_gpu": gpu is not None, "on": d.on,
                             "why": d.why, "value": d.value})
    json.dump({"validated_arch": "gfx1100", "rows": rows}, open(os.path.join(HERE, "switches_golden.json"), "w"),
              indent=0)


if __name__ == "__main__":
    attn_golden()
    merge_golden()
    switches_golden()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith((".pt", ".json"))))
