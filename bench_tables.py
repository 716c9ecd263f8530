#!/usr/bin/env python
"""Measurement tables beside bench.py: sweeps a reader of the profiles can re-run. Nothing
here is part of the bench line.

    python bench_tables.py --latency     decode latency (walk + merge, us a layer) over the reference's
                                         requests x context grid, next to hk-dsl's own published column
    python bench_tables.py --prefill     paged prefill TFLOP/s over a few prompt shapes, against the
                                         measured bf16 tensor peak
    python bench_tables.py --prefill-trace [--case 1x0+8192]
                                         where the tensor-memory prefill kernel's cycles go, by role
    python bench_tables.py --attrib      the decode walk with one stage left out: what each stage costs
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

#: us a layer of hk-dsl's own decode on an MI355X (8 TB/s HBM3e), Qwen3-8B's attention shape, from
#: docs/history/39-cdna-paged.md:163-177 of the reference: (requests, context) -> hk's column.
REFERENCE_MI355X_US = {(1, 512): 9.2, (1, 1024): 9.1, (1, 4096): 13.5, (1, 8192): 16.1, (4, 1024): 9.9,
                       (4, 8192): 28.2, (16, 1024): 17.3, (16, 8192): 88.7, (32, 1024): 25.4, (32, 8192): 171.4,
                       (64, 4096): 167.3, (128, 1024): 84.0, (128, 8192): 659.2}


def _flash_attn_decode_us(st, layers, reps):
    """vLLM's FlashAttention paged decode on token-major copies of the same caches, same graph-replay timing."""
    import torch
    from vllm.vllm_flash_attn import flash_attn_varlen_func as fa

    try:
        kcs = [c.contiguous() for c in st.k_caches[:layers]]
        vcs = [c.contiguous() for c in st.v_caches[:layers]]
        n = st.query.shape[0]
        cu = torch.arange(n + 1, dtype=torch.int32, device=st.query.device)
        out = torch.empty_like(st.query)
        ctx = int(max(st.lens))

        def call(l):
            fa(st.query, kcs[l], vcs[l], max_seqlen_q=1, cu_seqlens_q=cu, max_seqlen_k=ctx, seqused_k=st.seq_lens,
               block_table=st.block_table, causal=True, softmax_scale=st.scale, out=out)

        for l in range(layers):
            call(l)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                for l in range(layers):
                    call(l)
        g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / (reps * layers))
        return statistics.median(times)
    except Exception:  # noqa: BLE001 -- another vLLM, another signature: no column
        torch.cuda.synchronize()
        return None


def latency_table():
    """The reference's kernel-level benchmark of this path (tools/hk-bench/paged_cdna.py decode):
    32 q / 8 kv heads, head_dim 128, bf16, uniform contexts; walk + merge timed as a CUDA graph
    whose calls rotate through enough caches to read past L2 (>= 256 MB a cycle), median of 7."""
    import torch

    from hk_dsl_b200 import workloads as W
    from hk_dsl_b200.ops import paged

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rows = []
    try:        # the FlashAttention paged decode vLLM ships, where a vLLM is installed: the same shapes on the same GPU
        from vllm.vllm_flash_attn import flash_attn_varlen_func  # noqa: F401
        fa_column = True
    except Exception:  # noqa: BLE001
        fa_column = False
    for (reqs, ctx), ref_us in REFERENCE_MI355X_US.items():
        spec = W.Spec(f"t{reqs}x{ctx}", reqs, 32, 8, dist="fixed", lo=ctx, hi=ctx)
        kv = spec.kv_bytes([ctx] * reqs)
        layers = max(2, min(128, -(-(256 << 20) // kv)))
        st = W.build_step(spec, dev, layers=layers, seed=1)
        splits = paged.plan_splits(reqs, 8, st.block_table.shape[1], device=dev)
        scratch = paged.split_scratch(reqs, 32, 128, splits, dev)

        def call(l):
            paged.paged_attention_decode(st.out, st.query, st.k_caches[l], st.v_caches[l], st.block_table,
                                         st.seq_lens, st.scale, num_splits=splits, scratch=scratch)

        for l in range(layers):
            call(l)
        torch.cuda.synchronize()
        reps = max(1, 64 // layers)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                for l in range(layers):
                    call(l)
        g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / (reps * layers))
        us = statistics.median(times)
        row = {"requests": reqs, "context": ctx, "us_per_layer": round(us, 2), "kv_gbs": round(kv / us / 1e3, 1),
               "parts": splits, "caches_rotated": layers, "reference_hk_mi355x_us": ref_us,
               "reference_over_ours": round(ref_us / us, 2)}
        fa_us = _flash_attn_decode_us(st, layers, reps) if fa_column else None
        if fa_us is not None:      # a library kernel on the same GPU, timed the same way: a baseline, not a path of this build
            row["vllm_flash_attn_us"] = round(fa_us, 2)
            row["vllm_flash_attn_over_ours"] = round(fa_us / us, 2)
        rows.append(row)
        del st, scratch, g
        torch.cuda.empty_cache()
    print(json.dumps({"table": "decode walk + merge, us a layer, 32q/8kv heads, D128, bf16, block 16, cold KV, "
                               "CUDA-graph replay, median of 7", "gpu": torch.cuda.get_device_name(dev), "rows": rows}),
          flush=True)
    return 0


def prefill_table(only: str = "", kv: str = "bf16"):
    """Paged prefill on 32 q / 8 kv heads, head_dim 128: causal flops = 4 * q_heads * head_dim *
    sum over query rows of the keys they see; timed with CUDA events, median of 7; against the
    measured bf16 tensor peak. `only` = "RxCTX+QLEN" (e.g. "1x0+8192") runs that one bf16 shape."""
    import torch

    from hk_dsl_b200.ops import paged

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hq, hkv, d, bs = 32, 8, 128, 16
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak = float(json.load(f)["bf16_tflops"])
    except Exception:  # noqa: BLE001
        peak = 1590.0
    rows = []
    g = torch.Generator(device=dev).manual_seed(3)
    cases = [(r, "bf16") for r in ([(0, 2048)], [(0, 8192)], [(0, 2048)] * 8, [(6144, 2048)] * 4, [(0, 512)] * 32)]
    cases += [([(0, 2048)] * 8, "fp16"), ([(0, 2048)] * 8, "fp8")]      # the other cache dtypes, one shape each
    if only:
        reps, _, rest = only.partition("x")
        ctx, _, qlen = rest.partition("+")
        cases = [([(int(ctx), int(qlen))] * int(reps), kv)]
    for reqs, kind in cases:
        seq = [c + n for c, n in reqs]
        pages = [-(-s // bs) for s in seq]
        nb = sum(pages) + 3
        k = torch.randn(nb, hkv, bs, d, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(nb, hkv, bs, d, device=dev, generator=g).to(torch.bfloat16)
        table = torch.zeros(len(reqs), max(pages), dtype=torch.int32)
        perm = torch.randperm(nb)
        at = 0
        for i, p in enumerate(pages):
            table[i, :p] = perm[at:at + p].to(torch.int32)
            at += p
        starts = [0]
        for _, n in reqs:
            starts.append(starts[-1] + n)
        q = torch.randn(starts[-1], hq, d, device=dev, generator=g).to(torch.bfloat16)
        extra = ()
        if kind == "fp16":
            q, k, v = q.to(torch.float16), k.to(torch.float16), v.to(torch.float16)
        elif kind == "fp8":
            one = torch.full((1,), 6.0 / 448.0, device=dev)
            k = (k.float() / one).clamp(-448, 448).to(torch.float8_e4m3fn)
            v = (v.float() / one).clamp(-448, 448).to(torch.float8_e4m3fn)
            extra = ("fp8", one, one)
        out = torch.empty_like(q)
        work = paged.work_list([(r, n) for r, (_, n) in enumerate(reqs)], paged.prefill_tile_rows(hq, hkv), dev,
                               seq_lens=seq)
        args = (out, q, k.transpose(1, 2), v.transpose(1, 2), table.to(dev), torch.tensor(seq, dtype=torch.int32, device=dev),
                torch.tensor(starts, dtype=torch.int32, device=dev), work, d ** -0.5) + extra
        for _ in range(3):
            paged.paged_prefill(*args)
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            paged.paged_prefill(*args)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        ms = statistics.median(times)
        keys_seen = sum(n * c + n * (n + 1) // 2 for c, n in reqs)
        flops = 4.0 * hq * d * keys_seen
        rows.append({"requests": len(reqs), "context": reqs[0][0], "q_len": reqs[0][1], "cache": kind, "ms": round(ms, 3),
                     "tflops": round(flops / ms / 1e9, 1), "frac_of_measured_bf16_peak": round(flops / ms / 1e9 / peak, 3)})
    print(json.dumps({"table": "paged prefill, 32q/8kv heads, D128, block 16", "kernel": "mma.sync" if os.environ.get("HKB_PREFILL_MMA_SYNC") == "1" else "tcgen05 + TMEM", "peak_tflops": peak,
                      "rows": rows}), flush=True)
    return 0


def prefill_trace(case: str, fp8: bool = False):
    """Where the tensor-memory prefill kernel's cycles go on one shape (default 1x0+8192): the traced
    build's per-CTA counters (hkb_paged_prefill_trace), summed over CTAs and divided by the key blocks
    walked -- cycles a 128-key block for each role and phase."""
    import torch

    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    reps, _, rest = (case or "1x0+8192").partition("x")
    ctx, _, qlen = rest.partition("+")
    reqs = [(int(ctx), int(qlen))] * int(reps)
    hq, hkv, d, bs = 32, 8, 128, 16
    g = torch.Generator(device=dev).manual_seed(3)
    seq = [c + n for c, n in reqs]
    pages = [-(-s // bs) for s in seq]
    nb = sum(pages) + 3
    k = torch.randn(nb, hkv, bs, d, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(nb, hkv, bs, d, device=dev, generator=g).to(torch.bfloat16)
    table = torch.zeros(len(reqs), max(pages), dtype=torch.int32)
    perm = torch.randperm(nb)
    at = 0
    for i, p_ in enumerate(pages):
        table[i, :p_] = perm[at:at + p_].to(torch.int32)
        at += p_
    starts = [0]
    for _, n in reqs:
        starts.append(starts[-1] + n)
    q = torch.randn(starts[-1], hq, d, device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    tile = paged.prefill_tile_rows(hq, hkv)
    work = paged.work_list([(r, n) for r, (_, n) in enumerate(reqs)], tile, dev, seq_lens=seq)
    table_d, lens_d = table.to(dev), torch.tensor(seq, dtype=torch.int32, device=dev)
    starts_d = torch.tensor(starts, dtype=torch.int32, device=dev)
    kc, vc = k.transpose(1, 2), v.transpose(1, 2)
    scales = (None, None)
    if fp8:     # the same values as an fp8-e4m3 cache with per-tensor scales
        ks, vs = (k.float().abs().max() / 448.0).reshape(1), (v.float().abs().max() / 448.0).reshape(1)
        kc, vc = (kc.float() / ks).to(torch.float8_e4m3fn), (vc.float() / vs).to(torch.float8_e4m3fn)
        scales = (ks.data_ptr(), vs.data_ptr())
    n_cta = work.shape[0] * hkv
    trace = torch.zeros(n_cta, 32, dtype=torch.int64, device=dev)
    lib = hkb.load()
    cache = lambda c: hkb.CacheT(c.data_ptr(), c.stride(0), c.stride(1), c.stride(2), c.shape[0])
    for _ in range(2):
        rc = lib.hkb_paged_prefill_trace(out.data_ptr(), out.stride(0), out.stride(1), q.data_ptr(), q.stride(0), q.stride(1),
                                         cache(kc), cache(vc), table_d.data_ptr(), table_d.stride(0), table_d.shape[1],
                                         lens_d.data_ptr(), starts_d.data_ptr(), work.data_ptr(), work.shape[0], q.shape[0], hq, hkv, d, bs,
                                         d ** -0.5, hkb.KV_FP8_E4M3 if fp8 else hkb.KV_BF16, scales[0], scales[1], trace.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
        hkb.check("hkb_paged_prefill_trace", rc)
    torch.cuda.synchronize()
    t = trace.cpu().double()
    # key blocks a CTA walks: those of its second query tile (the longer one)
    blocks = 0
    for r, row0 in work.cpu().tolist():
        c, n = reqs[r]
        blocks += -(-min(c + n, c + min(row0 + tile, n)) // 128)
    blocks *= hkv
    names = {0: "softmax tile 0: wait for scores", 1: "softmax tile 0: loads + maximum", 2: "softmax tile 0: exponentials",
             3: "softmax tile 0: wait for previous product (+ rescale)", 4: "softmax tile 0: store P, arrive", 5: "softmax tile 0: epilogue",
             6: "softmax tile 0: staging the query rows", 7: "softmax tile 0: CTA set-up before it",
             8: "softmax tile 1: wait for scores", 9: "softmax tile 1: loads + maximum", 10: "softmax tile 1: exponentials",
             11: "softmax tile 1: wait for previous product (+ rescale)", 12: "softmax tile 1: store P, arrive", 13: "softmax tile 1: epilogue",
             16: "mma: wait for Q", 17: "mma: wait for K", 18: "mma: issue first q.K", 19: "mma: wait for V", 20: "mma: wait for P of tile 0",
             21: "mma: issue p.V", 22: "mma: wait for P of tile 1", 23: "mma: issue the next q.K", 24: "K producer: wait for a free slot", 25: "K producer: issue copies",
             26: "K producer: wait for copies", 27: "K producer (fp8 caches): load staged tile, widen, store", 28: "V producer: wait for a free slot", 29: "V producer: issue copies",
             30: "V producer: wait for copies", 31: "CTA total"}
    rows = {names[i]: round(float(t[:, i].sum()) / blocks, 1) for i in sorted(names)}
    life = t[:, 31][t[:, 31] > 0]          # the persistent grid's CTAs: lifetimes in cycles
    print(json.dumps({"table": "tensor-memory prefill, cycles a 128-key block (both query tiles), by role and phase",
                      "case": case or "1x0+8192", "work_items": n_cta, "ctas": int(life.numel()), "key_blocks": blocks,
                      "cta_lifetime_cycles": {"min": float(life.min()), "mean": round(float(life.mean()), 0),
                                              "max": float(life.max())},
                      "ideal_tensor_cycles_a_block": 2048, "rows": rows}, indent=1), flush=True)
    return 0


def attribution_table():
    """What each stage of the decode walk costs on the headline shape (c2: batch 64, 32 q / 8 kv heads,
    2k-8k tokens, bf16): the walk timed whole and with one stage left out (hkb_paged_decode_ablate),
    each as a CUDA graph of 20 launches over cold caches, median of 7; the difference to the whole walk
    is the stage's cost where stages do not overlap, and an upper bound where they do. The reference
    builds the same table from its `ablate=` switches (tools/hk-bench/paged_attrib.py)."""
    import torch

    from hk_dsl_b200 import workloads as W
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    spec = W.CONFIGS["c2"]
    st = W.build_step(spec, dev)
    n, hq, d = st.query.shape
    splits = paged.plan_splits(n, st.kv_heads, st.block_table.shape[1], device=dev)
    po, pl = paged.split_scratch(n, hq, d, splits, dev)
    lib = hkb.load()
    kc, vc = st.k_caches[0], st.v_caches[0]
    cache = lambda c: hkb.CacheT(c.data_ptr(), c.stride(0), c.stride(1), c.stride(2), c.shape[0])
    stream = torch.cuda.current_stream().cuda_stream

    def launch(mask):
        rc = lib.hkb_paged_decode_ablate(st.out.data_ptr(), st.out.stride(0), st.out.stride(1), st.query.data_ptr(),
                                         st.query.stride(0), st.query.stride(1), cache(kc), cache(vc),
                                         st.block_table.data_ptr(), st.block_table.stride(0), st.block_table.shape[1],
                                         st.seq_lens.data_ptr(), None, n, hq, st.kv_heads, d, spec.block_size, st.scale,
                                         hkb.KV_BF16, None, None, splits, po.data_ptr(), pl.data_ptr(), mask,
                                         torch.cuda.current_stream().cuda_stream)
        hkb.check("hkb_paged_decode_ablate", rc)

    names = {0: "the whole walk", 1: "without the page-table reads", 2: "without the K copies", 4: "without the V copies",
             6: "without any copy (math on stale tiles)", 8: "without the q.K products", 16: "without the softmax",
             32: "without the p.V products", 56: "without any math (copies only)"}
    rows, whole = [], None
    for mask, what in names.items():
        for _ in range(3):
            launch(mask)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(20):
                launch(mask)
        g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / 20)
        us = statistics.median(times)
        whole = us if mask == 0 else whole
        rows.append({"mask": mask, "walk": what, "us": round(us, 2), "saves_us": round(whole - us, 2),
                     "kv_gbs_if_all_bytes_moved": round(st.kv_bytes / us / 1e3, 1)})
    del stream
    print(json.dumps({"table": "decode walk on c2 with one stage left out, us a launch (cold KV, graph of 20, median of 7)",
                      "kv_bytes": st.kv_bytes, "splits": splits, "rows": rows}, indent=1), flush=True)
    return 0


def shards_table():
    """One rank's share of the headline config (c2) cut by kv head over 1, 2, 4 and 8 GPUs, run on
    ONE GPU: the decode step (`decode_step`: the walk writes the new rows, then the merge) and its
    one-launch form (the walk also folds: `arrivals`), as a graph of 20 steps rotating through caches
    past L2, median of 7. `of_ideal` = (the world-1 step / world) / this step: what the fixed costs of
    a step -- launches, the walk's ramp and tail, the merge -- leave of perfect strong scaling."""
    import torch

    from hk_dsl_b200 import workloads as W
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    spec = W.CONFIGS["c2"]
    rows, base = [], None
    for world in (1, 2, 4, 8):
        kv1 = spec.kv_bytes(W.seq_lens_of(spec, int(spec.name[1:]))) // world
        layers = max(2, min(16, -(-(300 << 20) // kv1)))
        st = W.build_step(spec, dev, world=world, rank=0, layers=layers)
        n, hq, d = st.query.shape
        splits = paged.plan_splits(n, st.kv_heads, st.block_table.shape[1], device=dev)
        scratch = paged.split_scratch(n, hq, d, splits, dev)
        row = {"world": world, "kv_heads_here": st.kv_heads, "kv_bytes": st.kv_bytes, "parts": splits, "caches_rotated": layers}
        for name, arrivals in (("two_launches", None), ("one_launch", paged.step_arrivals(n, st.kv_heads, dev))):
            def call(l):
                paged.decode_step(st.out, st.query, st.key, st.value, st.k_caches[l], st.v_caches[l], st.slot_mapping,
                                  st.block_table, st.seq_lens, st.scale, num_splits=splits, scratch=scratch,
                                  arrivals=arrivals)
            for l in range(layers):
                call(l)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(20):
                    call(i % layers)
            g.replay()
            torch.cuda.synchronize()
            times = []
            for _ in range(7):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) * 1e3 / 20)
            us = statistics.median(times)
            row[name + "_us"] = round(us, 2)
            row[name + "_kv_gbs"] = round(st.kv_bytes / us / 1e3, 1)
            del g
        # the walk alone (cache already written, no merge), and the walk with its math left out: the copies' floor
        lib, cache = hkb.load(), (lambda c: hkb.CacheT(c.data_ptr(), c.stride(0), c.stride(1), c.stride(2), c.shape[0]))

        def walk(l, mask):
            if mask == 0:
                paged.paged_attention_decode(st.out, st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens,
                                             st.scale, num_splits=splits, scratch=scratch, merge=False)
                return
            rc = lib.hkb_paged_decode_ablate(st.out.data_ptr(), st.out.stride(0), st.out.stride(1), st.query.data_ptr(),
                                             st.query.stride(0), st.query.stride(1), cache(st.k_caches[l]), cache(st.v_caches[l]),
                                             st.block_table.data_ptr(), st.block_table.stride(0), st.block_table.shape[1],
                                             st.seq_lens.data_ptr(), None, n, hq, st.kv_heads, d, spec.block_size, st.scale,
                                             hkb.KV_BF16, None, None, splits, scratch[0].data_ptr(), scratch[1].data_ptr(), mask,
                                             torch.cuda.current_stream().cuda_stream)
            hkb.check("hkb_paged_decode_ablate", rc)

        for name, mask in (("walk_only", 0), ("copies_only", 56)):
            for l in range(layers):
                walk(l, mask)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(20):
                    walk(i % layers, mask)
            g.replay()
            torch.cuda.synchronize()
            times = []
            for _ in range(7):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) * 1e3 / 20)
            row[name + "_us"] = round(statistics.median(times), 2)
            del g
        if world == 1:
            base = min(row["two_launches_us"], row["one_launch_us"])
        row["of_ideal_two_launches"] = round(base / world / row["two_launches_us"], 3)
        row["of_ideal_one_launch"] = round(base / world / row["one_launch_us"], 3)
        rows.append(row)
        del st, scratch
        torch.cuda.empty_cache()
    print(json.dumps({"table": "c2 cut by kv head: one rank's decode step on one GPU, us a step (cold KV, graph of 20, median of 7)",
                      "rows": rows}, indent=1), flush=True)
    return 0


def exchange_table(only: str = ""):
    """The KV-split step's exchange on ONE GPU (the rank is its own only peer: no NVLink in it, the
    kernels' own cost): the long-context config's shape (c5: 2 sequences x 131072 tokens, 32 q / 8 kv
    heads, 256 local splits), walk then exchange in one launch (hkb_kvsplit_exchange) or in two
    (hkb_kvsplit_push, hkb_kvsplit_merge), each a graph of 20 steps, median of 7. `only`: "one" or
    "two", a short eager run for a profiler."""
    import torch

    from hk_dsl_b200 import workloads as W
    from hk_dsl_b200.ops import paged, paged_dist

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    spec = W.CONFIGS["c5"]
    st = W.build_step(spec, dev)
    n, hq, d = st.query.shape
    splits = paged.plan_splits(n, st.kv_heads, st.block_table.shape[1], device=dev)
    rows = []
    for name, exchange in (("one", "peer"), ("two", "peer2")):
        if only and only != name:
            continue
        dec = paged_dist.SplitKVDecoder(n, hq, st.kv_heads, d, dev, splits, exchange=exchange)

        def step():
            dec.decode(st.out, st.query, st.k_caches[0], st.v_caches[0], st.block_table, st.seq_lens, st.scale,
                       key=st.key, value=st.value, slot_mapping=st.slot_mapping)

        def walk():
            paged.decode_step_record(None, None, st.query, st.key, st.value, st.k_caches[0], st.v_caches[0], st.slot_mapping,
                                     st.block_table, st.seq_lens, st.scale, num_splits=dec.local_splits, scratch=dec.scratch)

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if only:
            return 0
        us = {}
        for what, call in (("step", step), ("walk", walk)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(20):
                    call()
            g.replay()
            torch.cuda.synchronize()
            times = []
            for _ in range(7):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) * 1e3 / 20)
            us[what] = statistics.median(times)
            del g
        assert dec.peer.error() == 0
        rows.append({"exchange": "one launch" if name == "one" else "two launches", "step_us": round(us["step"], 2),
                     "walk_us": round(us["walk"], 2), "exchange_us": round(us["step"] - us["walk"], 2)})
    print(json.dumps({"table": "c5 on one GPU as a KV split of one rank: walk + exchange, us a step (graph of 20, median of 7)",
                      "local_splits": splits, "rows": rows}, indent=1), flush=True)
    return 0


def layouts_table(only: str = ""):
    """The decode (walk + merge) on the headline shape (c2) over the same KV values in the two cache
    layouts the walk reads in place: (blocks, page, kv_heads, head_dim) and vLLM's x-split pair
    (K (blocks, kv_heads, head_dim / 8, page, 8), V^T (blocks, kv_heads, head_dim, page)). Graph of 20
    launches over KV larger than L2, median of 7; the two answers are compared bit for bit. `only`:
    one layout ("nhd" or "x-split"), a short run for a profiler."""
    import torch

    from hk_dsl_b200 import workloads as W
    from hk_dsl_b200.ops import paged

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    spec = W.CONFIGS["c2"]
    st = W.build_step(spec, dev)
    n, hq, d = st.query.shape
    splits = paged.plan_splits(n, st.kv_heads, st.block_table.shape[1], device=dev)
    scratch = paged.split_scratch(n, hq, d, splits, dev)
    kc, vc = st.k_caches[0], st.v_caches[0]
    k5, v4 = paged.x_split_caches(kc, vc)
    outs = {"nhd": torch.empty_like(st.out), "x-split": torch.empty_like(st.out)}
    calls = {
        "nhd": lambda: paged.paged_attention_decode(outs["nhd"], st.query, kc, vc, st.block_table, st.seq_lens, st.scale,
                                                    num_splits=splits, scratch=scratch),
        "x-split": lambda: paged.paged_attention_decode_xsplit(outs["x-split"], st.query, k5, v4, st.block_table,
                                                               st.seq_lens, st.scale, num_splits=splits, scratch=scratch),
    }
    rows = []
    if only:
        for _ in range(3):
            calls[only]()
        torch.cuda.synchronize()
        return 0
    for name, call in calls.items():
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(20):
                call()
        g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / 20)
        us = statistics.median(times)
        rows.append({"layout": name, "us": round(us, 2), "kv_gbs": round(st.kv_bytes / us / 1e3, 1)})
    same = bool(torch.equal(outs["nhd"].view(torch.int16), outs["x-split"].view(torch.int16)))
    print(json.dumps({"table": "decode (walk + merge) on c2 by cache layout, us a step (cold KV, graph of 20, median of 7)",
                      "kv_bytes": st.kv_bytes, "splits": splits, "answers_bitwise_equal": same, "rows": rows}, indent=1),
          flush=True)
    return 0 if same else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--latency", action="store_true")
    ap.add_argument("--prefill", action="store_true")
    ap.add_argument("--case", default="", help="with --prefill: one shape, REQUESTSxCONTEXT+QLEN; with --layouts: nhd or "
                                               "x-split (a small case for a profiler)")
    ap.add_argument("--prefill-trace", action="store_true", help="cycles by role and phase of the tensor-memory prefill kernel")
    ap.add_argument("--attrib", action="store_true", help="the decode walk with one stage left out: what each stage costs")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8"], help="with --prefill-trace, or --prefill --case: the cache type")
    ap.add_argument("--exchange", action="store_true", help="the KV-split exchange kernels on one GPU (one launch against two)")
    ap.add_argument("--shards", action="store_true", help="one rank's share of c2 over 1/2/4/8 GPUs, on one GPU: the step's fixed costs")
    ap.add_argument("--layouts", action="store_true", help="the decode over the usual and the x-split cache layout")
    args = ap.parse_args()
    if args.exchange:
        return exchange_table(args.case)
    if args.shards:
        return shards_table()
    if args.layouts:
        return layouts_table(args.case)
    if args.attrib:
        return attribution_table()
    if args.prefill_trace:
        return prefill_trace(args.case, args.kv == "fp8")
    if args.prefill:
        return prefill_table(args.case, args.kv)
    return latency_table()


if __name__ == "__main__":
    sys.exit(main())
