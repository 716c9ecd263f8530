#!/usr/bin/env python
"""Benchmark of the paged KV hot path: cache write + paged GQA decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the hot path over one batch -- the cache write of every sequence's new
token, the decode walk and the LSE merge -- through `paged.decode_step` (two launches: the walk
writes the new rows itself). The metric is the KV bytes
the decode must read (sum(seq_len) x kv_heads x head_dim x (K + V), tokens counted exactly)
divided by time: KV GB/s, whole job over all ranks. One JSON line is printed by rank 0.

  value     device-timed: inputs resident in HBM, K steps replayed as one CUDA graph that
            rotates over enough distinct caches that a cycle reads >= 1 GiB (cold KV; the
            cache is far larger than L2 in any case), CUDA events, max over ranks.
  roofline  the walk kernel alone: a graph of K walk launches between two CUDA events on the
            launching stream, replayed for about a second.
  e2e       the same step through the public Python API with HOST (pinned) inputs:
            host->device copies of q, k, v, slot_mapping, block_table, seq_lens and the
            device->host read of the output are inside the timed region, every step (the step
            replayed as a CUDA graph; the eager figure is reported beside it).
            The KV cache is the path's persistent state and stays on the device.
  cpu_baseline  the oracle's torch port of the path timed on this box's host cores on a
            bounded sample (rank 0, N=1), also used to check the GPU output of that sample.

`--impl reference` times that CPU port alone (hk-dsl's own kernels are generated HIP for AMD
GPUs and cannot run on this machine; its torch reference code is what can).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "paged decode attn KV GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
#: DRAM bytes moved per algorithmic KV byte by the walk kernel, from the ncu captures
#: summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum of one launch over
#: that launch's KV bytes, on a small case; traffic grows in proportion to the tokens walked).
TRAFFIC_PER_KV_BYTE = {"cc": 1.013, "mma": 1.007}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------ clocks

class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed regions run."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        self.proc = None
        self.marks = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu=timestamp,{self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", gpu_id], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
            out = ""
        rows = []
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                rows.append((float(f[1]), float(f[2]), float(f[3]), f[4:8]))
            except ValueError:
                continue
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        pmax = max(r[2] for r in rows)
        loaded = [r for r in rows if r[2] >= 0.5 * pmax] or rows
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in loaded for n, v in zip(names, r[3]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(r[0] for r in loaded), "sm_max_mhz": rows[0][1],
                "power_w_max": pmax, "samples": len(rows), "samples_under_load": len(loaded), "reasons": reasons}


# ---------------------------------------------------------------------- CPU port timing

def _cpu_sample(spec, lens, budget_tokens):
    """Host tensors of the first sequences of the workload (cut to `budget_tokens` tokens)."""
    import torch

    take, total = [], 0
    for s in lens:
        if total >= budget_tokens:
            break
        s = min(s, max(16, budget_tokens - total))
        take.append(s)
        total += s
    g = torch.Generator().manual_seed(7)
    bs, d, hkv, hq = spec.block_size, spec.head_dim, spec.kv_heads, spec.q_heads
    pages = [-(-s // bs) for s in take]
    nb = sum(pages) + 1
    table = torch.zeros(len(take), max(pages), dtype=torch.int32)
    perm = torch.randperm(nb, generator=g)
    at = 0
    for i, p in enumerate(pages):
        table[i, :p] = perm[at:at + p].to(torch.int32)
        at += p
    k = torch.randn(nb, bs, hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(nb, bs, hkv, d, generator=g).to(torch.bfloat16)
    ks = vs = None
    if spec.fp8:
        from oracle import paged_oracle as orc
        ks = vs = torch.tensor([6.0 / 448.0])
        k, v = orc.quantize_fp8(k, ks), orc.quantize_fp8(v, vs)
    q = torch.randn(len(take), hq, d, generator=g).to(torch.bfloat16)
    kn = torch.randn(len(take), hkv, d, generator=g).to(torch.bfloat16)
    vn = torch.randn(len(take), hkv, d, generator=g).to(torch.bfloat16)
    slots = torch.tensor([int(table[i, (s - 1) // bs]) * bs + (s - 1) % bs for i, s in enumerate(take)])
    return dict(q=q, k=k, v=v, kn=kn, vn=vn, slots=slots, table=table, lens=torch.tensor(take, dtype=torch.int32),
                ks=ks, vs=vs, tokens=total, bytes=total * hkv * d * 2 * spec.kv_elt)


def _cpu_step(spec, c):
    from oracle import paged_oracle as orc

    orc.reshape_and_cache_ref(c["kn"], c["vn"], c["k"], c["v"], c["slots"], spec.kv_cache_dtype, c["ks"], c["vs"])
    return orc.paged_decode_ref_fp32(c["q"], c["k"], c["v"], c["table"], c["lens"], None, c["ks"], c["vs"])


def cpu_port_rate(spec, lens, seconds: float, repeats: int = 3):
    """(GB/s, sample description, cores) of the oracle's fp32 torch port on the host cores."""
    import torch

    cores = torch.get_num_threads()
    probe = _cpu_sample(spec, lens, 4096)
    t0 = time.perf_counter()
    _cpu_step(spec, probe)
    rate = probe["tokens"] / max(time.perf_counter() - t0, 1e-6)          # tokens/s, cold
    budget = int(min(sum(lens), max(4096, rate * seconds / max(1, repeats))))
    c = _cpu_sample(spec, lens, budget)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        _cpu_step(spec, c)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    what = (f"first {len(c['lens'])} sequences ({c['tokens']} tokens, {c['bytes'] / 1e6:.0f} MB of KV) of {spec.name}; "
            f"torch CPU fp32 port of the reference's decode + scatter, median of {repeats}")
    return c["bytes"] / t / 1e9, what, cores


def reference_arm(args):
    """`--impl reference`: the reference's own CPU implementation of the path (its torch
    reference code, restated in oracle/) on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import torch

    from hk_dsl_b200 import workloads as W

    spec = W.CONFIGS[args.config]
    lens = W.seq_lens_of(spec)
    if args.batch:
        lens = lens[:args.batch]
    cores = torch.get_num_threads()
    total_budget_s = 150.0
    probe = _cpu_sample(spec, lens, 4096)
    t0 = time.perf_counter()
    _cpu_step(spec, probe)
    rate = probe["tokens"] / max(time.perf_counter() - t0, 1e-6)
    per_step = total_budget_s / max(1, args.steps + args.warmup)
    c = _cpu_sample(spec, lens, int(min(sum(lens), max(2048, rate * per_step))))
    for _ in range(args.warmup):
        _cpu_step(spec, c)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _cpu_step(spec, c)
    t = (time.perf_counter() - t0) / max(1, args.steps)
    gbs = c["bytes"] / t / 1e9
    sample = (f"each step: first {len(c['lens'])} sequences ({c['tokens']} tokens, {c['bytes'] / 1e6:.0f} MB of KV) "
              f"of {spec.name}, torch CPU fp32")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(spec, lens, 1, "reference torch CPU port"),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "seqs_per_s": len(c["lens"]) / t, "tokens_per_s": len(c["lens"]) / t,
        "note": "hk-dsl's kernels are generated HIP for AMD GPUs; what runs here is its torch reference "
                "(tests/hk/gpu/_attn_ref.py, tools/hk-bench/paged_cdna.py:132-140) restated in oracle/",
    }
    print(json.dumps(line), flush=True)
    return 0


def config_of(spec, lens, world, how):
    return {"workload": f"{spec.name}: {spec.what}", "batch": len(lens), "q_heads": spec.q_heads,
            "kv_heads": spec.kv_heads, "head_dim": spec.head_dim, "block_size": spec.block_size,
            "kv_cache_dtype": "bf16" if not spec.fp8 else "fp8_e4m3", "seq_len_min": min(lens),
            "seq_len_max": max(lens), "total_tokens": sum(lens), "kv_bytes_per_step": spec.kv_bytes(lens),
            "partition": how, "world": world,
            "cold_kv": "inputs larger than L2: every step walks a different cache of a rotation >= 1 GiB"}


# -------------------------------------------------------------------------------- ours

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c2")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--splits", type=int, default=0, help="0 = the planner's choice")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--batch", type=int, default=0,
                    help="keep only the first N sequences of the config (small cases for profiler captures)")
    ap.add_argument("--table", action="store_true",
                    help="decode latency (walk + merge, us a layer) over the reference's requests x context grid")
    ap.add_argument("--prefill", action="store_true",
                    help="paged prefill (the next row of the path): TFLOP/s over a few prompt shapes")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.table:
        return latency_table()
    if args.prefill:
        return prefill_table()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from hk_dsl_b200 import workloads as W
    from hk_dsl_b200.ops import paged, paged_dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the paged KV path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime

        # a rank that never arrives ends the run with an error after two minutes instead of hanging it
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))

    spec = W.CONFIGS[args.config]
    all_lens = W.seq_lens_of(spec)
    if args.batch:
        all_lens = all_lens[:args.batch]
    kv_total = spec.kv_bytes(all_lens)
    # enough distinct caches that one rotation reads >= 1 GiB on this rank
    local_kv = kv_total / world
    layers = max(1, min(16, -(-(1 << 30) // int(max(local_kv, 1)))))
    st = W.build_step(spec, dev, world=world, rank=rank, layers=layers, lens=all_lens)
    n = len(st.lens)
    d = spec.head_dim
    max_tiles = st.block_table.shape[1] * (spec.block_size // 16)
    kvsplit = st.shard.kind == "kvsplit"
    splits = args.splits or paged.plan_splits(n, st.kv_heads, max_tiles, device=dev)
    from hk_dsl_b200.runtime import lib as hkb_lib
    path = "mma" if hkb_lib.load().hkb_walk_uses_mma(spec.q_heads // spec.kv_heads, 1 if spec.fp8 else 0) else "cc"
    dec = None
    if kvsplit:
        dec = paged_dist.SplitKVDecoder(n, st.q_heads, st.kv_heads, d, dev, splits)
        splits = dec.local_splits
    scratch = paged.split_scratch(n, st.q_heads, d, splits, dev) if splits > 1 else None
    # ours; NCCL's not counted. One GPU's step is paged.decode_step: the walk writes the new rows
    # itself (2 launches with the merge); a KV-split step keeps the write apart (write, walk,
    # local merge, merge of the gathered partials)
    joined = not kvsplit and splits > 1 and n <= 2048
    launches_per_step = (2 if joined else 1 + 1 + (1 if splits > 1 else 0)) + (1 if kvsplit else 0)

    def write(l, key=st.key, value=st.value, slots=st.slot_mapping):
        paged.reshape_and_cache(key, value, st.k_caches[l], st.v_caches[l], slots, spec.kv_cache_dtype,
                                st.k_scale, st.v_scale)

    def walk(l, q=st.query, table=st.block_table, lens=st.seq_lens, merge=False):
        if kvsplit:
            dec.local_partial(q, st.k_caches[l], st.v_caches[l], table, lens, st.scale, spec.kv_cache_dtype,
                              st.k_scale, st.v_scale)
            return
        paged.paged_attention_decode(st.out, q, st.k_caches[l], st.v_caches[l], table, lens, st.scale,
                                     spec.kv_cache_dtype, st.k_scale, st.v_scale, num_splits=splits,
                                     scratch=scratch, merge=merge)

    def step(i, **kw):
        l = i % layers
        if kvsplit:
            write(l)
            dec.decode(st.out, st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens, st.scale,
                       spec.kv_cache_dtype, st.k_scale, st.v_scale)
        else:
            paged.decode_step(st.out, st.query, st.key, st.value, st.k_caches[l], st.v_caches[l], st.slot_mapping,
                              st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype, st.k_scale, st.v_scale,
                              num_splits=splits, scratch=scratch)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    props = torch.cuda.get_device_properties(dev)
    gpu_id = f"GPU-{props.uuid}" if getattr(props, "uuid", None) else str(local)
    sampler = ClockSampler(gpu_id) if rank == 0 else None

    K, Wm = args.steps, args.warmup
    for i in range(Wm):
        step(i)
    torch.cuda.synchronize()

    # ---- value: K steps as one CUDA graph, device-timed, max over ranks
    # A step with a collective in it (the KV split's all-gather) is NOT captured: it is timed
    # as K eager launches between the same two events. (A run that captured 100 all-gathers in
    # one graph on 2 GPUs did not finish on this pool; the cause was not established, so the
    # collective stays outside graphs.)
    graph = torch.cuda.CUDAGraph()
    captured = not (kvsplit and world > 1)
    capture_error = None
    if captured:
        try:
            with torch.cuda.graph(graph):
                for i in range(K):
                    step(i)
        except Exception as ex:  # noqa: BLE001
            captured = False
            capture_error = f"{type(ex).__name__}: {str(ex).splitlines()[0][:200]}"
            torch.cuda.synchronize()
    else:
        # the launches either side of the collective are captured (one graph a rotated cache for the
        # write + walk + local merge, one for the merge of the gathered records); the all-gather
        # itself is launched eagerly between them
        capture_error = "collective in the step: its launches either side are graphs, the all-gather is eager"
        pre = []
        for l in range(layers):
            gl = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gl):
                write(l)
                walk(l)
            pre.append(gl)
        post = torch.cuda.CUDAGraph()
        with torch.cuda.graph(post):
            dec.merge(st.out)

        def step(i, **kw):      # noqa: F811  (replaces the eager step for the timed runs)
            pre[i % layers].replay()
            dec.gather()
            post.replay()

    def run_k():
        if captured:
            graph.replay()
        else:
            for i in range(K):
                step(i)

    run_k()                                  # an untimed pass: more warm-up than asked for
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    run_k()
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / K
    value = kv_total / (ms_step * 1e-3) / 1e9

    # ---- roofline: the walk kernel alone -- K launches replayed as one CUDA graph between two
    # events on the launching stream, average = elapsed / K (the gaps between consecutive
    # launches are inside, so the figure is conservative); repeated for about a second so that
    # the clock sampler sees the GPU under this load
    wgraph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(wgraph):
        for i in range(K):
            walk(i % layers)
    wgraph.replay()
    torch.cuda.synchronize()
    walk_ms = []
    t_end = time.perf_counter() + 1.0
    while not walk_ms or (time.perf_counter() < t_end and len(walk_ms) < 200):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        wgraph.replay()
        b.record()
        torch.cuda.synchronize()
        walk_ms.append(a.elapsed_time(b) / K)
    walk_avg_ms = max_over_ranks(statistics.fmean(walk_ms))
    peak, peak_kind = measured_peak()
    achieved = st.kv_bytes / (walk_avg_ms * 1e-3) / 1e9          # this rank's walk over this rank's bytes
    kernel = ("walk_stream_kernel<" if splits > 1 and n <= 2048 else "walk_") + ("StreamCC" if path == "cc" else "WalkMMA")
    roofline = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "traffic": TRAFFIC_PER_KV_BYTE[path] * st.kv_bytes, "algorithmic_bytes": st.kv_bytes,
                "avg_launch_us": walk_avg_ms * 1e3, "launches_timed": len(walk_ms) * K}

    # ---- e2e: the public API with host inputs; H2D of the step's inputs and D2H of its output inside
    # the step's host inputs live in ONE pinned staging buffer (as an engine's input batch does),
    # so a step is one host->device copy; the device tensors the API takes are views of its twin
    names = ("query", "key", "value", "slot_mapping", "block_table", "seq_lens")
    sizes = [(getattr(st, k).numel() * getattr(st, k).element_size() + 255) // 256 * 256 for k in names]
    stage_h = torch.empty(sum(sizes), dtype=torch.uint8).pin_memory()
    stage_d = torch.empty(sum(sizes), dtype=torch.uint8, device=dev)
    devb, at = {}, 0
    for k, sz in zip(names, sizes):
        t = getattr(st, k)
        nb = t.numel() * t.element_size()
        stage_h[at:at + nb].view(t.dtype).view(t.shape).copy_(t.cpu())
        devb[k] = stage_d[at:at + nb].view(t.dtype).view(t.shape)
        at += sz
    out_host = torch.empty(st.out.shape, dtype=st.out.dtype).pin_memory()
    h2d = stage_h.numel()
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step(i):
        l = i % layers
        stage_d.copy_(stage_h, non_blocking=True)
        if kvsplit:
            paged.reshape_and_cache(devb["key"], devb["value"], st.k_caches[l], st.v_caches[l], devb["slot_mapping"],
                                    spec.kv_cache_dtype, st.k_scale, st.v_scale)
            dec.decode(st.out, devb["query"], st.k_caches[l], st.v_caches[l], devb["block_table"],
                       devb["seq_lens"], st.scale, spec.kv_cache_dtype, st.k_scale, st.v_scale)
        else:
            paged.decode_step(st.out, devb["query"], devb["key"], devb["value"], st.k_caches[l], st.v_caches[l],
                              devb["slot_mapping"], devb["block_table"], devb["seq_lens"], st.scale,
                              spec.kv_cache_dtype, st.k_scale, st.v_scale, num_splits=splits, scratch=scratch)
        out_host.copy_(st.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()      # the caller reads the result before the next step

    def timed(fn):
        for i in range(Wm):
            fn(i)
        barrier()
        e0.record()
        for i in range(K):
            fn(i)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / K

    eager_ms = timed(e2e_step)
    e2e_ms, how = eager_ms, "eager: one host->device copy, the API call(s), one device->host copy, a stream sync a step"
    if not (kvsplit and world > 1):
        # The same step as an engine runs it: captured once (a graph a rotated cache) and replayed. A
        # replay performs the host->device copy of the step's inputs from pinned memory, the launches
        # of decode_step and the device->host copy of the result; then the caller syncs and reads.
        try:
            graphs = []
            for l in range(layers):
                gl = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gl):
                    stage_d.copy_(stage_h, non_blocking=True)
                    paged.decode_step(st.out, devb["query"], devb["key"], devb["value"], st.k_caches[l], st.v_caches[l],
                                      devb["slot_mapping"], devb["block_table"], devb["seq_lens"], st.scale,
                                      spec.kv_cache_dtype, st.k_scale, st.v_scale, num_splits=splits, scratch=scratch)
                    out_host.copy_(st.out, non_blocking=True)
                graphs.append(gl)

            def replay_step(i):
                graphs[i % layers].replay()
                torch.cuda.current_stream().synchronize()

            e2e_ms = timed(replay_step)
            how = ("the step (host->device copy of its inputs from pinned memory, decode_step, device->host copy of "
                   "its output) captured as a CUDA graph and replayed, then a stream sync: every replay performs both copies")
        except Exception as ex:  # noqa: BLE001
            how += f" (graph capture of the step failed: {type(ex).__name__})"
            torch.cuda.synchronize()
    e2e = {"value": kv_total / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
           "api": "hk_dsl_b200.ops.paged.decode_step" if not kvsplit else
           "hk_dsl_b200.ops.paged.reshape_and_cache + paged_dist.SplitKVDecoder.decode",
           "how": how, "eager_value": kv_total / (eager_ms * 1e-3) / 1e9, "eager_ms_per_step": eager_ms}

    clocks = sampler.stop() if sampler is not None else None

    # ---- CPU baseline on a bounded sample, and the GPU output of that sample checked against it
    cpu = None
    parity = None
    if rank == 0 and world == 1 and not args.no_cpu:
        gbs, what, cores = cpu_port_rate(spec, all_lens, seconds=15.0)
        cpu = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": what}
        parity = sample_parity(spec, st, splits, scratch)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16" if not spec.fp8 else "fp8_e4m3 KV, bf16 q, fp32 accumulate", "data": "synthetic",
            "config": config_of(spec, all_lens, world,
                                {"single": "one GPU", "heads": "by kv-head group", "seqs": "by sequence",
                                 "kvsplit": "KV axis split across GPUs + all-gather(out, lse) + merge"}[st.shard.kind]),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches_per_step * K, "clocks": clocks,
            "seqs_per_s": len(all_lens) / (ms_step * 1e-3), "tokens_per_s": len(all_lens) / (ms_step * 1e-3),
            "frac_of_aggregate_hbm_measured": value / (peak * world),
            "frac_of_aggregate_hbm_nominal": value / (NOMINAL_HBM_GBS * world),
            "splits": splits, "layers_rotated": layers, "cuda_graph": captured, "parity_sample": parity,
        }
        if not captured:
            line["cuda_graph_error"] = capture_error
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


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


def prefill_table():
    """Paged prefill on 32 q / 8 kv heads, head_dim 128, bf16: causal flops = 4 * q_heads * head_dim *
    sum over query rows of the keys they see; timed with CUDA events, median of 7; against the
    measured bf16 tensor peak (this kernel is the mma.sync form of the contraction)."""
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
    print(json.dumps({"table": "paged prefill, 32q/8kv heads, D128, block 16; mma.sync form", "peak_tflops": peak,
                      "rows": rows}), flush=True)
    return 0


def sample_parity(spec, st, splits, scratch):
    """The GPU answer for the first sequences against the oracle's float64 evaluation (the
    checker leg: nothing of the oracle is timed or shipped here)."""
    import torch

    from hk_dsl_b200.ops import paged
    from oracle import paged_oracle as orc

    take = min(2, len(st.lens))
    paged.decode_step(st.out, st.query, st.key, st.value, st.k_caches[0], st.v_caches[0], st.slot_mapping,
                      st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype, st.k_scale, st.v_scale,
                      num_splits=splits, scratch=scratch)
    torch.cuda.synchronize()
    bs = spec.block_size
    rows = []
    for i in range(take):
        s = st.lens[i]
        pages = st.block_table[i, : -(-s // bs)].long()
        kc = st.k_caches[0][pages].cpu()
        vc = st.v_caches[0][pages].cpu()
        table = torch.arange(kc.shape[0], dtype=torch.int32)[None]
        want = orc.paged_decode_ref(st.query[i:i + 1].cpu(), kc, vc, table, torch.tensor([s], dtype=torch.int32),
                                    st.scale, st.k_scale.cpu() if st.k_scale is not None else None,
                                    st.v_scale.cpu() if st.v_scale is not None else None)
        rows.append((st.out[i:i + 1].float().cpu() - want).abs())
    err = torch.cat(rows)
    return {"sequences": take, "max_abs": err.max().item(), "mean_abs": err.mean().item(),
            "bound": "max-abs 2e-2, mean-abs 2e-3 vs float64 softmax",
            "ok": bool(err.max().item() <= 2e-2 and err.mean().item() <= 2e-3)}


if __name__ == "__main__":
    sys.exit(main())
