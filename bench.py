#!/usr/bin/env python
"""Benchmark of the paged KV hot path: cache write + paged GQA decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c2] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the hot path over one batch -- the cache write of every sequence's new
token, the decode walk and the LSE merge -- through `paged.decode_step` (two launches: the walk
writes the new rows itself). The metric is the KV bytes the decode must read
(sum(seq_len) x kv_heads x head_dim x (K + V), tokens counted exactly) divided by time:
KV GB/s, whole job over all ranks. One JSON line is printed by rank 0.

  value     device-timed: inputs resident in HBM, K steps replayed as one CUDA graph that
            rotates over enough distinct caches that a cycle reads >= 1 GiB (the KV of a step is
            larger than L2 in any case), CUDA events, max over ranks; the median of 7 replays
            (`rounds`, with min and max beside it).
  roofline  the walk kernel alone: a graph of K walk launches between two CUDA events on the
            launching stream, replayed for about a second; against the measured copy peak, the
            nominal 8 TB/s and this build's own read-only streaming probe.
  e2e       the same step through the public Python API with HOST (pinned) inputs:
            host->device copies of q, k, v, slot_mapping, block_table, seq_lens and the
            device->host read of the output are inside the timed region, every step (the step
            replayed as a CUDA graph; the eager figure is reported beside it).
            The KV cache is the path's persistent state and stays on the device.
  cpu_baseline  the oracle's torch port of the path timed on this box's host cores on a
            bounded sample (rank 0, N=1).
  parity    at every N, every rank: the step's output for the whole local batch against the
            oracle's fp32 evaluation, and for a few sequences against its float64 evaluation;
            a KV axis cut across GPUs compares the merged answer with the float64 fold of the
            ranks' float64 partials.
  configs   after the headline workload (c2) the other measured configurations (c3, c4, c5) run
            briefly with the same method; their value, roofline fraction, partition and parity
            are attached under "configs". `--only` skips them.

`--impl reference` times the CPU port alone (hk-dsl's own kernels are generated HIP for AMD
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
ROUNDS = 7
#: DRAM bytes moved per algorithmic KV byte by the walk kernel of a (config, worker):
#: dram__bytes_read.sum + dram__bytes_write.sum of one launch over that launch's KV bytes, from an
#: ncu capture of a small case of that config (traffic grows in proportion to the tokens
#: walked: every tile is read once). None: no capture of that pair.
TRAFFIC_PER_KV_BYTE = {("c2", "mma"): 1.013, ("c2", "cc"): 1.014, ("c3", "mma"): 1.05, ("c3", "cc"): 1.03,
                       ("c5", "mma"): 1.007}
PARTITION = {"single": "one GPU", "heads": "by kv-head group", "seqs": "by sequence",
             "kvsplit": "KV axis split across GPUs + exchange of (out, lse) + merge"}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, "fallback"


def host_cores() -> int:
    """Cores this process may use: the physical cores of the box, within its affinity mask.
    A launcher's OMP_NUM_THREADS (torch.distributed.run exports 1) does not count."""
    try:
        usable = len(os.sched_getaffinity(0))
    except AttributeError:
        usable = os.cpu_count() or 1
    try:
        import psutil

        phys = psutil.cpu_count(logical=False) or usable
    except Exception:  # noqa: BLE001
        phys = usable
    return max(1, min(usable, phys))


# ------------------------------------------------------------------------------ clocks

class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed regions run."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        self.proc = None
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
    kn = torch.randn(len(take), hkv, d, generator=g).to(torch.bfloat16)
    vn = torch.randn(len(take), hkv, d, generator=g).to(torch.bfloat16)
    ks = vs = None
    if spec.fp8:
        from oracle import paged_oracle as orc
        ks = (torch.maximum(k.float().abs().max(), kn.float().abs().max()) / 448.0).reshape(1)
        vs = (torch.maximum(v.float().abs().max(), vn.float().abs().max()) / 448.0).reshape(1)
        k, v = orc.quantize_fp8(k, ks), orc.quantize_fp8(v, vs)
    q = torch.randn(len(take), hq, d, generator=g).to(torch.bfloat16)
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

    cores = host_cores()
    torch.set_num_threads(cores)
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
    reference code, restated in oracle/) on the host cores; rank 0 only, on every core of the
    box whatever thread count the launcher exported."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import torch

    from hk_dsl_b200 import workloads as W

    spec = W.CONFIGS[args.config]
    lens = W.seq_lens_of(spec)
    if args.batch:
        lens = lens[:args.batch]
    cores = host_cores()
    torch.set_num_threads(cores)
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
              f"of {spec.name}, torch CPU fp32, {cores} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": dtype_of(spec), "data": "synthetic",
        "config": config_of(spec, lens),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "seqs_per_s": len(c["lens"]) / t, "tokens_per_s": len(c["lens"]) / t,
        "arithmetic": "the CPU port evaluates in fp32 on the bf16 / fp8 inputs",
        "note": "hk-dsl's kernels are generated HIP for AMD GPUs; what runs here is its torch reference "
                "(tests/hk/gpu/_attn_ref.py, tools/hk-bench/paged_cdna.py:132-140) restated in oracle/",
    }
    print(json.dumps(line), flush=True)
    return 0


def dtype_of(spec) -> str:
    return "bf16" if not spec.fp8 else "fp8_e4m3 KV, bf16 q, fp32 accumulate"


def config_of(spec, lens):
    """The workload, the same dict from either arm (how a run partitions it is reported beside it)."""
    return {"workload": f"{spec.name}: {spec.what}", "batch": len(lens), "q_heads": spec.q_heads,
            "kv_heads": spec.kv_heads, "head_dim": spec.head_dim, "block_size": spec.block_size,
            "kv_cache_dtype": "bf16" if not spec.fp8 else "fp8_e4m3", "seq_len_min": min(lens),
            "seq_len_max": max(lens), "total_tokens": sum(lens), "kv_bytes_per_step": spec.kv_bytes(lens),
            "cold_kv": "inputs larger than L2: the KV a step reads is several times the 126 MB L2"}


# -------------------------------------------------------------------------------- ours

class Ctx:
    """What every leg of a run shares: the process group, the device, timing helpers."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the paged KV path has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import datetime

            # a rank that never arrives ends the run with an error after two minutes instead of hanging it
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=120))
        self.peak, self.peak_kind = measured_peak()
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed_ms(self, fn) -> float:
        """fn() between two events on the current stream, a barrier and a device sync either side; max over ranks."""
        self.barrier()
        self.e0.record()
        fn()
        self.e1.record()
        self.barrier()
        return self.max_over_ranks(self.e0.elapsed_time(self.e1))


def read_probe(ctx, seconds: float = 3.0):
    """This build's read-only streaming probe (hkb_hbm_read_probe): four rotating 512 MB buffers,
    a sweep of CTAs an SM x loads in flight a thread, best GB/s of a launch (CUDA events)."""
    torch = ctx.torch
    from hk_dsl_b200.runtime import lib as hkb

    lib = hkb.load()
    nbytes = 512 << 20
    bufs = [torch.full((nbytes,), 0x5a, dtype=torch.uint8, device=ctx.dev) for _ in range(4)]
    sink = torch.zeros(4, dtype=torch.int32, device=ctx.dev)
    st = torch.cuda.current_stream().cuda_stream
    best, how, bi = 0.0, None, 0
    t_end = time.perf_counter() + seconds
    for ctas in (1, 2, 4, 8):
        for inflight in (2, 4, 8, 16):
            if time.perf_counter() > t_end and best > 0:
                break
            for _ in range(2):
                hkb.check("hkb_hbm_read_probe", lib.hkb_hbm_read_probe(bufs[bi % 4].data_ptr(), nbytes, ctas, inflight,
                                                                       sink.data_ptr(), st))
                bi += 1
            ms = []
            for _ in range(6):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                lib.hkb_hbm_read_probe(bufs[bi % 4].data_ptr(), nbytes, ctas, inflight, sink.data_ptr(), st)
                b.record()
                torch.cuda.synchronize()
                ms.append(a.elapsed_time(b))
                bi += 1
            gbs = nbytes / (min(ms) * 1e-3) / 1e9
            if gbs > best:
                best, how = gbs, {"ctas_per_sm": ctas, "loads_in_flight": inflight}
    del bufs
    torch.cuda.empty_cache()
    return {"gbs": best, "bytes_a_launch": nbytes, "buffers_rotated": 4, "best_at": how,
            "what": "read-only 16-byte loads, best launch of the sweep (hkb_hbm_read_probe)"}


def run_config(ctx, name: str, *, headline: bool, probe_gbs=None):
    """Build one configuration on this rank and measure it; returns rank 0's record (None elsewhere)."""
    torch, dist, args = ctx.torch, ctx.dist, ctx.args
    from hk_dsl_b200 import workloads as W
    from hk_dsl_b200.ops import paged, paged_dist
    from hk_dsl_b200.runtime import lib as hkb_lib

    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    spec = W.CONFIGS[name]
    all_lens = W.seq_lens_of(spec)
    if args.batch and headline:
        all_lens = all_lens[:args.batch]
    kv_total = spec.kv_bytes(all_lens)
    K = args.steps if headline else max(3, min(args.steps, 20))
    Wm = args.warmup
    # enough distinct caches that one rotation reads >= 1 GiB on this rank
    local_kv = kv_total / world
    layers = max(1, min(16, -(-(1 << 30) // int(max(local_kv, 1)))))
    st = W.build_step(spec, dev, world=world, rank=rank, layers=layers, lens=all_lens)
    n = len(st.lens)
    d = spec.head_dim
    max_tiles = st.block_table.shape[1] * (spec.block_size // 16)
    kvsplit = st.shard.kind == "kvsplit"
    splits = args.splits or paged.plan_splits(n, st.kv_heads, max_tiles, device=dev)
    path = "mma" if hkb_lib.load().hkb_walk_uses_mma(spec.q_heads // spec.kv_heads, 1 if spec.fp8 else 0) else "cc"
    dec = None
    exchange = None
    if kvsplit:
        # the ranks' records go over peer memory (one kernel of this build after the walk, no collective) where the
        # box maps it; HKB_KVSPLIT_EXCHANGE=nccl, or a box that cannot, takes the all-gather
        exchange = os.environ.get("HKB_KVSPLIT_EXCHANGE", "peer")
        try:
            dec = paged_dist.SplitKVDecoder(n, st.q_heads, st.kv_heads, d, dev, splits, exchange=exchange)
        except Exception as ex:  # noqa: BLE001
            if not exchange.startswith("peer"):
                raise
            exchange = f"nccl (peer memory unavailable: {type(ex).__name__}: {str(ex).splitlines()[0][:120]})"
            dec = paged_dist.SplitKVDecoder(n, st.q_heads, st.kv_heads, d, dev, splits, exchange="nccl")
        if world > 1:       # every rank takes the same path
            flag = torch.tensor([1 if dec.peer is not None else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if dec.peer is not None and int(flag.item()) == 0:
                exchange = "nccl (peer memory unavailable on another rank)"
                dec = paged_dist.SplitKVDecoder(n, st.q_heads, st.kv_heads, d, dev, splits, exchange="nccl")
        splits = dec.local_splits
    scratch = paged.split_scratch(n, st.q_heads, d, splits, dev) if splits > 1 else None
    owns_new = bool((st.slot_mapping >= 0).any().item())
    # this build's launches a step; NCCL's are not counted. One GPU's step is paged.decode_step: the
    # walk writes the new rows itself, then the merge. A KV-split step: walk (+ rows), merge of the
    # local splits into this rank's record, [exchange], merge of the ranks' records.
    joined = not kvsplit and splits > 1 and n <= 2048
    launches_per_step = (2 if exchange == "peer" and dec is not None and dec.peer is not None else 3) if kvsplit else (2 if joined else 1 + 1 + (1 if splits > 1 else 0))

    def walk(l):
        if kvsplit:
            dec.walk(st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens, st.scale,
                     spec.kv_cache_dtype, st.k_scale, st.v_scale)
            return
        paged.paged_attention_decode(st.out, st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens,
                                     st.scale, spec.kv_cache_dtype, st.k_scale, st.v_scale, num_splits=splits,
                                     scratch=scratch, merge=False)

    def new_rows():
        return dict(key=st.key, value=st.value, slot_mapping=st.slot_mapping) if owns_new else {}

    def step(i):
        l = i % layers
        if kvsplit:
            dec.decode(st.out, st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens, st.scale,
                       spec.kv_cache_dtype, st.k_scale, st.v_scale, **new_rows())
        else:
            paged.decode_step(st.out, st.query, st.key, st.value, st.k_caches[l], st.v_caches[l], st.slot_mapping,
                              st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype, st.k_scale, st.v_scale,
                              num_splits=splits, scratch=scratch)

    for i in range(Wm):
        step(i)
    torch.cuda.synchronize()

    # ---- value: K steps as one CUDA graph, device-timed, max over ranks, median of ROUNDS replays.
    # A step with a collective in it (the KV split's exchange) keeps the collective outside graphs:
    # the launches either side of it are captured (one graph a rotated cache for the walk + the
    # local merge, one for the merge of the gathered records) and the all-gather is launched
    # eagerly between them.
    peer = kvsplit and dec.peer is not None
    captured = not (kvsplit and world > 1) or peer      # a step without a collective is captured whole
    capture_note = None
    graph = torch.cuda.CUDAGraph()
    if captured:
        try:
            with torch.cuda.graph(graph):
                for i in range(K):
                    step(i)
        except Exception as ex:  # noqa: BLE001
            captured = False
            capture_note = f"{type(ex).__name__}: {str(ex).splitlines()[0][:200]}"
            torch.cuda.synchronize()

        def run_k():
            if captured:
                graph.replay()
            else:
                for i in range(K):
                    step(i)
    else:
        capture_note = "collective in the step: its launches either side are graphs, the all-gather is eager"
        pre = []
        for l in range(layers):
            gl = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gl):
                dec.local_partial(st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens, st.scale,
                                  spec.kv_cache_dtype, st.k_scale, st.v_scale, **new_rows())
            pre.append(gl)
        post = torch.cuda.CUDAGraph()
        with torch.cuda.graph(post):
            dec.merge(st.out)

        def run_k():
            for i in range(K):
                pre[i % layers].replay()
                dec.gather()
                post.replay()

    run_k()                                  # an untimed pass: more warm-up than asked for
    round_ms = [ctx.timed_ms(run_k) / K for _ in range(ROUNDS)]
    ms_step = statistics.median(round_ms)
    value = kv_total / (ms_step * 1e-3) / 1e9

    # ---- roofline: the walk kernel alone -- K launches replayed as one CUDA graph between two
    # events on the launching stream, average = elapsed / K (the gaps between consecutive launches
    # are inside, so the figure is conservative); repeated for about a second (headline) so that the
    # clock sampler sees the GPU under this load
    wgraph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(wgraph):
        for i in range(K):
            walk(i % layers)
    wgraph.replay()
    torch.cuda.synchronize()
    walk_ms = []
    t_end = time.perf_counter() + (1.0 if headline else 0.3)
    while not walk_ms or (time.perf_counter() < t_end and len(walk_ms) < 200):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        wgraph.replay()
        b.record()
        torch.cuda.synchronize()
        walk_ms.append(a.elapsed_time(b) / K)
    mine = statistics.fmean(walk_ms)
    walk_avg_ms = ctx.max_over_ranks(mine)
    # the rank with the slowest walk reports its own bytes over its own time
    slow_bytes = st.kv_bytes
    if world > 1:
        t = torch.tensor([mine, float(st.kv_bytes)], device=dev, dtype=torch.float64)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        slow_bytes = max(every, key=lambda x: float(x[0]))[1].item()
    achieved = slow_bytes / (walk_avg_ms * 1e-3) / 1e9
    stream = splits > 1 and n <= 2048
    kernel = ("walk_stream_kernel<" if stream else "walk_") + ("StreamCC" if path == "cc" else
                                                               ("WalkMMAF8" if spec.fp8 and stream else "WalkMMA"))
    ratio = TRAFFIC_PER_KV_BYTE.get((name, path))
    roofline = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": ctx.peak,
                "unit": "GB/s", "frac": achieved / ctx.peak, "peak_kind": f"of {ctx.peak_kind}",
                "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                "traffic": ratio * slow_bytes if ratio else None, "algorithmic_bytes": slow_bytes,
                "avg_launch_us": walk_avg_ms * 1e3, "launches_timed": len(walk_ms) * K}
    if probe_gbs:
        roofline["read_probe_gbs"] = probe_gbs
        roofline["frac_of_read_probe"] = achieved / probe_gbs

    rec = {"value": value, "unit": "GB/s", "ms_per_step": ms_step, "rounds": ROUNDS,
           "ms_per_step_min": min(round_ms), "ms_per_step_max": max(round_ms), "steps": K,
           "dtype": dtype_of(spec), "config": config_of(spec, all_lens), "partition": PARTITION[st.shard.kind],
           "world": world, "roofline": roofline, "gpu_launches": launches_per_step * K * ROUNDS,
           "launches_per_step": launches_per_step,
           "seqs_per_s": len(all_lens) / (ms_step * 1e-3), "tokens_per_s": len(all_lens) / (ms_step * 1e-3),
           "frac_of_aggregate_hbm_measured": value / (ctx.peak * world),
           "frac_of_aggregate_hbm_nominal": value / (NOMINAL_HBM_GBS * world),
           "splits": splits, "cuda_graph": captured,
           "cold_kv_detail": {"layers_rotated": layers, "kv_bytes_a_step_this_rank": st.kv_bytes,
                              "bytes_a_rotation_this_rank": st.kv_bytes * layers}}
    if capture_note:
        rec["cuda_graph_note"] = capture_note
    if kvsplit:
        rec["exchange"] = exchange if not peer else "peer memory: hkb_kvsplit_push + hkb_kvsplit_merge, no collective"
        if peer:
            rec["exchange_error_word"] = dec.peer.error()
    if kvsplit and world > 1:
        rec["breakdown_us"] = (peer_breakdown if peer else kvsplit_breakdown)(ctx, spec, st, dec, layers, K, owns_new)

    if headline:
        rec["e2e"] = e2e_leg(ctx, spec, st, dec, layers, splits, scratch, kv_total, K, Wm, kvsplit, owns_new)
    rec["parity"] = parity_leg(ctx, spec, st, step)
    del st, dec, scratch, graph, wgraph
    torch.cuda.empty_cache()
    return rec if rank == 0 else None


def kvsplit_breakdown(ctx, spec, st, dec, layers, K, owns_new):
    """Where a KV-split step's time goes: the pieces launched one by one, eagerly, with a CUDA event
    between them; averages over K steps, max over ranks. (The cache write is its own launch here so
    that it can be told from the walk; in the measured step the walk does it.)"""
    torch = ctx.torch
    from hk_dsl_b200.ops import paged

    names = ("write_us", "walk_us", "local_merge_us", "all_gather_us", "merge_us")
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(K)]
    ctx.barrier()
    for i in range(K):
        l = i % layers
        ev[i][0].record()
        if owns_new:
            paged.reshape_and_cache(st.key, st.value, st.k_caches[l], st.v_caches[l], st.slot_mapping,
                                    spec.kv_cache_dtype, st.k_scale, st.v_scale)
        ev[i][1].record()
        dec.walk(st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype,
                 st.k_scale, st.v_scale)
        ev[i][2].record()
        dec.local_merge()
        ev[i][3].record()
        dec.gather()
        ev[i][4].record()
        dec.merge(st.out)
        ev[i][5].record()
    ctx.barrier()
    out = {}
    for j, nm in enumerate(names):
        out[nm] = ctx.max_over_ranks(statistics.fmean(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(K)) * 1e3)
    out["how"] = "eager launches, one CUDA event between pieces, mean of the steps, max over ranks"
    return out


def peer_breakdown(ctx, spec, st, dec, layers, K, owns_new):
    """The launches of a KV-split step over peer memory, eagerly, a CUDA event between them: the walk (it
    writes the new rows), then the exchange -- one kernel (fold of the local splits, stores into every
    rank, the wait for every rank's rows, the fold), or as two (push, merge) with HKB_KVSPLIT_EXCHANGE=peer2.
    Means over K steps, max over ranks."""
    torch = ctx.torch
    from hk_dsl_b200.ops import paged

    one = dec.exchange == "peer"
    names = ("walk_us", "exchange_us") if one else ("walk_us", "push_us", "wait_and_merge_us")
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K)]
    new = dict(key=st.key, value=st.value, slot_mapping=st.slot_mapping) if owns_new else dict(key=None, value=None, slot_mapping=None)
    ctx.barrier()
    for i in range(K):
        l = i % layers
        ev[i][0].record()
        paged.decode_step_record(None, None, st.query, new["key"], new["value"], st.k_caches[l], st.v_caches[l],
                                 new["slot_mapping"], st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype,
                                 st.k_scale, st.v_scale, num_splits=dec.local_splits, scratch=dec.scratch)
        ev[i][1].record()
        if one:
            dec.peer.exchange(dec.scratch, dec.local_splits, st.out)
            ev[i][2].record()
        else:
            dec.peer.push(dec.scratch, dec.local_splits)
            ev[i][2].record()
            dec.peer.merge(st.out)
            ev[i][3].record()
    ctx.barrier()
    out = {nm: ctx.max_over_ranks(statistics.fmean(ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(K)) * 1e3)
           for j, nm in enumerate(names)}
    out["how"] = "eager launches, one CUDA event between pieces, mean of the steps, max over ranks"
    return out


def e2e_leg(ctx, spec, st, dec, layers, splits, scratch, kv_total, K, Wm, kvsplit, owns_new):
    """The public API with host inputs; H2D of the step's inputs and D2H of its output inside.
    The step's host inputs live in ONE pinned staging buffer (as an engine's input batch does),
    so a step is one host->device copy; the device tensors the API takes are views of its twin."""
    torch = ctx.torch
    from hk_dsl_b200.ops import paged

    dev, world = ctx.dev, ctx.world
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

    def api_step(l):
        if kvsplit:
            new = dict(key=devb["key"], value=devb["value"], slot_mapping=devb["slot_mapping"]) if owns_new else {}
            dec.decode(st.out, devb["query"], st.k_caches[l], st.v_caches[l], devb["block_table"],
                       devb["seq_lens"], st.scale, spec.kv_cache_dtype, st.k_scale, st.v_scale, **new)
        else:
            paged.decode_step(st.out, devb["query"], devb["key"], devb["value"], st.k_caches[l], st.v_caches[l],
                              devb["slot_mapping"], devb["block_table"], devb["seq_lens"], st.scale,
                              spec.kv_cache_dtype, st.k_scale, st.v_scale, num_splits=splits, scratch=scratch)

    def e2e_step(i):
        stage_d.copy_(stage_h, non_blocking=True)
        api_step(i % layers)
        out_host.copy_(st.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()      # the caller reads the result before the next step

    def timed(fn):
        for i in range(Wm):
            fn(i)

        def run():
            for i in range(K):
                fn(i)
        return ctx.timed_ms(run) / K

    eager_ms = timed(e2e_step)
    e2e_ms, how = eager_ms, "eager: one host->device copy, the API call(s), one device->host copy, a stream sync a step"
    if not (kvsplit and world > 1) or (dec is not None and dec.peer is not None):
        # The same step as an engine runs it: captured once (a graph a rotated cache) and replayed. A
        # replay performs the host->device copy of the step's inputs from pinned memory, the launches
        # of decode_step and the device->host copy of the result; then the caller syncs and reads.
        try:
            graphs = []
            for l in range(layers):
                gl = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gl):
                    stage_d.copy_(stage_h, non_blocking=True)
                    api_step(l)
                    out_host.copy_(st.out, non_blocking=True)
                graphs.append(gl)

            def replay_step(i):
                graphs[i % layers].replay()
                torch.cuda.current_stream().synchronize()

            e2e_ms = statistics.median(timed(replay_step) for _ in range(3))
            how = ("the step (host->device copy of its inputs from pinned memory, decode_step, device->host copy of "
                   "its output) captured as a CUDA graph and replayed, then a stream sync: every replay performs both "
                   "copies; median of 3 runs of K steps")
        except Exception as ex:  # noqa: BLE001
            how += f" (graph capture of the step failed: {type(ex).__name__})"
            torch.cuda.synchronize()
    return {"value": kv_total / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
            "api": "hk_dsl_b200.ops.paged.decode_step" if not kvsplit else "hk_dsl_b200.ops.paged_dist.SplitKVDecoder.decode",
            "how": how, "eager_value": kv_total / (eager_ms * 1e-3) / 1e9, "eager_ms_per_step": eager_ms}


def parity_leg(ctx, spec, st, step):
    """One step on cache 0, then its output checked on the host against the oracle (the checker
    leg: nothing of the oracle is timed or shipped). Every rank checks its own share; the worst
    figures over ranks are reported."""
    torch, dist = ctx.torch, ctx.dist
    from oracle import paged_oracle as orc

    st.out.zero_()
    step(0)
    torch.cuda.synchronize()
    got = st.out.float().cpu()
    n = len(st.lens)
    kc, vc = st.k_caches[0].cpu(), st.v_caches[0].cpu()
    table, lens, q = st.block_table.cpu(), st.seq_lens.cpu(), st.query.cpu()
    ks = st.k_scale.cpu() if st.k_scale is not None else None
    vs = st.v_scale.cpu() if st.v_scale is not None else None
    rec = {"bound": "max-abs 2e-2, mean-abs 2e-3, worst row 4 bf16 ulps", "sequences": n}
    t0 = time.perf_counter()
    if st.shard.kind == "kvsplit":
        # this rank's float64 partial over its tokens of every sequence, gathered, folded in float64
        hkv, g, d = st.kv_heads, st.q_heads // st.kv_heads, spec.head_dim
        po = torch.zeros(n, st.q_heads, d)
        pl = torch.full((n, st.q_heads), float("-inf"))
        bs = spec.block_size
        for i, s in enumerate(st.lens):
            if s <= 0:
                continue
            pages = table[i, : -(-s // bs)].long()
            k_seq, v_seq = kc[pages], vc[pages]                    # (pages, block, kv heads, d)
            for kh in range(hkv):
                kk = orc._as_float_cache(k_seq[:, :, kh], ks).reshape(-1, d)[:s]
                vv = orc._as_float_cache(v_seq[:, :, kh], vs).reshape(-1, d)[:s]
                hs = slice(kh * g, (kh + 1) * g)
                po[i, hs], pl[i, hs] = orc.partial_ref(q[i, hs], kk, vv, st.scale)
        both = torch.cat([po.reshape(-1), pl.reshape(-1)]).to(ctx.dev)
        every = [torch.zeros_like(both) for _ in range(ctx.world)]
        dist.all_gather(every, both)
        cut = n * st.q_heads * d
        want, _ = orc.merge_lse_ref(torch.stack([e[:cut].cpu().view(n, st.q_heads, d) for e in every]),
                                    torch.stack([e[cut:].cpu().view(n, st.q_heads) for e in every]))
        rec["against"] = "float64 fold of every rank's float64 partial, whole batch"
        errs = [(got - want).abs()]
        worst_ulps = orc.ulps(got, want)
    else:
        want32 = orc.paged_decode_ref_fp32(q, kc, vc, table, lens, st.scale, ks, vs)
        few = sorted(range(n), key=lambda i: (st.lens[i], i))
        few = sorted({few[0], few[len(few) // 2], few[-1]})          # shortest, median, longest
        bs = spec.block_size
        want64 = torch.zeros(len(few), st.q_heads, spec.head_dim)
        for j, i in enumerate(few):
            s = st.lens[i]
            pages = table[i, : -(-s // bs)].long()
            want64[j] = orc.paged_decode_ref(q[i:i + 1], kc[pages], vc[pages], torch.arange(len(pages), dtype=torch.int32)[None],
                                             torch.tensor([s], dtype=torch.int32), st.scale, ks, vs)[0]
        rec["against"] = (f"the oracle's fp32 evaluation of all {n} local sequences and its float64 evaluation of "
                          f"{len(few)} (shortest, median, longest)")
        errs = [(got - want32).abs(), (got[few] - want64).abs()]
        worst_ulps = max(orc.ulps(got, want32), orc.ulps(got[few], want64))
    mx = max(e.max().item() for e in errs) if n else 0.0
    mean = max(e.mean().item() for e in errs) if n else 0.0
    finite = bool(torch.isfinite(got).all().item())
    if ctx.world > 1:
        t = torch.tensor([mx, mean, worst_ulps, 0.0 if finite else 1.0], device=ctx.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        mx, mean, worst_ulps, finite = float(t[0]), float(t[1]), float(t[2]), float(t[3]) == 0.0
    rec.update(max_abs=mx, mean_abs=mean, worst_row_bf16_ulps=worst_ulps, ranks_checked=ctx.world,
               oracle_seconds=round(time.perf_counter() - t0, 2),
               ok=bool(finite and mx <= 2e-2 and mean <= 2e-3 and worst_ulps < orc.ULPS))
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="c2")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--splits", type=int, default=0, help="0 = the planner's choice")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--only", action="store_true", help="the named config alone: no read probe, no other configs")
    ap.add_argument("--batch", type=int, default=0,
                    help="keep only the first N sequences of the config (small cases for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)

    ctx = Ctx(args)
    torch = ctx.torch
    from hk_dsl_b200 import workloads as W

    props = torch.cuda.get_device_properties(ctx.dev)
    gpu_id = f"GPU-{props.uuid}" if getattr(props, "uuid", None) else str(ctx.local)
    sampler = ClockSampler(gpu_id) if ctx.rank == 0 else None
    alone = args.only or bool(args.batch)
    probe = None
    if not alone:
        probe = read_probe(ctx)          # every rank runs it (the GPUs stay in step); rank 0's figure is reported
    head = run_config(ctx, args.config, headline=True, probe_gbs=probe["gbs"] if probe else None)
    clocks = sampler.stop() if sampler is not None else None

    # ---- CPU baseline on a bounded sample (rank 0, N=1)
    cpu = None
    if ctx.rank == 0 and ctx.world == 1 and not args.no_cpu:
        spec = W.CONFIGS[args.config]
        lens = W.seq_lens_of(spec)
        gbs, what, cores = cpu_port_rate(spec, lens[:args.batch] if args.batch else lens, seconds=15.0)
        cpu = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": what}

    others = {}
    if not alone and args.config == "c2":
        for name in ("c3", "c4", "c5"):
            rec = run_config(ctx, name, headline=False, probe_gbs=probe["gbs"] if probe else None)
            if rec is not None:
                others[name] = rec

    if ctx.rank == 0:
        line = {
            "metric": METRIC, "value": head["value"], "unit": "GB/s", "n_gpus": ctx.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic", "config": head["config"],
            "rounds": head["rounds"], "ms_per_step_min": head["ms_per_step_min"], "ms_per_step_max": head["ms_per_step_max"],
            "roofline": head["roofline"], "cpu_baseline": cpu, "e2e": head["e2e"],
            "gpu_launches": head["gpu_launches"], "clocks": clocks,
            "partition": head["partition"], "world": ctx.world,
            "seqs_per_s": head["seqs_per_s"], "tokens_per_s": head["tokens_per_s"],
            "frac_of_aggregate_hbm_measured": head["frac_of_aggregate_hbm_measured"],
            "frac_of_aggregate_hbm_nominal": head["frac_of_aggregate_hbm_nominal"],
            "splits": head["splits"], "cold_kv_detail": head["cold_kv_detail"], "cuda_graph": head["cuda_graph"],
            "parity": head["parity"], "read_probe": probe,
        }
        for k in ("cuda_graph_note", "breakdown_us", "exchange", "exchange_error_word"):
            if k in head:
                line[k] = head[k]
        if others:
            line["configs"] = others
        print(json.dumps(line), flush=True)
    if ctx.world > 1:
        ctx.dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
