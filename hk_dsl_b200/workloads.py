"""Seeded synthetic decode workloads: the five configurations this path is measured on.

No dataset or model weights are involved in this metric (the reference's own kernel
benchmarks draw random tensors too, tools/hk-bench/paged_cdna.py:63-100); each config is
a shape, a sequence-length distribution and a seed:

  c1  4 sequences, 8 q / 2 kv heads, lens U[64, 512], pool of 256 blocks        (CPU-checkable)
  c2  Llama-3-8B-shaped: batch 64, 32 q / 8 kv heads, lens U[2048, 8192], bf16 KV
  c3  Qwen3-8B-shaped:   batch 128, 32 q / 8 kv heads, lens U[1024, 4096], fp8-e4m3 KV,
      k_scale = amax(K) / 448 and v_scale = amax(V) / 448 per tensor, amax taken over the seeded draws
  c4  mixed serving batch: 256 sequences, 32 q / 4 kv heads, lens log-normal(median 1024,
      sigma 1) clipped to [16, 32768], bf16 KV
  c5  long context: 2 sequences of 131072 tokens, 64 q / 8 kv heads, bf16 KV

All with head_dim 128, block_size 16, q / k / v ~ N(0, 1) in bf16, scale 1/sqrt(128), block
tables a random permutation of the pool, slot_mapping = each sequence's last position.
The cache is built by running the cache-write kernel over every token but the last of each
sequence; the measured step then writes the last token and decodes.

Across GPUs a config is partitioned the way a tensor-parallel engine hands it to a rank:
by kv-head group where kv_heads % world == 0 (c2, c3, c5's heads are NOT split: c5 cuts the
KV axis), else by sequence, longest first into the least-loaded rank (c4).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .ops import paged
from .ops.paged_dist import kv_range, pack_sequences, shard_heads


@dataclass(frozen=True)
class Spec:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int = 128
    block_size: int = 16
    kv_cache_dtype: str = "auto"
    dist: str = "uniform"       # uniform | lognormal | fixed
    lo: int = 0
    hi: int = 0
    pool_blocks: int = 0        # 0: sized to fit every sequence, plus 3 spare
    multi_gpu: str = "heads"    # heads | seqs | kvsplit
    what: str = ""

    @property
    def fp8(self) -> bool:
        return self.kv_cache_dtype != "auto"

    @property
    def kv_elt(self) -> int:
        return 1 if self.fp8 else 2

    def kv_bytes(self, lens: List[int]) -> int:
        """Algorithmic KV bytes of one decode call: sum(len) x kv_heads x head_dim x (K + V)."""
        return sum(lens) * self.kv_heads * self.head_dim * 2 * self.kv_elt


CONFIGS: Dict[str, Spec] = {s.name: s for s in (
    Spec("c1", 4, 8, 2, dist="uniform", lo=64, hi=512, pool_blocks=256, multi_gpu="heads",
         what="CPU-runnable parity case"),
    Spec("c2", 64, 32, 8, dist="uniform", lo=2048, hi=8192, multi_gpu="heads",
         what="Llama-3-8B-shaped decode, bf16 KV"),
    Spec("c3", 128, 32, 8, kv_cache_dtype="fp8", dist="uniform", lo=1024, hi=4096, multi_gpu="heads",
         what="Qwen3-8B-shaped decode, fp8-e4m3 KV"),
    Spec("c4", 256, 32, 4, dist="lognormal", lo=16, hi=32768, multi_gpu="seqs",
         what="mixed-length serving batch, 4 kv heads"),
    Spec("c5", 2, 64, 8, dist="fixed", lo=131072, hi=131072, multi_gpu="kvsplit",
         what="long-context split-KV decode"),
)}


def seq_lens_of(spec: Spec, seed: Optional[int] = None) -> List[int]:
    """The config's sequence lengths (seed defaults to the config's index)."""
    seed = int(spec.name[1:]) if seed is None else seed
    g = torch.Generator().manual_seed(seed)
    if spec.dist == "fixed":
        return [spec.lo] * spec.batch
    if spec.dist == "uniform":
        return torch.randint(spec.lo, spec.hi + 1, (spec.batch,), generator=g).tolist()
    z = torch.randn(spec.batch, generator=g)
    lens = torch.exp(math.log(1024.0) + 1.0 * z).round().clamp(spec.lo, spec.hi).long()
    return lens.tolist()


# ------------------------------------------------------------------------- sharding

@dataclass
class Shard:
    """What one rank of `world` owns."""
    kind: str                       # single | heads | seqs | kvsplit
    rank: int = 0
    world: int = 1
    kv_heads: Tuple[int, int] = (0, 0)       # [lo, hi) of the global kv heads
    seqs: List[int] = field(default_factory=list)   # global sequence indices owned
    tokens: Tuple[int, int] = (0, 0)         # kvsplit: [lo, hi) of every sequence's tokens


def shard_of(spec: Spec, lens: List[int], world: int, rank: int) -> Shard:
    every = list(range(len(lens)))
    if world == 1:
        return Shard("single", 0, 1, (0, spec.kv_heads), every, (0, 0))
    if spec.multi_gpu == "kvsplit":
        return Shard("kvsplit", rank, world, (0, spec.kv_heads), every,
                     kv_range(lens[0], world, rank, spec.block_size))
    if spec.multi_gpu == "heads" and spec.kv_heads % world == 0:
        return Shard("heads", rank, world, shard_heads(spec.kv_heads, world, rank), every, (0, 0))
    return Shard("seqs", rank, world, (0, spec.kv_heads), pack_sequences(lens, world)[rank], (0, 0))


# --------------------------------------------------------------------------- tensors

def _dist_ready() -> bool:
    import torch.distributed as dist
    return dist.is_available() and dist.is_initialized()


@dataclass
class Step:
    """One rank's tensors for one decode step over `layers` distinct caches."""
    spec: Spec
    shard: Shard
    lens: List[int]                 # local sequence lengths INCLUDING the token written this step
    q_heads: int
    kv_heads: int
    query: torch.Tensor             # (seqs, q_heads, d) bf16
    key: torch.Tensor               # (seqs, kv_heads, d) bf16: the step's new token
    value: torch.Tensor
    slot_mapping: torch.Tensor      # (seqs,) int64; -1 where this rank does not own the new token
    block_table: torch.Tensor       # (seqs, max_pages) int32
    seq_lens: torch.Tensor          # (seqs,) int32
    k_caches: List[torch.Tensor]    # `layers` caches, each a (blocks, block_size, kv_heads, d) VIEW
    v_caches: List[torch.Tensor]
    k_scale: Optional[torch.Tensor]
    v_scale: Optional[torch.Tensor]
    scale: float
    out: torch.Tensor

    @property
    def kv_bytes(self) -> int:
        return sum(self.lens) * self.kv_heads * self.spec.head_dim * 2 * self.spec.kv_elt


def build_step(spec: Spec, device, *, world: int = 1, rank: int = 0, layers: int = 1, seed: Optional[int] = None,
               layout: str = "hnd", lens: Optional[List[int]] = None, fill_chunk: int = 32768) -> Step:
    """Allocate and fill one rank's share of `spec` on `device` (a CUDA device: the cache is
    filled by the cache-write kernel). `layout`: "hnd" = hk's head-major storage
    (blocks, kv_heads, block, d) viewed as (blocks, block, kv_heads, d); "nhd" = vLLM's."""
    seed = int(spec.name[1:]) if seed is None else seed
    all_lens = seq_lens_of(spec, seed) if lens is None else list(lens)
    sh = shard_of(spec, all_lens, world, rank)
    d, bs = spec.head_dim, spec.block_size
    hkv = sh.kv_heads[1] - sh.kv_heads[0]
    group = spec.q_heads // spec.kv_heads
    hq = hkv * group
    dev = torch.device(device)
    fill_seed = 1000 * seed + 17 * rank + 1          # this rank's K/V draws
    # the query: every rank of a KV split attends with the SAME query
    gq = torch.Generator(device=dev).manual_seed(1000 * seed + 5 + (0 if sh.kind == "kvsplit" else 17 * rank))
    gc = torch.Generator().manual_seed(1000 * seed + 3)       # host-side choices: same on every rank

    if sh.kind == "kvsplit":
        local = [sh.tokens[1] - sh.tokens[0]] * len(all_lens)
        owns_new = sh.tokens[1] == all_lens[0]
    else:
        local = [all_lens[i] for i in sh.seqs]
        owns_new = True
    n = len(local)
    pages = [max(1, -(-s // bs)) for s in local]
    max_pages = max(pages) if pages else 1
    nb = spec.pool_blocks or (sum(pages) + 3)
    perm = torch.randperm(nb, generator=gc)
    table = torch.zeros(n, max_pages, dtype=torch.int32)
    at = 0
    for i, p in enumerate(pages):
        table[i, :p] = perm[at:at + p].to(torch.int32)
        at += p
    last_slot = torch.tensor([int(table[i, (s - 1) // bs]) * bs + (s - 1) % bs if s > 0 else -1
                              for i, s in enumerate(local)], dtype=torch.int64)
    if not owns_new:
        last_slot.fill_(-1)

    cache_dtype = torch.float8_e4m3fn if spec.fp8 else torch.bfloat16

    def new_cache():
        if layout == "hnd":
            store = torch.zeros(nb, hkv, bs, d, device=dev, dtype=torch.bfloat16).to(cache_dtype) \
                if spec.fp8 else torch.zeros(nb, hkv, bs, d, device=dev, dtype=cache_dtype)
            return store.transpose(1, 2)
        if spec.fp8:
            return torch.zeros(nb, bs, hkv, d, device=dev, dtype=torch.bfloat16).to(cache_dtype)
        return torch.zeros(nb, bs, hkv, d, device=dev, dtype=cache_dtype)

    # every token's slot but the last of each sequence (that one is the step's write)
    slots = []
    for i, s in enumerate(local):
        fill = s - 1 if owns_new else s
        if fill <= 0:
            continue
        pos = torch.arange(fill)
        slots.append(table[i, pos // bs].long() * bs + pos % bs)
    fill_slots = torch.cat(slots).to(dev) if slots else torch.zeros(0, dtype=torch.int64, device=dev)

    def draws(gen):
        """The K/V rows of the workload in the order they are drawn: (layer, slots, K rows, V rows)
        for every chunk of every cache, then (None, None, key, value) -- the step's new token."""
        for layer in range(layers):
            for a in range(0, fill_slots.numel(), fill_chunk):
                sl = fill_slots[a:a + fill_chunk]
                kk = torch.randn(sl.numel(), hkv, d, device=dev, dtype=torch.float32, generator=gen).to(torch.bfloat16)
                vv = torch.randn(sl.numel(), hkv, d, device=dev, dtype=torch.float32, generator=gen).to(torch.bfloat16)
                yield layer, sl, kk, vv
        yield (None, None,
               torch.randn(n, hkv, d, device=dev, dtype=torch.float32, generator=gen).to(torch.bfloat16),
               torch.randn(n, hkv, d, device=dev, dtype=torch.float32, generator=gen).to(torch.bfloat16))

    k_scale = v_scale = None
    if spec.fp8:
        # per-tensor scales = amax / 448 of the values that are quantised: a first pass over the
        # same seeded draws finds the amax (over every rank's share when the process group is up, so
        # that all ranks hold one scale, as a checkpoint's per-tensor scale is one number)
        amax = torch.zeros(2, device=dev, dtype=torch.float32)
        for _, _, kk, vv in draws(torch.Generator(device=dev).manual_seed(fill_seed)):
            amax[0] = torch.maximum(amax[0], kk.float().abs().max()) if kk.numel() else amax[0]
            amax[1] = torch.maximum(amax[1], vv.float().abs().max()) if vv.numel() else amax[1]
        if world > 1 and _dist_ready():
            import torch.distributed as dist
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        amax = amax.clamp_min(1e-12) / 448.0
        k_scale, v_scale = amax[0:1].clone(), amax[1:2].clone()

    k_caches = [new_cache() for _ in range(layers)]
    v_caches = [new_cache() for _ in range(layers)]
    key = value = None
    for layer, sl, kk, vv in draws(torch.Generator(device=dev).manual_seed(fill_seed)):
        if layer is None:
            key, value = kk, vv
        else:
            paged.reshape_and_cache(kk, vv, k_caches[layer], v_caches[layer], sl, spec.kv_cache_dtype, k_scale, v_scale)

    query = torch.randn(n, hq, d, device=dev, dtype=torch.float32, generator=gq).to(torch.bfloat16)
    return Step(spec=spec, shard=sh, lens=local, q_heads=hq, kv_heads=hkv,
                query=query, key=key, value=value,
                slot_mapping=last_slot.to(dev), block_table=table.to(dev),
                seq_lens=torch.tensor(local, dtype=torch.int32, device=dev),
                k_caches=k_caches, v_caches=v_caches, k_scale=k_scale, v_scale=v_scale,
                scale=d ** -0.5, out=torch.empty(n, hq, d, device=dev, dtype=torch.bfloat16))
