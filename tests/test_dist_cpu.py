"""Multi-GPU host logic on CPU: who owns what, and the split-KV exchange as two gloo ranks.
The device merge is stood in for by the oracle's merge over the gathered record views, so
what is tested is the partition, the record layout and the all-gather plumbing."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hk_dsl_b200 import workloads as W
from hk_dsl_b200.ops import paged_dist
from oracle import paged_oracle as orc


def test_head_shards_tile_the_heads():
    for world in (1, 2, 4, 8):
        got = [paged_dist.shard_heads(8, world, r) for r in range(world)]
        assert got[0][0] == 0 and got[-1][1] == 8 and all(a[1] == b[0] for a, b in zip(got, got[1:]))
    with pytest.raises(ValueError, match="shard by sequence"):
        paged_dist.shard_heads(4, 8, 0)
    with pytest.raises(ValueError):
        paged_dist.shard_heads(8, 2, 2)


def test_sequences_are_dealt_evenly_by_tokens():
    spec = W.CONFIGS["c4"]
    lens = W.seq_lens_of(spec)
    for world in (2, 4, 8):
        bins = paged_dist.pack_sequences(lens, world)
        assert sorted(i for b in bins for i in b) == list(range(len(lens)))
        loads = [sum(lens[i] for i in b) for b in bins]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) / (sum(lens) / world) < 1.02
        assert bins == paged_dist.pack_sequences(lens, world)          # deterministic
    assert paged_dist.pack_sequences([5], 4) == [[0], [], [], []]


def test_kv_ranges_tile_the_sequence_in_whole_pages():
    for n in (1, 16, 17, 100, 131072, 131073):
        for world in (1, 2, 4, 8):
            r = [paged_dist.kv_range(n, world, k) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == n and all(a[1] == b[0] for a, b in zip(r, r[1:]))
            assert all(lo % 16 == 0 or lo == hi for lo, hi in r)      # an empty range may sit at the end


def test_shard_of_follows_the_config():
    lens5 = W.seq_lens_of(W.CONFIGS["c5"])
    assert W.shard_of(W.CONFIGS["c2"], [10] * 64, 4, 1).kind == "heads"
    assert W.shard_of(W.CONFIGS["c2"], [10] * 64, 4, 1).kv_heads == (2, 4)
    assert W.shard_of(W.CONFIGS["c4"], W.seq_lens_of(W.CONFIGS["c4"]), 8, 3).kind == "seqs"   # 4 kv heads, 8 GPUs
    s = W.shard_of(W.CONFIGS["c5"], lens5, 8, 7)
    assert s.kind == "kvsplit" and s.tokens == (114688, 131072)
    assert W.shard_of(W.CONFIGS["c5"], lens5, 1, 0).kind == "single"
    for name, spec in W.CONFIGS.items():
        lens = W.seq_lens_of(spec)
        assert len(lens) == spec.batch and lens == W.seq_lens_of(spec)
        assert all(1 <= x <= 131072 for x in lens)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, q, k, v, lens, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, hq, d = q.shape
        hkv = k.shape[2]
        g = hq // hkv
        dec = paged_dist.SplitKVDecoder(n, hq, hkv, d, "cpu", local_splits=2)
        assert dec.world == world and dec.rec % 4 == 0
        # this rank's partial over its token range of every sequence (the oracle stands in for the walk)
        for i in range(n):
            lo, hi = paged_dist.kv_range(int(lens[i]), world, rank)
            for kh in range(hkv):
                hs = slice(kh * g, (kh + 1) * g)
                dec.my_out[i, hs], dec.my_lse[i, hs] = orc.partial_ref(q[i, hs], k[i, lo:hi, kh], v[i, lo:hi, kh], d ** -0.5)
        dec.gather()
        rec = dec.all.view(world, dec.rec)
        po = rec[:, : n * hq * d].reshape(world, n, hq, d)
        pl = rec[:, n * hq * d: n * hq * (d + 1)].reshape(world, n, hq)
        out, _ = orc.merge_lse_ref(po, pl)
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def test_split_kv_exchange_two_gloo_ranks():
    g = torch.Generator().manual_seed(3)
    n, hq, hkv, d, t = 2, 8, 2, 64, 70
    q = torch.randn(n, hq, d, generator=g).to(torch.bfloat16)
    k = torch.randn(n, t, hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(n, t, hkv, d, generator=g).to(torch.bfloat16)
    lens = torch.tensor([70, 9])            # the second sequence lives on rank 0 alone
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_rank, args=(world, _free_port(), q, k, v, lens, ret), nprocs=world, join=True)
    want = torch.zeros(n, hq, d)
    for i in range(n):
        for kh in range(hkv):
            hs = slice(kh * 4, (kh + 1) * 4)
            want[i, hs] = orc.softmax_v64(q[i, hs], k[i, : lens[i], kh], v[i, : lens[i], kh], d ** -0.5)
    for r in range(world):
        assert (ret[r] - want).abs().max().item() < 1e-5       # every rank ends with the full answer
