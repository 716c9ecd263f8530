"""The paged decode across the GPUs of one box: who owns what, and the one exchange step.

hk-dsl itself has no multi-GPU plan for this path -- tensor parallelism is the engine's, and
a rank sees only its own heads (docs/performance/scorecard.md:14-20 of the reference) -- and
its only long-context device is the KV split inside one GPU (python/hk/ops/paged.py:171-194).
This module carries that split one level up:

* kv heads divide the world size  -> each rank owns a kv-head group and its query heads:
  independent work, no collective (`shard_heads`);
* otherwise                        -> whole sequences are dealt to ranks, longest first into the
  least-loaded rank, so every rank reads about the same KV bytes; no collective (`pack_sequences`);
* one long sequence                -> the KV axis is cut into contiguous token ranges, one a rank;
  every rank walks its range into a partial `(out fp32, lse)`, the partials are all-gathered
  with NCCL (they land in this rank's OWN memory: no peer loads, no multicast) and the same
  LSE-merge kernel that folds one GPU's splits folds the ranks' (`SplitKVDecoder`).

One process per GPU; `torch.distributed` (NCCL) is the plumbing.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ..runtime import lib as _lib
from . import paged


def shard_heads(num_kv_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """[lo, hi) of the kv heads rank `rank` owns; kv heads must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of world {world}")
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} kv heads do not divide over {world} ranks: shard by sequence")
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per


def pack_sequences(lens: Sequence[int], world: int) -> List[List[int]]:
    """Deal sequences to `world` ranks, longest first into the least-loaded rank (by tokens =
    KV bytes). Returns each rank's sequence indices, ascending. Deterministic."""
    bins: List[List[int]] = [[] for _ in range(world)]
    load = [0] * world
    for i in sorted(range(len(lens)), key=lambda i: (-lens[i], i)):
        r = min(range(world), key=lambda r: (load[r], r))
        bins[r].append(i)
        load[r] += lens[i]
    return [sorted(b) for b in bins]


def kv_range(seq_len: int, world: int, rank: int, block_size: int = paged.KV_BLOCK) -> Tuple[int, int]:
    """[lo, hi) of a sequence's tokens rank `rank` holds under a KV split: contiguous, whole
    pages a rank, the ranges of all ranks tiling [0, seq_len)."""
    per = -(-seq_len // world)
    per = -(-per // block_size) * block_size
    return min(seq_len, rank * per), min(seq_len, (rank + 1) * per)


def record_floats(num_seqs: int, num_q_heads: int, head_dim: int) -> int:
    """Floats of one rank's partial record -- out `(seqs, heads, d)` then lse `(seqs, heads)` --
    padded to 4 so every rank's record starts 16-byte aligned in the gathered buffer."""
    n = num_seqs * num_q_heads * (head_dim + 1)
    return (n + 3) // 4 * 4


class PeerExchange:
    """The exchange of a KV split over peer memory: every rank's gather buffer and state block live
    in symmetric memory that all ranks of the box have mapped, the fold of a rank's splits stores its
    record into every peer directly, and the final fold waits (boundedly) for every rank's flags. No
    collective in the step. `exchange` does it in one launch (hkb_kvsplit_exchange: a flag a row);
    `push` + `merge` are the two-launch form (hkb_kvsplit_push / hkb_kvsplit_merge: a flag a rank).

    With one rank (or no process group) the buffers are plain device tensors and the rank is its
    own only peer: the same kernels, usable on one GPU."""

    #: polls of a flag before the merge gives up (about a tenth of a microsecond each: ~1 s)
    SPIN_LIMIT = 10_000_000

    def __init__(self, num_seqs: int, num_q_heads: int, head_dim: int, device, group=None):
        import torch.distributed as dist

        lib = _lib.load()
        live = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if live else 1
        self.rank = dist.get_rank(group) if live else 0
        self.n, self.hq, self.d = num_seqs, num_q_heads, head_dim
        gbytes = lib.hkb_exchange_gather_bytes(self.world, num_seqs, num_q_heads, head_dim)
        if gbytes == 0:
            raise ValueError(f"hk.ops.paged_dist: no peer exchange for {self.world} ranks (1 to 8), {num_seqs} sequences")
        self.gather_bytes = (gbytes + 255) // 256 * 256
        self.state_bytes = lib.hkb_exchange_state_bytes_rows(num_seqs, num_q_heads)
        total = self.gather_bytes + (self.state_bytes + 255) // 256 * 256
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm

            self.buf = symm.empty(total, dtype=torch.uint8, device=device)
            self.buf.zero_()
            handle = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            self._handle = handle
            torch.cuda.synchronize(device)
            dist.barrier(group)              # nobody pushes into a state block that is still being zeroed
        else:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=device)
            ptrs = [self.buf.data_ptr()]
        x = _lib.ExchangeT()
        x.world, x.rank = self.world, self.rank
        for r in range(self.world):
            x.gather[r] = ptrs[r]
            x.state[r] = ptrs[r] + self.gather_bytes
        self.x = x
        # the ranks' flags, the counters and the error word, then the rows' flags
        self.state = self.buf[self.gather_bytes:self.gather_bytes + self.state_bytes].view(torch.int32)

    def push(self, scratch, num_splits: int) -> None:
        """Fold this rank's splits (`scratch` of the walk) and store the record into every rank."""
        po, pl = scratch
        rc = _lib.load().hkb_kvsplit_push(self.x, po.data_ptr(), pl.data_ptr(), num_splits, self.n, self.hq, self.d,
                                          paged._stream(po))
        _lib.check("hkb_kvsplit_push", rc)

    def merge(self, out: torch.Tensor, spin_limit: Optional[int] = None) -> torch.Tensor:
        """Wait for every rank's record of this step and fold them into `out` (seqs, heads, d)."""
        kind = {torch.bfloat16: 0, torch.float16: 2}.get(out.dtype)
        if kind is None or tuple(out.shape) != (self.n, self.hq, self.d) or out.stride(2) != 1:
            raise ValueError(f"hk.ops.paged_dist: the exchange writes ({self.n}, {self.hq}, {self.d}) bf16 or fp16, "
                             f"out is {tuple(out.shape)} {out.dtype}")
        rc = _lib.load().hkb_kvsplit_merge(self.x, out.data_ptr(), out.stride(0), out.stride(1), kind, self.n, self.hq,
                                           self.d, int(spin_limit or self.SPIN_LIMIT), paged._stream(out))
        _lib.check("hkb_kvsplit_merge", rc)
        return out

    def exchange(self, scratch, num_splits: int, out: torch.Tensor, spin_limit: Optional[int] = None) -> torch.Tensor:
        """`push` and `merge` in one launch: fold this rank's splits, store the rows into every rank,
        wait for every rank's rows and fold them into `out` (seqs, heads, d)."""
        po, pl = scratch
        kind = {torch.bfloat16: 0, torch.float16: 2}.get(out.dtype)
        if kind is None or tuple(out.shape) != (self.n, self.hq, self.d) or out.stride(2) != 1:
            raise ValueError(f"hk.ops.paged_dist: the exchange writes ({self.n}, {self.hq}, {self.d}) bf16 or fp16, "
                             f"out is {tuple(out.shape)} {out.dtype}")
        rc = _lib.load().hkb_kvsplit_exchange(self.x, po.data_ptr(), pl.data_ptr(), num_splits, out.data_ptr(),
                                              out.stride(0), out.stride(1), kind, self.n, self.hq, self.d,
                                              int(spin_limit or self.SPIN_LIMIT), paged._stream(out))
        _lib.check("hkb_kvsplit_exchange", rc)
        return out

    def error(self) -> int:
        """0, or 1 + the rank whose record a merge gave up waiting for (reads the device: a sync)."""
        return int(self.state[19].item())

    def reset(self) -> None:
        """Zero the state block (flags, step counter, error word). After a miss every rank calls this
        (and they meet at a barrier) before the next step."""
        self.state.zero_()


class SplitKVDecoder:
    """Decode of sequences whose KV is cut along the token axis across the ranks of `group`.

    Every rank calls `decode` with its own cache shard, block table and LOCAL lengths (the
    tokens of each sequence it holds; 0 is fine) and the same queries. Buffers are allocated
    once here, so a step allocates nothing: walk (writing the step's new rows where this rank
    holds them) -> merge of the local splits into this rank's record -> `all_gather_into_tensor`
    on the current stream -> cross-rank merge. Every rank ends with the full answer."""

    def __init__(self, num_seqs: int, num_q_heads: int, num_kv_heads: int, head_dim: int, device,
                 local_splits: int, group=None, exchange: str = "nccl"):
        """`exchange`: "nccl" -- `all_gather_into_tensor` of the ranks' records between two launches;
        "peer" -- the records go over peer memory inside ONE launch after the walk (`PeerExchange.exchange`);
        "peer2" -- the same in two launches (`push`, `merge`), the comparison arm."""
        import torch.distributed as dist

        if exchange not in ("nccl", "peer", "peer2"):
            raise ValueError(f"hk.ops.paged_dist: exchange {exchange!r} is not 'nccl', 'peer' or 'peer2'")
        self.exchange = exchange
        self.peer = PeerExchange(num_seqs, num_q_heads, head_dim, device, group) if exchange != "nccl" else None

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.n, self.hq, self.hkv, self.d = num_seqs, num_q_heads, num_kv_heads, head_dim
        self.local_splits = max(2, int(local_splits))       # the walk must write (out, lse) partials
        self.rec = record_floats(num_seqs, num_q_heads, head_dim)
        self.scratch = paged.split_scratch(num_seqs, num_q_heads, head_dim, self.local_splits, device)
        self.mine = torch.zeros(self.rec, device=device, dtype=torch.float32)
        self.all = torch.zeros(self.world * self.rec, device=device, dtype=torch.float32)
        n_out = num_seqs * num_q_heads * head_dim
        self.my_out = self.mine[:n_out].view(num_seqs, num_q_heads, head_dim)
        self.my_lse = self.mine[n_out:n_out + num_seqs * num_q_heads].view(num_seqs, num_q_heads)
        self._no_out = None

    def local_partial(self, query, key_cache, value_cache, block_tables, local_lens, scale,
                      kv_cache_dtype="auto", k_scale=None, v_scale=None, *, key=None, value=None,
                      slot_mapping=None) -> None:
        """This rank's record (normalised partial + lse) into `self.mine`: the walk over its tokens
        and the merge of its splits, two launches. The rank that holds the sequences' last position
        passes the step's new rows (`key`, `value`, `slot_mapping`): its walk writes them."""
        paged.decode_step_record(self.my_out, self.my_lse, query, key, value, key_cache, value_cache, slot_mapping,
                                 block_tables, local_lens, scale, kv_cache_dtype, k_scale, v_scale,
                                 num_splits=self.local_splits, scratch=self.scratch)

    # the two launches of `local_partial` on their own, for timing them apart and for tests
    def walk(self, query, key_cache, value_cache, block_tables, local_lens, scale,
             kv_cache_dtype="auto", k_scale=None, v_scale=None) -> None:
        """The walk alone: this rank's split partials into `self.scratch` (no cache write, no merge)."""
        if self._no_out is None or self._no_out.dtype != query.dtype:
            self._no_out = torch.zeros(self.n, self.hq, self.d, device=query.device, dtype=query.dtype)
        # with more than one split and merge=False the walk writes partials only; `out` is untouched
        paged.paged_attention_decode(self._no_out, query, key_cache, value_cache, block_tables, local_lens, scale,
                                     kv_cache_dtype, k_scale, v_scale, num_splits=self.local_splits,
                                     scratch=self.scratch, merge=False)

    def local_merge(self) -> None:
        """The merge of this rank's splits into its record (`self.mine`)."""
        po, pl = self.scratch
        n, hq, d, s = self.n, self.hq, self.d, self.local_splits
        rc = _lib.load().hkb_merge(self.my_out.data_ptr(), hq * d, d, 1, self.my_lse.data_ptr(),
                                   po.data_ptr(), hq * d, s * hq * d, pl.data_ptr(), hq, s * hq,
                                   s, n, hq, d, None, None, paged._stream(po))
        _lib.check("hkb_merge", rc)

    def gather(self) -> None:
        if self.world == 1:
            self.all.copy_(self.mine)
        else:
            self.dist.all_gather_into_tensor(self.all, self.mine, group=self.group)

    def merge(self, out: torch.Tensor) -> torch.Tensor:
        """Fold the gathered records of all ranks into `out` `(seqs, heads, d)` bf16."""
        n, hq, d = self.n, self.hq, self.d
        base = self.all.data_ptr()
        rc = _lib.load().hkb_merge(out.data_ptr(), out.stride(0), out.stride(1), 0, None,
                                   base, self.rec, hq * d, base + 4 * n * hq * d, self.rec, hq,
                                   self.world, n, hq, d, None, None, paged._stream(out))
        _lib.check("hkb_merge", rc)
        return out

    def decode(self, out, query, key_cache, value_cache, block_tables, local_lens, scale,
               kv_cache_dtype="auto", k_scale=None, v_scale=None, *, key=None, value=None,
               slot_mapping=None) -> torch.Tensor:
        """The whole step: two launches, one all-gather, one launch -- or, over peer memory, two
        launches and no collective (the walk; then one kernel that folds the local splits, stores this
        rank's rows into every rank, waits -- boundedly -- for every rank's rows and folds them)."""
        if self.peer is not None:
            paged.decode_step_record(None, None, query, key, value, key_cache, value_cache, slot_mapping, block_tables,
                                     local_lens, scale, kv_cache_dtype, k_scale, v_scale, num_splits=self.local_splits,
                                     scratch=self.scratch)
            if self.exchange == "peer":
                return self.peer.exchange(self.scratch, self.local_splits, out)
            self.peer.push(self.scratch, self.local_splits)
            return self.peer.merge(out)
        self.local_partial(query, key_cache, value_cache, block_tables, local_lens, scale,
                           kv_cache_dtype, k_scale, v_scale, key=key, value=value, slot_mapping=slot_mapping)
        self.gather()
        return self.merge(out)
