"""Paged KV cache write and paged GQA decode attention: the host side.

Mirrors the decode half of hk-dsl's `hk.ops.paged` (python/hk/ops/paged.py): the launch
contract (`check_decode`, :746-802), the split planner (`plan_splits`, :877-914), the
split scratch (`fused_scratch`, :733-743), the two-launch driver (`decode`, :811-828) and
the merge (`merge_splits`, :283-317) -- with the kernels behind them hand-written CUDA for
sm_100a reached through the C ABI (include/hkb.h) instead of generated HIP.

Two call forms:

* the engine-flat form the vLLM-style routes use,
  `reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype,
  k_scale, v_scale)` and `paged_attention_decode(out, query, key_cache, value_cache,
  block_tables, seq_lens, scale, kv_cache_dtype, k_scale, v_scale, ...)`, whose caches are
  `(num_blocks, block_size, num_kv_heads, head_dim)` views with any strides (hk's
  head-major storage is passed as `.transpose(1, 2)`, as the reference's backend passes it
  to vLLM's cache write, python/hk/integration/vllm_backend.py:594-599);
* hk's own form, `decode(q, k_cache, v_cache, block_table, seq_lens, out, scratch, splits)`
  on `(requests, kv_heads, group, head_dim)` q/out and `(blocks, kv_heads, KV_BLOCK, head_dim)`
  caches.

Everything launches on torch's current stream, reads nothing back, allocates nothing after
the scratch exists, and so can be captured into a CUDA graph. There is no fallback: a call
the kernels do not take raises.
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..runtime import lib as _lib

#: The cache's page size the backend declares; the kernels read any multiple of 16.
KV_BLOCK = 16
#: Most query rows (the GQA group) a kv head may have.
Q_TILE = 16
HEAD_DIMS = (64, 128, 256)       # head sizes the kernels take, for 16-bit and fp8 caches alike
DECODE_HEAD_DIMS = HEAD_DIMS
MAX_SPLITS = _lib.MAX_SPLITS

_FP8_NAMES = ("fp8", "fp8_e4m3")
ACT_DTYPES = (torch.bfloat16, torch.float16)   # activations: query, new K/V rows, output
_FP8_DTYPES = tuple(d for d in (getattr(torch, "float8_e4m3fn", None), torch.uint8) if d is not None)


def kv_dtype_code(kv_cache_dtype: str, cache: torch.Tensor, q_dtype=torch.bfloat16) -> int:
    """hkb's KV element code for vLLM's `kv_cache_dtype` string and the cache tensor given."""
    name = (kv_cache_dtype or "auto").lower()
    if name.startswith("auto") or name in ("bfloat16", "bf16", "float16", "half", "fp16"):
        # "auto" keeps the cache in the model's dtype: bf16, or fp16 for a model served in float16
        # (then the query, the new rows and the output are fp16 too)
        want = torch.float16 if name in ("float16", "half", "fp16") else \
            torch.bfloat16 if name in ("bfloat16", "bf16") else q_dtype
        if cache.dtype != want or want not in ACT_DTYPES:
            raise TypeError(f"hk.ops.paged: kv_cache_dtype {kv_cache_dtype!r} keeps the cache in {want}, "
                            f"the cache is {cache.dtype} (bfloat16 and float16 are implemented)")
        return _lib.KV_F16 if want == torch.float16 else _lib.KV_BF16
    if name in _FP8_NAMES:
        if q_dtype != torch.bfloat16:
            raise TypeError(f"hk.ops.paged: an fp8 cache goes with bfloat16 activations, the query is {q_dtype}")
        if cache.dtype not in _FP8_DTYPES:
            raise TypeError(f"hk.ops.paged: kv_cache_dtype {kv_cache_dtype!r} needs a float8_e4m3fn (or uint8) "
                            f"cache, the cache is {cache.dtype}")
        return _lib.KV_FP8_E4M3
    raise NotImplementedError(f"hk.ops.paged: kv_cache_dtype {kv_cache_dtype!r}: only auto (bf16) and "
                              f"fp8 / fp8_e4m3 caches are implemented")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _cache_t(c: torch.Tensor) -> _lib.CacheT:
    """A `(blocks, block_size, kv_heads, head_dim)` view as hkb_cache_t."""
    return _lib.CacheT(c.data_ptr(), c.stride(0), c.stride(1), c.stride(2), c.shape[0])


def _need_cuda(*ts: torch.Tensor) -> None:
    """Every tensor on ONE CUDA device, and that device current (the C ABI launches on the current
    device; one process per GPU sets it once)."""
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("hk.ops.paged: tensors must be on a CUDA device; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"hk.ops.paged: tensors on different devices ({dev} and {t.device})")
    if dev is not None and dev.index != torch.cuda.current_device():
        raise RuntimeError(f"hk.ops.paged: the tensors live on {dev} but the current CUDA device is "
                           f"cuda:{torch.cuda.current_device()}; call torch.cuda.set_device({dev.index}) "
                           f"(or use `with torch.cuda.device(...)`) before launching")


def _scale_ptr(s: Optional[torch.Tensor], fp8: bool, name: str) -> Optional[int]:
    if s is None:
        if fp8:
            raise ValueError(f"hk.ops.paged: an fp8 cache needs {name} (a float32 tensor of one element)")
        return None
    if s.dtype != torch.float32 or s.numel() != 1:
        raise TypeError(f"hk.ops.paged: {name} is {tuple(s.shape)} {s.dtype}; per-tensor float32 scale needed")
    return s.data_ptr()


# --------------------------------------------------------------------------------------
# engine-flat form
# --------------------------------------------------------------------------------------

def reshape_and_cache(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                      value_cache: torch.Tensor, slot_mapping: torch.Tensor, kv_cache_dtype: str = "auto",
                      k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    """Scatter new K/V rows into the paged caches by slot; slot < 0 is skipped.

    vLLM's `reshape_and_cache_flash` signature and argument order
    (tests/hk/engines/test_vllm_contract.py:271-277). `key`/`value` are
    `(tokens, kv_heads, head_dim)` bf16; the caches `(blocks, block_size, kv_heads, head_dim)`
    views of any strides, bf16 or fp8-e4m3; `slot_mapping` int64 or int32."""
    _need_cuda(key, value, key_cache, value_cache, slot_mapping)
    if key.dim() != 3 or value.shape != key.shape or key.dtype not in ACT_DTYPES or value.dtype != key.dtype:
        raise ValueError(f"hk.ops.paged: key {tuple(key.shape)} {key.dtype} / value {tuple(value.shape)} "
                         f"{value.dtype}; the cache write reads (tokens, kv_heads, head_dim) bfloat16 or float16")
    t, hkv, d = key.shape
    for name, c in (("key_cache", key_cache), ("value_cache", value_cache)):
        if c.dim() != 4 or c.shape[2] != hkv or c.shape[3] != d or c.stride(3) != 1:
            raise ValueError(f"hk.ops.paged: {name} is {tuple(c.shape)} strides {c.stride()}; the cache write "
                             f"needs (blocks, block_size, {hkv}, {d}) with head_dim contiguous")
    if key.stride(2) != 1 or value.stride(2) != 1:
        raise ValueError("hk.ops.paged: key/value head_dim must be contiguous")
    if slot_mapping.dim() != 1 or slot_mapping.dtype not in (torch.int64, torch.int32) \
            or not slot_mapping.is_contiguous():
        raise TypeError(f"hk.ops.paged: slot_mapping is {tuple(slot_mapping.shape)} {slot_mapping.dtype}; "
                        f"contiguous int64 or int32 (tokens,) needed")
    n = min(t, slot_mapping.shape[0])
    code = kv_dtype_code(kv_cache_dtype, key_cache, key.dtype)
    if value_cache.dtype != key_cache.dtype or value_cache.shape[1] != key_cache.shape[1]:
        raise ValueError("hk.ops.paged: key_cache and value_cache differ in dtype or block_size")
    fp8 = code == _lib.KV_FP8_E4M3
    rc = _lib.load().hkb_reshape_and_cache(
        key.data_ptr(), value.data_ptr(), key.stride(0), key.stride(1), value.stride(0), value.stride(1),
        _cache_t(key_cache), _cache_t(value_cache), slot_mapping.data_ptr(),
        1 if slot_mapping.dtype == torch.int64 else 0, n, hkv, d, key_cache.shape[1], code,
        _scale_ptr(k_scale, fp8, "k_scale"), _scale_ptr(v_scale, fp8, "v_scale"), _stream(key))
    _lib.check("hkb_reshape_and_cache", rc)


def split_scratch(num_seqs: int, num_q_heads: int, head_dim: int, num_splits: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(part_out, part_lse) for a split decode: fp32 normalised partials
    `(num_seqs * num_splits, num_q_heads, head_dim)` and their natural-log lse
    `(num_seqs * num_splits, num_q_heads)`."""
    rows = num_seqs * num_splits
    return (torch.empty(rows, num_q_heads, head_dim, device=device, dtype=torch.float32),
            torch.empty(rows, num_q_heads, device=device, dtype=torch.float32))


def x_split_why_not(key_cache, value_cache, head_dim: int) -> str:
    """Why these caches are not vLLM's x-split pair as the decode reads it, or "": K
    (blocks, kv_heads, head_dim / 8, block_size, 8) and V (blocks, kv_heads, head_dim, block_size),
    16-bit, everything inside a block contiguous (python/hk/ops/paged_prefill.py:768-772)."""
    if key_cache.dim() != 5 or value_cache.dim() != 4:
        return f"caches {tuple(key_cache.shape)} / {tuple(value_cache.shape)}: not the 5-D K, 4-D V pair"
    nb, hkv, chunks, page, x = key_cache.shape
    if key_cache.dtype not in ACT_DTYPES or value_cache.dtype != key_cache.dtype:
        return f"x-split caches of {key_cache.dtype} / {value_cache.dtype} (16-bit only)"
    if x != 8 or chunks * x != head_dim or head_dim != 128:
        return f"x-split K {tuple(key_cache.shape)} at head size {head_dim} (x = 8, head size 128 only)"
    if tuple(value_cache.shape) != (nb, hkv, head_dim, page):
        return f"x-split V {tuple(value_cache.shape)} beside K {tuple(key_cache.shape)}"
    if page % 16:
        return f"block size {page} (a multiple of 16)"
    if key_cache.stride()[1:] != (head_dim * page, page * 8, 8, 1) or value_cache.stride()[1:] != (head_dim * page, page, 1):
        return "x-split caches not contiguous inside a block"
    if key_cache.stride(0) < hkv * head_dim * page or value_cache.stride(0) < hkv * head_dim * page:
        return "x-split blocks overlap"
    return ""


def _decode_call(out, query, key_cache, value_cache, block_tables, seq_lens, query_start_loc, x_split: bool = False):
    """Validate the tensors of a decode call; returns (seqs, q_heads, head_dim, block_size, kv_heads, q_start ptr)."""
    _need_cuda(out, query, key_cache, value_cache, block_tables, seq_lens)
    if query.dim() != 3 or query.dtype not in ACT_DTYPES or query.stride(2) != 1:
        raise ValueError(f"hk.ops.paged: query is {tuple(query.shape)} {query.dtype}; the decode reads "
                         f"(tokens, q_heads, head_dim) bfloat16 or float16 with head_dim contiguous")
    if out.shape != query.shape or out.dtype != query.dtype or out.stride(2) != 1:
        raise ValueError(f"hk.ops.paged: out is {tuple(out.shape)} {out.dtype}; it must match query "
                         f"{tuple(query.shape)} {query.dtype}")
    _, hq, d = query.shape
    if x_split:
        why = x_split_why_not(key_cache, value_cache, d)
        if why:
            raise ValueError(f"hk.ops.paged: {why}")
        bs, hkv = key_cache.shape[3], key_cache.shape[1]
    else:
        if key_cache.dim() != 4 or value_cache.shape != key_cache.shape or key_cache.stride(3) != 1 \
                or value_cache.stride(3) != 1 or key_cache.shape[3] != d or value_cache.dtype != key_cache.dtype:
            raise ValueError(f"hk.ops.paged: key_cache {tuple(key_cache.shape)} / value_cache "
                             f"{tuple(value_cache.shape)}; the decode reads two (blocks, block_size, kv_heads, {d}) "
                             f"views of one dtype")
        _, bs, hkv, _ = key_cache.shape
    if block_tables.dim() != 2 or block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
        raise TypeError(f"hk.ops.paged: block_tables is {tuple(block_tables.shape)} {block_tables.dtype}; "
                        f"(seqs, max_pages) int32 needed")
    if seq_lens.dim() != 1 or seq_lens.dtype != torch.int32 or not seq_lens.is_contiguous():
        raise TypeError(f"hk.ops.paged: seq_lens is {tuple(seq_lens.shape)} {seq_lens.dtype}; "
                        f"contiguous (seqs,) int32 needed")
    n = seq_lens.shape[0]
    if block_tables.shape[0] < n:
        raise ValueError(f"hk.ops.paged: block_tables has {block_tables.shape[0]} rows for {n} sequences")
    qsl = None
    if query_start_loc is not None:
        if query_start_loc.dtype != torch.int32 or query_start_loc.numel() < n + 1 \
                or not query_start_loc.is_contiguous():
            raise TypeError("hk.ops.paged: query_start_loc must be contiguous int32 of seqs + 1 entries")
        qsl = query_start_loc.data_ptr()
    elif query.shape[0] < n:
        raise ValueError(f"hk.ops.paged: {query.shape[0]} query rows for {n} sequences")
    return n, hq, d, bs, hkv, qsl


def _scratch_ptrs(scratch, n, hq, d, num_splits, device):
    if num_splits <= 1:
        return None, None, scratch
    if scratch is None:
        scratch = split_scratch(n, hq, d, num_splits, device)
    po, pl = scratch[0], scratch[1]
    if po.dtype != torch.float32 or pl.dtype != torch.float32 or po.numel() < n * num_splits * hq * d \
            or pl.numel() < n * num_splits * hq or not po.is_contiguous() or not pl.is_contiguous():
        raise ValueError(f"hk.ops.paged: scratch too small or not contiguous fp32 for {n} sequences x "
                         f"{num_splits} splits x {hq} heads x {d} (split_scratch)")
    return po, pl, scratch


def paged_attention_decode(out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                           value_cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                           scale: float, kv_cache_dtype: str = "auto",
                           k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None, *,
                           num_splits: Optional[int] = None,
                           scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                           query_start_loc: Optional[torch.Tensor] = None,
                           max_seq_len: Optional[int] = None, merge: bool = True) -> torch.Tensor:
    """Decode attention of one query token a sequence over a block-paged KV cache.

    `query`/`out`: `(tokens, q_heads, head_dim)` bf16 (head_dim contiguous); caches
    `(blocks, block_size, kv_heads, head_dim)` views, bf16 or fp8-e4m3 with per-tensor
    `k_scale`/`v_scale`; `block_tables` `(seqs, max_pages)` int32; `seq_lens` `(seqs,)` int32.
    `num_splits` None plans it from the batch and the table's width (host values only);
    with more than one split the walk writes partials into `scratch` (allocated here if
    not given -- pass it to stay allocation-free) and the merge kernel folds them
    (`merge=False` stops after the walk and leaves the partials in `scratch`)."""
    n, hq, d, bs, hkv, qsl = _decode_call(out, query, key_cache, value_cache, block_tables, seq_lens, query_start_loc)
    code = kv_dtype_code(kv_cache_dtype, key_cache, query.dtype)
    fp8 = code == _lib.KV_FP8_E4M3
    if num_splits is None:
        tiles = block_tables.shape[1] * (bs // 16) if max_seq_len is None else -(-max_seq_len // 16)
        num_splits = plan_splits(n, hkv, tiles, device=query.device)
    po, pl, scratch = _scratch_ptrs(scratch, n, hq, d, num_splits, query.device)
    lib = _lib.load()
    st = _stream(query)
    rc = lib.hkb_paged_decode(
        out.data_ptr(), out.stride(0), out.stride(1), query.data_ptr(), query.stride(0), query.stride(1),
        _cache_t(key_cache), _cache_t(value_cache), block_tables.data_ptr(), block_tables.stride(0),
        block_tables.shape[1], seq_lens.data_ptr(), qsl, n, hq, hkv, d, bs, float(scale), code,
        _scale_ptr(k_scale, fp8, "k_scale"), _scale_ptr(v_scale, fp8, "v_scale"), num_splits,
        po.data_ptr() if po is not None else None, pl.data_ptr() if pl is not None else None, st)
    _lib.check("hkb_paged_decode", rc)
    if num_splits > 1 and merge:
        rc = lib.hkb_merge(out.data_ptr(), out.stride(0), out.stride(1), 2 if out.dtype == torch.float16 else 0, None,
                           po.data_ptr(), hq * d, num_splits * hq * d, pl.data_ptr(), hq, num_splits * hq,
                           num_splits, n, hq, d, seq_lens.data_ptr(), qsl, st)
        _lib.check("hkb_merge", rc)
    return out


def paged_attention_decode_xsplit(out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                                  value_cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                                  scale: float, *, num_splits: Optional[int] = None,
                                  scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                                  query_start_loc: Optional[torch.Tensor] = None,
                                  max_seq_len: Optional[int] = None) -> torch.Tensor:
    """`paged_attention_decode` over vLLM's x-split caches, read in place: `key_cache`
    (blocks, kv_heads, head_dim / 8, block_size, 8), `value_cache` (blocks, kv_heads, head_dim,
    block_size), bf16 or fp16, head_dim 128 (`x_split_why_not`). What the reference reaches through
    `rocm_views` and `_rocm_decode` (python/hk/ops/paged_prefill.py:768-772,
    python/hk/integration/vllm_prefill.py:1332-1356). Always the balanced tile stream: at least
    two splits, at most 2048 sequences."""
    n, hq, d, bs, hkv, qsl = _decode_call(out, query, key_cache, value_cache, block_tables, seq_lens, query_start_loc,
                                          x_split=True)
    if num_splits is None:
        tiles = block_tables.shape[1] * (bs // 16) if max_seq_len is None else -(-max_seq_len // 16)
        num_splits = plan_splits(n, hkv, tiles, device=query.device)
    num_splits = max(2, int(num_splits))
    po, pl, scratch = _scratch_ptrs(scratch, n, hq, d, num_splits, query.device)
    lib = _lib.load()
    st = _stream(query)
    code = _lib.KV_F16 if query.dtype == torch.float16 else _lib.KV_BF16
    rc = lib.hkb_paged_decode_xsplit(
        out.data_ptr(), out.stride(0), out.stride(1), query.data_ptr(), query.stride(0), query.stride(1),
        key_cache.data_ptr(), key_cache.stride(0), value_cache.data_ptr(), value_cache.stride(0), key_cache.shape[0],
        block_tables.data_ptr(), block_tables.stride(0), block_tables.shape[1], seq_lens.data_ptr(), qsl,
        n, hq, hkv, d, bs, float(scale), code, num_splits, po.data_ptr(), pl.data_ptr(), st)
    _lib.check("hkb_paged_decode_xsplit", rc)
    rc = lib.hkb_merge(out.data_ptr(), out.stride(0), out.stride(1), 2 if out.dtype == torch.float16 else 0, None,
                       po.data_ptr(), hq * d, num_splits * hq * d, pl.data_ptr(), hq, num_splits * hq,
                       num_splits, n, hq, d, seq_lens.data_ptr(), qsl, st)
    _lib.check("hkb_merge", rc)
    return out


def x_split_caches(key_cache: torch.Tensor, value_cache: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """A (blocks, block_size, kv_heads, head_dim) cache pair copied into the x-split layout (for
    tests and tools; an engine that uses the layout allocates it so)."""
    nb, bs, hkv, d = key_cache.shape
    k5 = key_cache.permute(0, 2, 1, 3).reshape(nb, hkv, bs, d // 8, 8).permute(0, 1, 3, 2, 4).contiguous()
    v4 = value_cache.permute(0, 2, 3, 1).contiguous()
    return k5, v4


def step_arrivals(num_seqs: int, num_kv_heads: int, device) -> torch.Tensor:
    """The arrival counters `decode_step` needs: zeroed once here, left zero by every step.
    One array a stream -- two steps in flight at once must not share it."""
    return torch.zeros(_lib.load().hkb_arrivals_bytes(num_seqs, num_kv_heads) // 4, device=device, dtype=torch.int32)


def decode_step(out: torch.Tensor, query: torch.Tensor, key: Optional[torch.Tensor], value: Optional[torch.Tensor],
                key_cache: torch.Tensor, value_cache: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                block_tables: torch.Tensor, seq_lens: torch.Tensor, scale: float, kv_cache_dtype: str = "auto",
                k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None, *,
                num_splits: Optional[int] = None, scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                arrivals: Optional[torch.Tensor] = None, query_start_loc: Optional[torch.Tensor] = None,
                max_seq_len: Optional[int] = None) -> torch.Tensor:
    """One decode step of a layer: `reshape_and_cache(key, value, ...)` then
    `paged_attention_decode(out, query, ...)`, in two launches instead of three -- or in one.

    The backend's decode step is a cache write and two launches
    (python/hk/integration/vllm_backend.py:582-599, 700-729); here the ring of the walk that owns
    a sequence's last tile writes the new row first, then the merge kernel runs. `key`/`value`:
    `(seqs, kv_heads, head_dim)` bf16, one new token a sequence, `slot_mapping[i]` = the slot of
    position `seq_lens[i] - 1` of sequence i (negative: skipped); both None when the cache is
    already written. With `arrivals` (`step_arrivals`) the walk also folds the partials -- the ring
    that finishes a sequence's last piece does it -- and the step is one launch; measured, that
    pays only for small evenly cut batches, so it is opt-in. `scratch` is allocated here if not
    given. Shapes the stream kernel does not take (one split, more than 2048 sequences) run the
    separate launches."""
    n, hq, d, bs, hkv, qsl = _decode_call(out, query, key_cache, value_cache, block_tables, seq_lens, query_start_loc)
    new = _new_rows(query, key, value, slot_mapping, n, hkv, d, query_start_loc)
    code = kv_dtype_code(kv_cache_dtype, key_cache, query.dtype)
    fp8 = code == _lib.KV_FP8_E4M3
    if num_splits is None:
        tiles = block_tables.shape[1] * (bs // 16) if max_seq_len is None else -(-max_seq_len // 16)
        num_splits = plan_splits(n, hkv, tiles, device=query.device)
    po, pl, scratch = _scratch_ptrs(scratch, n, hq, d, num_splits, query.device)
    lib = _lib.load()
    if num_splits > 1 and arrivals is not None:
        if arrivals.dtype != torch.int32 or not arrivals.is_contiguous() \
                or arrivals.numel() * 4 < lib.hkb_arrivals_bytes(n, hkv):
            raise ValueError(f"hk.ops.paged: arrivals too small or not contiguous int32 for {n} sequences x {hkv} "
                             f"kv heads (step_arrivals)")
        _need_cuda(arrivals)
    rc = lib.hkb_decode_step(
        out.data_ptr(), out.stride(0), out.stride(1), query.data_ptr(), query.stride(0), query.stride(1),
        *new, _cache_t(key_cache), _cache_t(value_cache), block_tables.data_ptr(),
        block_tables.stride(0), block_tables.shape[1], seq_lens.data_ptr(), qsl, n, hq, hkv, d, bs, float(scale), code,
        _scale_ptr(k_scale, fp8, "k_scale"), _scale_ptr(v_scale, fp8, "v_scale"), num_splits,
        po.data_ptr() if po is not None else None, pl.data_ptr() if pl is not None else None,
        arrivals.data_ptr() if arrivals is not None and num_splits > 1 else None, _stream(query))
    _lib.check("hkb_decode_step", rc)
    return out


def _new_rows(query, key, value, slot_mapping, n, hkv, d, query_start_loc):
    """The step's new K/V rows as the C ABI takes them: (key ptr, value ptr, four strides, slot ptr, slot_is_i64)."""
    if (key is None) != (value is None):
        raise ValueError("hk.ops.paged: decode_step takes key and value together")
    if key is None:
        return (None, None, 0, 0, 0, 0, None, 0)
    _need_cuda(key, value, slot_mapping)
    if key.dim() != 3 or value.shape != key.shape or key.dtype != query.dtype or value.dtype != key.dtype \
            or key.shape[1] != hkv or key.shape[2] != d or key.stride(2) != 1 or value.stride(2) != 1:
        raise ValueError(f"hk.ops.paged: key {tuple(key.shape)} {key.dtype} / value {tuple(value.shape)} "
                         f"{value.dtype}; the step writes (seqs, {hkv}, {d}) rows of the query's dtype ({query.dtype})")
    if slot_mapping is None or slot_mapping.dim() != 1 or slot_mapping.dtype not in (torch.int64, torch.int32) \
            or not slot_mapping.is_contiguous():
        raise TypeError("hk.ops.paged: slot_mapping must be a contiguous int64 or int32 (rows,) tensor")
    rows = query.shape[0] if query_start_loc is not None else n
    if key.shape[0] < rows or slot_mapping.shape[0] < rows:
        raise ValueError(f"hk.ops.paged: {key.shape[0]} new rows / {slot_mapping.shape[0]} slots for {rows} query rows")
    return (key.data_ptr(), value.data_ptr(), key.stride(0), key.stride(1), value.stride(0), value.stride(1),
            slot_mapping.data_ptr(), 1 if slot_mapping.dtype == torch.int64 else 0)


def decode_step_record(rec_out: torch.Tensor, rec_lse: torch.Tensor, query: torch.Tensor,
                       key: Optional[torch.Tensor], value: Optional[torch.Tensor], key_cache: torch.Tensor,
                       value_cache: torch.Tensor, slot_mapping: Optional[torch.Tensor], block_tables: torch.Tensor,
                       local_lens: torch.Tensor, scale: float, kv_cache_dtype: str = "auto",
                       k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None, *,
                       num_splits: int, scratch: Tuple[torch.Tensor, torch.Tensor],
                       query_start_loc: Optional[torch.Tensor] = None) -> None:
    """One rank's decode step of a KV axis cut across GPUs: the walk over this rank's tokens
    (`local_lens`; it writes the new rows when `key` / `value` are given, i.e. on the rank that
    holds the sequences' last position) and a merge of its splits into the rank's record --
    `rec_out` `(seqs, q_heads, head_dim)` fp32 normalised and `rec_lse` `(seqs, q_heads)` fp32
    natural-log sum-exp (-inf where the rank holds nothing of a sequence). Two launches.
    `merge_partials` (or `SplitKVDecoder.merge`) folds the gathered records of all ranks.
    `rec_out` = `rec_lse` = None: the walk alone, one launch; the split partials stay in `scratch`
    for `PeerExchange.push` to fold."""
    n = local_lens.shape[0]
    _, hq, d = query.shape
    walk_only = rec_out is None and rec_lse is None      # the partials stay in `scratch` for the caller to fold
    if not walk_only and (rec_out is None or rec_lse is None or rec_out.dtype != torch.float32
                          or rec_lse.dtype != torch.float32 or not rec_out.is_contiguous()
                          or not rec_lse.is_contiguous() or rec_out.numel() < n * hq * d or rec_lse.numel() < n * hq):
        raise ValueError(f"hk.ops.paged: the record is contiguous fp32 ({n}, {hq}, {d}) and ({n}, {hq})")
    if num_splits < 2:
        raise ValueError("hk.ops.paged: a record is written by the merge of at least two splits")
    _need_cuda(rec_out, rec_lse)
    # the record stands where a decode's 16-bit out would; the query is passed in that position only to be checked
    n, hq, d, bs, hkv, qsl = _decode_call(query, query, key_cache, value_cache, block_tables, local_lens,
                                          query_start_loc)
    new = _new_rows(query, key, value, slot_mapping, n, hkv, d, query_start_loc)
    code = kv_dtype_code(kv_cache_dtype, key_cache, query.dtype)
    fp8 = code == _lib.KV_FP8_E4M3
    po, pl, _ = _scratch_ptrs(scratch, n, hq, d, num_splits, query.device)
    rc = _lib.load().hkb_decode_step_record(
        None if walk_only else rec_out.data_ptr(), None if walk_only else rec_lse.data_ptr(), query.data_ptr(), query.stride(0), query.stride(1), *new,
        _cache_t(key_cache), _cache_t(value_cache), block_tables.data_ptr(), block_tables.stride(0),
        block_tables.shape[1], local_lens.data_ptr(), qsl, n, hq, hkv, d, bs, float(scale), code,
        _scale_ptr(k_scale, fp8, "k_scale"), _scale_ptr(v_scale, fp8, "v_scale"), num_splits,
        po.data_ptr(), pl.data_ptr(), _stream(query))
    _lib.check("hkb_decode_step_record", rc)


# --------------------------------------------------------------------------------------
# prefill (the rows of a batch that are not single-token decodes)
# --------------------------------------------------------------------------------------

def prefill_tile_rows(num_q_heads: int, num_kv_heads: int) -> int:
    """Query tokens one work item of the prefill kernels covers: 256 rows / GP, GP the largest of
    8, 4, 2, 1 dividing the GQA group (hkb_prefill_tile_rows)."""
    g = num_q_heads // num_kv_heads
    gp = 8 if g % 8 == 0 else 4 if g % 4 == 0 else 2 if g % 2 == 0 else 1
    return 256 // gp


def work_list(reqs, tile_rows: int, device, seq_lens=None) -> torch.Tensor:
    """The prefill's grid, built on the host where the query lengths already are: `reqs` is
    [(request, q_len)]; one (request, first row) pair a `tile_rows`-row query tile, the tiles that
    see the most keys first (`seq_lens`, host ints, if given) so the long ones do not trail.
    The counterpart of hk-dsl's `work_list` (python/hk/ops/paged_prefill.py:879-968)."""
    items = []
    for r, n in reqs:
        for row0 in range(0, int(n), tile_rows):
            end = min(int(n), row0 + tile_rows)
            keys = (int(seq_lens[r]) - int(n) + end) if seq_lens is not None else end
            items.append((-keys, r, row0))
    items.sort()
    flat = [x for _, r, row0 in items for x in (r, row0)]
    return torch.tensor(flat, dtype=torch.int32).view(-1, 2).to(device, non_blocking=True)


def paged_prefill(out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                  block_tables: torch.Tensor, seq_lens: torch.Tensor, query_start_loc: torch.Tensor,
                  work: torch.Tensor, scale: float, kv_cache_dtype: str = "auto",
                  k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every request's new tokens over its paged cache (prefix + new tokens,
    already written). `query`/`out` `(tokens, q_heads, head_dim)` bf16; caches
    `(blocks, block_size, kv_heads, head_dim)` views, bf16 or fp8-e4m3 with per-tensor scales; `seq_lens` the tokens in the cache a
    request (int32), `query_start_loc` cu_seqlens_q (int32, requests + 1); `work` from `work_list`.
    Requests that are not in `work` keep their output rows untouched."""
    _need_cuda(out, query, key_cache, value_cache, block_tables, seq_lens, query_start_loc, work)
    if query.dim() != 3 or query.dtype not in ACT_DTYPES or query.stride(2) != 1 or out.shape != query.shape \
            or out.dtype != query.dtype or out.stride(2) != 1:
        raise ValueError(f"hk.ops.paged: prefill reads/writes (tokens, q_heads, head_dim) bfloat16 or float16; query "
                         f"{tuple(query.shape)} {query.dtype}, out {tuple(out.shape)} {out.dtype}")
    _, hq, d = query.shape
    if key_cache.dim() != 4 or value_cache.shape != key_cache.shape or key_cache.shape[3] != d \
            or key_cache.stride(3) != 1 or value_cache.stride(3) != 1:
        raise ValueError(f"hk.ops.paged: key_cache {tuple(key_cache.shape)} / value_cache {tuple(value_cache.shape)}: "
                         f"two (blocks, block_size, kv_heads, {d}) views needed")
    for name, t in (("block_tables", block_tables), ("seq_lens", seq_lens), ("query_start_loc", query_start_loc),
                    ("work", work)):
        if t.dtype != torch.int32 or t.stride(-1) != 1:
            raise TypeError(f"hk.ops.paged: {name} is {t.dtype} {tuple(t.shape)}; contiguous int32 needed")
    if work.dim() != 2 or work.shape[1] != 2 or not work.is_contiguous():
        raise ValueError("hk.ops.paged: work must be (items, 2) int32 (work_list)")
    code = kv_dtype_code(kv_cache_dtype, key_cache, query.dtype)
    fp8 = code == _lib.KV_FP8_E4M3
    _, bs, hkv, _ = key_cache.shape
    rc = _lib.load().hkb_paged_prefill(
        out.data_ptr(), out.stride(0), out.stride(1), query.data_ptr(), query.stride(0), query.stride(1),
        _cache_t(key_cache), _cache_t(value_cache), block_tables.data_ptr(), block_tables.stride(0),
        block_tables.shape[1], seq_lens.data_ptr(), query_start_loc.data_ptr(), work.data_ptr(), work.shape[0],
        query.shape[0], hq, hkv, d, bs, float(scale), code, _scale_ptr(k_scale, fp8, "k_scale"), _scale_ptr(v_scale, fp8, "v_scale"),
        _stream(query))
    _lib.check("hkb_paged_prefill", rc)
    return out


def merge_partials(out: torch.Tensor, part_out: torch.Tensor, part_lse: torch.Tensor,
                   out_lse: Optional[torch.Tensor] = None, seq_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fold `(parts, seqs, q_heads, head_dim)` fp32 normalised partials with their
    `(parts, seqs, q_heads)` natural-log lse into `out` `(seqs, q_heads, head_dim)` (bf16, or
    fp32 when `out_lse` `(seqs, q_heads)` is given so a second merge can follow). The same
    kernel folds one GPU's KV splits and the all-gathered partials of several GPUs."""
    _need_cuda(out, part_out, part_lse)
    p, n, hq, d = part_out.shape
    if part_out.dtype != torch.float32 or part_lse.dtype != torch.float32 or tuple(part_lse.shape) != (p, n, hq) \
            or not part_out.is_contiguous() or not part_lse.is_contiguous():
        raise ValueError("hk.ops.paged: merge reads contiguous fp32 (parts, seqs, heads, head_dim) and (parts, seqs, heads)")
    kind = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}.get(out.dtype)
    if tuple(out.shape) != (n, hq, d) or kind is None or out.stride(2) != 1:
        raise ValueError(f"hk.ops.paged: merge writes (seqs, heads, head_dim) bf16, fp16 or fp32, out is {tuple(out.shape)} {out.dtype}")
    if out_lse is not None and (out_lse.dtype != torch.float32 or tuple(out_lse.shape) != (n, hq)
                                or not out_lse.is_contiguous()):
        raise ValueError("hk.ops.paged: out_lse must be contiguous fp32 (seqs, heads)")
    rc = _lib.load().hkb_merge(out.data_ptr(), out.stride(0), out.stride(1), kind,
                               out_lse.data_ptr() if out_lse is not None else None,
                               part_out.data_ptr(), n * hq * d, hq * d, part_lse.data_ptr(), n * hq, hq,
                               p, n, hq, d, seq_lens.data_ptr() if seq_lens is not None else None, None,
                               _stream(out))
    _lib.check("hkb_merge", rc)
    return out


# --------------------------------------------------------------------------------------
# hk's own form: contract, plan, scratch, driver
# --------------------------------------------------------------------------------------

def check_decode(q, k_cache, v_cache, block_table, seq_lens, out, *, rows: str = "group",
                 head_dim: Optional[int] = None, scratch=None, splits: int = 1) -> None:
    """Refuse, before anything is launched, a decode whose tensors do not have the shapes the
    kernels read; ValueError names the tensor, the shape it has and the one it needs.

    The contract of python/hk/ops/paged.py:746-802: `q` and `out` are
    (requests, kv_heads, rows, head_dim) bf16 with 1..Q_TILE rows (the GQA group); the caches
    (blocks, kv_heads, page, head_dim) with page a multiple of 16, bf16 or fp8-e4m3;
    `block_table` (requests', pages) and `seq_lens` (requests',) int32 with requests' >=
    requests; `scratch` the split partials (`fused_scratch`). Contents are not read: that
    would be a device sync. Works on CPU tensors too (it only looks at metadata)."""

    def no(name, t, want):
        raise ValueError(f"hk.ops.paged: {name} is {tuple(t.shape)} {t.dtype}; the decode reads {want}")

    if q.dim() != 4:
        no("q", q, "(requests, kv_heads, rows, head_dim)")
    reqs, heads, n_rows, d = q.shape
    if head_dim is not None and d != head_dim:
        no("q", q, f"head_dim {head_dim} (this kernel's)")
    if d not in DECODE_HEAD_DIMS:
        no("q", q, f"head_dim in {DECODE_HEAD_DIMS}")
    if rows == "tile" and n_rows != Q_TILE:
        no("q", q, f"(requests, kv_heads, {Q_TILE}, head_dim): a whole {Q_TILE}-row tile")
    if not 1 <= n_rows <= Q_TILE:
        no("q", q, f"1 to {Q_TILE} query rows (the GQA group) a kv head")
    if q.dtype not in ACT_DTYPES:
        no("q", q, "bfloat16 or float16")
    if out.shape != q.shape or out.dtype != q.dtype:
        no("out", out, f"q's shape and dtype, {tuple(q.shape)} {q.dtype}")
    kinds = (q.dtype,) + (_FP8_DTYPES if q.dtype == torch.bfloat16 else ())
    for name, t in (("k_cache", k_cache), ("v_cache", v_cache)):
        if (t.dim() != 4 or t.shape[1] != heads or t.shape[3] != d or t.shape[2] % 16 or t.shape[2] == 0
                or t.dtype not in kinds):
            no(name, t, f"(blocks, {heads}, page, {d}) of q's dtype (or float8_e4m3fn with a bfloat16 q): q's kv heads, a page of a "
               f"multiple of 16 tokens, q's head_dim")
    if v_cache.shape != k_cache.shape or v_cache.dtype != k_cache.dtype:
        no("v_cache", v_cache, f"k_cache's shape and dtype, {tuple(k_cache.shape)} {k_cache.dtype}")
    if block_table.dim() != 2 or block_table.shape[0] < reqs or block_table.dtype != torch.int32:
        no("block_table", block_table, f"(requests >= {reqs}, pages) int32")
    if seq_lens.dim() != 1 or seq_lens.shape[0] < reqs or seq_lens.dtype != torch.int32:
        no("seq_lens", seq_lens, f"(requests >= {reqs},) int32")
    if splits > 1:
        if scratch is None:
            raise ValueError(f"hk.ops.paged: {splits} splits need scratch (fused_scratch)")
        o_part, lse = scratch
        if (o_part.dim() != 4 or o_part.shape[0] < reqs * splits or o_part.dtype != torch.float32
                or tuple(o_part.shape[1:]) != (heads, n_rows, d)):
            no("scratch o_part", o_part, f"(>= {reqs * splits}, {heads}, {n_rows}, {d}) float32: a row a "
               f"(request, split), q's group rows (fused_scratch)")
        if (lse.dim() != 3 or lse.shape[0] < reqs * splits or lse.dtype != torch.float32
                or tuple(lse.shape[1:]) != (heads, n_rows)):
            no("scratch lse_part", lse, f"(>= {reqs * splits}, {heads}, {n_rows}) float32 (fused_scratch)")


def fused_scratch(rows: int, n_kv_heads: int, head_dim: int, device, group: int = 4):
    """(o_part, lse_part) for `rows` = requests x splits: each split's normalised fp32 partial
    for the `group` query rows, and its natural-log lse (python/hk/ops/paged.py:733-743 keeps
    (m, l) pairs; one lse carries the same information)."""
    return (torch.empty(rows, n_kv_heads, group, head_dim, device=device, dtype=torch.float32),
            torch.empty(rows, n_kv_heads, group, device=device, dtype=torch.float32))


_SM_COUNT: dict = {}


def sm_count(device=None) -> int:
    """SMs of `device` (148 on a B200), or 148 where no GPU is present."""
    if not torch.cuda.is_available():
        return 148
    idx = torch.device(device).index if device is not None else None
    if idx is None:
        idx = torch.cuda.current_device()
    n = _SM_COUNT.get(idx)
    if n is None:
        n = _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def plan_splits(n_reqs: int, n_kv_heads: int, n_pages: int, device=None) -> int:
    """How many ways to cut the KV axis, given how empty the machine is.

    `n_pages` counts 16-token tiles of the longest sequence the plan must serve -- a host
    value (the table's width or max_model_len), never a step's lengths, so a captured graph's
    plan holds for every replay. `HK_SPLITS` = auto | off | 0 | 1 | N overrides as in
    python/hk/ops/paged.py:891-914; the result is a power of two as
    python/hk/integration/vllm_backend.py:137-151 rounds it."""
    forced = os.environ.get("HK_SPLITS", "auto").strip().lower() or "auto"
    if forced in ("off", "0", "1"):
        return 1
    if forced in ("auto", "plan"):
        return plan_splits_for(n_reqs, n_kv_heads, n_pages, sm_count(device))
    want = max(1, min(int(forced), max(1, n_pages), MAX_SPLITS))
    return 1 << (want.bit_length() - 1)


def plan_splits_for(n_reqs: int, n_kv_heads: int, n_pages: int, sms: int) -> int:
    """The planner's rule in Python, equal to hkb_plan_splits (tests hold them together): the
    partial slots a sequence gets. The tiles of all sequences of a kv head are dealt in equal
    shares to the W warps serving that head (two four-warp CTAs an SM, divided among the heads);
    1 + 8 W / n slots keep a sequence up to 8x the mean from limiting the shares; capped by the
    pieces the longest allowed sequence can usefully have (2 tiles a piece) and MAX_SPLITS; a power of two."""
    sms = sms if sms > 0 else 148
    n = max(1, n_reqs)
    w = max(1, (sms * 2) // max(1, n_kv_heads)) * 4
    want = 1 + -(-(8 * w) // n)
    cap = -(-n_pages // 2) + 1 if n_pages > 0 else 2
    want = max(2, min(want, cap))
    p = 1 << (want - 1).bit_length()
    return min(p, MAX_SPLITS)


def _row_stride(t: torch.Tensor) -> int:
    """Stride between consecutive query heads of an evenly strided (requests, kv_heads, group, d) tensor."""
    return t.stride(2) if t.shape[2] > 1 else t.stride(1)


def even_heads(t: torch.Tensor, name: str) -> None:
    """A (requests, kv_heads, group, head_dim) tensor can be read as (requests, q_heads, head_dim)
    only if head_dim is contiguous and a kv head's stride is group x the row stride; anything
    else (a transposed view, say) would be read at the wrong elements, so it is refused."""
    if t.dim() != 4 or t.stride(3) != 1 or (t.shape[2] > 1 and t.shape[1] > 1 and t.stride(1) != t.shape[2] * t.stride(2)):
        raise ValueError(f"hk.ops.paged: {name} has strides {tuple(t.stride())} for shape {tuple(t.shape)}; head_dim must be "
                         f"contiguous and the heads evenly strided (kv head stride = group x row stride)")


#: Shapes check_decode has passed (python/hk/ops/paged.py:805-825).
_PASSED: set = set()
_PASSED_CAP = 4096


def decode(q, k_cache, v_cache, block_table, seq_lens, out, scratch, splits: int, *,
           scale: Optional[float] = None, k_scale=None, v_scale=None) -> None:
    """The split decode's launches on hk's tensor forms: q/out (requests, kv_heads, group,
    head_dim), caches (blocks, kv_heads, page, head_dim). Checked against the contract once a
    shape (`check_decode`), then the walk and, with more than one split, the merge."""
    key = (q.shape, q.dtype, k_cache.shape, k_cache.dtype, v_cache.shape, block_table.shape, block_table.dtype,
           seq_lens.shape, seq_lens.dtype, out.shape, out.dtype, splits,
           scratch[0].shape if splits > 1 and scratch is not None else None,
           scratch[1].shape if splits > 1 and scratch is not None else None)
    if key not in _PASSED:
        check_decode(q, k_cache, v_cache, block_table, seq_lens, out, scratch=scratch, splits=splits)
        if len(_PASSED) < _PASSED_CAP:
            _PASSED.add(key)
    even_heads(q, "q")          # strides are not part of the shape key: checked on every call
    even_heads(out, "out")
    reqs, hkv, g, d = q.shape
    hq = hkv * g
    fp8 = k_cache.dtype not in ACT_DTYPES
    q3 = q.as_strided((reqs, hq, d), (q.stride(0), _row_stride(q), 1))
    o3 = out.as_strided((reqs, hq, d), (out.stride(0), _row_stride(out), 1))
    sc = None
    if splits > 1:
        sc = (scratch[0].view(-1, hq, d), scratch[1].view(-1, hq))
    paged_attention_decode(o3, q3, k_cache.transpose(1, 2), v_cache.transpose(1, 2), block_table[:reqs] if
                           block_table.shape[0] != reqs else block_table, seq_lens[:reqs] if
                           seq_lens.shape[0] != reqs else seq_lens, d ** -0.5 if scale is None else scale,
                           "fp8" if fp8 else "auto", k_scale, v_scale, num_splits=splits, scratch=sc)


def merge_splits(o_part: torch.Tensor, lse_part: torch.Tensor, splits: int, out: torch.Tensor) -> torch.Tensor:
    """Combine `splits` normalised partials `(requests x splits, kv_heads, group, head_dim)`
    and their lse `(requests x splits, kv_heads, group)` into `out` on the device: the kernel
    form of python/hk/ops/paged.py:283-317 (which folds unnormalised partials in torch; this
    build keeps ONE convention end to end -- normalised partial + natural-log lse)."""
    rs, hkv, g, d = o_part.shape
    reqs = rs // splits
    hq = hkv * g
    po = o_part.view(reqs, splits, hq, d)
    pl = lse_part.view(reqs, splits, hq)
    o3 = out.view(reqs, hq, d)
    rc = _lib.load().hkb_merge(o3.data_ptr(), o3.stride(0), o3.stride(1),
                               {torch.float32: 1, torch.float16: 2}.get(out.dtype, 0),
                               None, po.data_ptr(), hq * d, splits * hq * d, pl.data_ptr(), hq, splits * hq,
                               splits, reqs, hq, d, None, None, _stream(out))
    _lib.check("hkb_merge", rc)
    return out
