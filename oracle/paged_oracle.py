"""CPU oracle of the paged KV path. TEST INFRASTRUCTURE ONLY.

A torch (CPU) restatement of what hk-dsl holds this path to. Only `tests/`,
`__graft_entry__.smoke()` and `bench.py`'s CPU-baseline / reference legs may import it;
the product (the `hk_dsl_b200` package) never does, and has no CPU path of its own.

The reference's device kernels are generated HIP for AMD GPUs and cannot run here, so the
oracle restates the reference's *own torch reference code* for the path, function by
function:

* `reshape_and_cache_ref`  -- the torch scatter of tests/hk/gpu/test_vllm_backend_decode.py:44-49
  (`want[0][s // PAGE, :, s % PAGE] = key[live]`, `live = slots >= 0`) and
  examples/09_kv_scatter.py:62-65.
* `softmax_v64`            -- tests/hk/gpu/_attn_ref.py:71-77 (explicit softmax in float64).
* `paged_decode_ref`       -- `_reference` of tests/hk/gpu/test_paged_decode.py:89-101 and
  tests/hk/gpu/test_vllm_backend_decode.py:74-86 (gather `table[i, :ceil(s/page)]`, cat pages,
  `[:s]`, q head hh reads kv head hh // group; a request of length 0 answers zeros).
* `paged_prefill_ref`      -- `_reference` of tests/hk/gpu/test_paged_prefill.py:54-70 (causal, cached
  prefix: query row j of a request at position ctx + j keeps keys <= its position).
* `paged_decode_ref_fp32`  -- the vectorised fp32 form of tools/hk-bench/paged_cdna.py:132-140
  (the fairer speed baseline).
* `merge_splits_unnormalised` -- python/hk/ops/paged.py:283-317 verbatim in meaning
  (unnormalised numerators, (m, l) in the log2 domain).
* `merge_lse_ref`          -- the same fold in this build's single convention: normalised
  partials + natural-log lse.
* `rel`, `ulps`, `check`   -- tests/hk/gpu/_attn_ref.py:80-107 (4 bf16 ulps a row, 2^-6 relative),
  and `check_baseline` the max-abs 2e-2 / mean-abs 2e-3 bound this build states for itself.

Pinning: `tests/golden/make_golden.py` runs the reference's `_attn_ref.py` (loaded by path)
and the reference's `merge_splits` (its source text executed stand-alone) in the build
container and stores their outputs; `tests/test_oracle_golden.py` holds this file to them.
fp8 (`quantize_fp8`, `dequantize_fp8`): the reference refuses fp8 KV caches
(python/hk/integration/vllm_backend.py:552-556), so for fp8 there is nothing of the
reference's to pin against -- PARITY UNPINNED for the fp8 scatter; it is defined here as
clamp(float(x) / scale, +-448) rounded to nearest-even e4m3fn, and checked against torch's
own float8_e4m3fn cast.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

ULPS = 4.0
TOL = 2.0 ** -6
MAX_ABS = 2e-2
MEAN_ABS = 2e-3
FP8_MAX = 448.0


# ----------------------------------------------------------------------------- fp8

def quantize_fp8(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """float(x) / scale, saturated to +-448, rounded to nearest-even e4m3fn.
    torch's cast does not saturate (465 -> NaN), hence the clamp first."""
    y = (x.float() / scale.float()).clamp(-FP8_MAX, FP8_MAX)
    return y.to(torch.float8_e4m3fn)


def dequantize_fp8(c: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    if c.dtype == torch.uint8:
        c = c.view(torch.float8_e4m3fn)
    return c.float() * scale.float()


# ------------------------------------------------------------------------- scatter

def reshape_and_cache_ref(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype="auto",
                          k_scale=None, v_scale=None) -> None:
    """In place on `(blocks, block_size, kv_heads, head_dim)` cache views: for live slots
    `cache[s // bs, s % bs] = key[live]`; fp8 caches take `quantize_fp8`."""
    bs = key_cache.shape[1]
    live = slot_mapping >= 0
    s = slot_mapping[live].long()
    fp8 = not str(kv_cache_dtype).startswith("auto")
    for src, dst, sc in ((key, key_cache, k_scale), (value, value_cache, v_scale)):
        rows = src[live]
        if fp8:
            rows = quantize_fp8(rows, sc)
            if dst.dtype == torch.uint8:
                rows = rows.view(torch.uint8)
        dst[s // bs, s % bs] = rows


# ----------------------------------------------------------------------- attention

def softmax_v64(qq, kk, vv, scale, keep=None):
    """One head: softmax(qq kk^T * scale) vv in float64 (2-D operands); float32 out."""
    s = (qq.double() @ kk.double().T) * scale
    if keep is not None:
        s = s.masked_fill(~keep, float("-inf"))
    return (torch.softmax(s, dim=-1) @ vv.double()).float()


def _as_float_cache(c, scale):
    if c.dtype in (torch.float8_e4m3fn, torch.uint8):
        return dequantize_fp8(c, scale)
    return c


def paged_decode_ref(q, key_cache, value_cache, block_tables, seq_lens, scale: Optional[float] = None,
                     k_scale=None, v_scale=None, query_start_loc=None):
    """Exact decode attention in float64, float32 out `(rows, q_heads, head_dim)`.

    Caches are `(blocks, block_size, kv_heads, head_dim)` views (fp8 caches are dequantised
    first, so the answer is the fp32/fp64 evaluation of the dequantised cache). Rows without
    a query (query_start_loc) and requests of length 0 stay zero."""
    n_rows, h, d = q.shape
    page, hkv = key_cache.shape[1], key_cache.shape[2]
    group = h // hkv
    scale = d ** -0.5 if scale is None else scale
    kc = _as_float_cache(key_cache, k_scale)
    vc = _as_float_cache(value_cache, v_scale)
    out = torch.zeros(n_rows, h, d, dtype=torch.float32)
    lens = seq_lens.tolist()
    qsl = query_start_loc.tolist() if query_start_loc is not None else None
    for i, s in enumerate(lens):
        if s <= 0:
            continue
        row = i
        if qsl is not None:
            if qsl[i + 1] <= qsl[i]:
                continue
            row = qsl[i]
        pages = block_tables[i, : -(-s // page)].long()
        kk_all = kc[pages].reshape(-1, hkv, d)[:s]      # (tokens, kv heads, d)
        vv_all = vc[pages].reshape(-1, hkv, d)[:s]
        for kh in range(hkv):
            heads = slice(kh * group, (kh + 1) * group)
            out[row, heads] = softmax_v64(q[row, heads], kk_all[:, kh], vv_all[:, kh], scale)
    return out


def paged_decode_ref_fp32(q, key_cache, value_cache, block_tables, seq_lens, scale: Optional[float] = None,
                          k_scale=None, v_scale=None, rows: Optional[Sequence[int]] = None):
    """The vectorised fp32 form (one einsum pair a request)."""
    n, h, d = q.shape
    page, hkv = key_cache.shape[1], key_cache.shape[2]
    g = h // hkv
    scale = d ** -0.5 if scale is None else scale
    out = torch.zeros(n, h, d, dtype=torch.float32)
    lens = seq_lens.tolist()
    for i in (range(len(lens)) if rows is None else rows):
        s = lens[i]
        if s <= 0:
            continue
        pages = block_tables[i, : -(-s // page)].long()
        kk = _as_float_cache(key_cache[pages], k_scale).reshape(-1, hkv, d)[:s].float()
        vv = _as_float_cache(value_cache[pages], v_scale).reshape(-1, hkv, d)[:s].float()
        qq = q[i].float().view(hkv, g, d)
        sc = torch.einsum("hgd,nhd->hgn", qq, kk) * scale
        out[i] = torch.einsum("hgn,nhd->hgd", torch.softmax(sc, -1), vv).reshape(h, d)
    return out


def paged_prefill_ref(q, key_cache, value_cache, block_tables, seq_lens, query_start_loc, scale=None):
    """Causal prefill over a paged cache in float64, float32 out: the `_reference` of
    tests/hk/gpu/test_paged_prefill.py:54-70 -- request i's q_len new tokens are the last q_len of
    its seq_lens[i] cached tokens; query row j sits at position ctx + j and keeps keys <= it."""
    n_tok, h, d = q.shape
    page, hkv = key_cache.shape[1], key_cache.shape[2]
    group = h // hkv
    scale = d ** -0.5 if scale is None else scale
    out = torch.zeros(n_tok, h, d, dtype=torch.float32)
    qsl, lens = query_start_loc.tolist(), seq_lens.tolist()
    for i in range(len(lens)):
        q0, q1, s = qsl[i], qsl[i + 1], lens[i]
        n, ctx = q1 - q0, s - (q1 - q0)
        if n <= 0:
            continue
        pages = block_tables[i, : -(-s // page)].long()
        kk_all = key_cache[pages].reshape(-1, hkv, d)[:s]
        vv_all = value_cache[pages].reshape(-1, hkv, d)[:s]
        pos = ctx + torch.arange(n)
        keep = torch.arange(s)[None, :] <= pos[:, None]
        for hh in range(h):
            out[q0:q1, hh] = softmax_v64(q[q0:q1, hh], kk_all[:, hh // group], vv_all[:, hh // group], scale, keep)
    return out


def partial_ref(q_row, kk, vv, scale):
    """(normalised out fp32 `(heads, d)`, natural-log lse `(heads,)`) of one kv head's group
    over tokens kk/vv, in float64; an empty range gives (zeros, -inf)."""
    if kk.shape[0] == 0:
        return (torch.zeros(q_row.shape[0], q_row.shape[1], dtype=torch.float32),
                torch.full((q_row.shape[0],), float("-inf"), dtype=torch.float32))
    s = (q_row.double() @ kk.double().T) * scale
    lse = torch.logsumexp(s, dim=-1)
    return (torch.softmax(s, dim=-1) @ vv.double()).float(), lse.float()


# --------------------------------------------------------------------------- merge

def merge_splits_unnormalised(o_part, ml_part, splits: int, out):
    """python/hk/ops/paged.py:283-317: o_part `(reqs*splits, hkv, tile, d)` unnormalised
    numerators under each split's own maximum, ml_part `(reqs*splits, hkv, 2, tile)` = (m, l)
    in the log2 domain; numerator and denominator both take exp2(m_s - m_max)."""
    r_s, hkv, tile, d = o_part.shape
    reqs = r_s // splits
    o = o_part.view(reqs, splits, hkv, tile, d)
    m = ml_part.view(reqs, splits, hkv, 2, tile)[:, :, :, 0]
    l = ml_part.view(reqs, splits, hkv, 2, tile)[:, :, :, 1]
    m_max = m.amax(dim=1, keepdim=True)
    rescale = torch.exp2(m - m_max)
    num = (o * rescale.unsqueeze(-1)).sum(dim=1)
    den = (l * rescale).sum(dim=1).clamp_min(1e-30)
    out.copy_((num / den.unsqueeze(-1)).to(out.dtype))
    return out


def merge_lse_ref(part_out, part_lse):
    """`(parts, seqs, heads, d)` normalised partials + `(parts, seqs, heads)` natural-log lse
    -> (out fp32 `(seqs, heads, d)`, lse `(seqs, heads)`), in float64. Parts with lse = -inf
    carry weight 0 whatever they hold; all -inf answers zero."""
    lse = part_lse.double()
    mx = lse.amax(dim=0, keepdim=True)
    mx_safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    w = torch.exp(lse - mx_safe)
    w = torch.where(torch.isinf(lse) & (lse < 0), torch.zeros_like(w), w)
    po = torch.where((w == 0).unsqueeze(-1), torch.zeros_like(part_out, dtype=torch.float64), part_out.double())
    den = w.sum(dim=0)
    num = (po * w.unsqueeze(-1)).sum(dim=0)
    out = torch.where(den.unsqueeze(-1) > 0, num / den.clamp_min(1e-300).unsqueeze(-1), torch.zeros_like(num))
    out_lse = torch.where(den > 0, mx_safe[0] + torch.log(den.clamp_min(1e-300)), torch.full_like(den, float("-inf")))
    return out.float(), out_lse.float()


def to_lse_convention(o_part_unnorm, ml_part):
    """(m, l) log2-domain unnormalised partials -> this build's (normalised out, natural lse)."""
    m = ml_part[:, :, 0]
    l = ml_part[:, :, 1]
    out = o_part_unnorm / l.clamp_min(1e-30).unsqueeze(-1)
    lse = (m + torch.log2(l.clamp_min(1e-300))) * math.log(2.0)
    return out, lse


# ---------------------------------------------------------------------- tolerances

def rel(got, want) -> float:
    got, want = got.float(), want.float()
    return ((got - want).abs().max() / want.abs().max().clamp_min(1e-30)).item()


def ulps(got, want) -> float:
    """Worst row's error in bf16 ulps of that row's largest |want| (a row = the last axis)."""
    d = want.shape[-1]
    g, w = got.float().reshape(-1, d), want.float().reshape(-1, d)
    m = w.abs().amax(-1).clamp_min(2.0 ** -126)
    ulp = torch.exp2(torch.floor(torch.log2(m)) - 7)
    return ((g - w).abs().amax(-1) / ulp).max().item()


def check(got, want) -> float:
    """The reference's bound: worst row within ULPS bf16 ulps, max-abs / max-ref < TOL."""
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all().item(), "output has non-finite elements"
    r, u = rel(got, want), ulps(got, want)
    assert u < ULPS and r < TOL, (
        f"worst row off by {u:.2f} bf16 ulps of its largest value (bound {ULPS}); "
        f"max |got - want| / max |want| = {r:.2e} (bound {TOL})")
    return r


def check_baseline(got, want) -> tuple:
    """This build's stated tolerance: max-abs <= 2e-2 and mean-abs <= 2e-3."""
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all().item(), "output has non-finite elements"
    err = (got - want).abs()
    mx, mean = err.max().item(), err.mean().item()
    assert mx <= MAX_ABS and mean <= MEAN_ABS, f"max-abs {mx:.3e} (bound {MAX_ABS}), mean-abs {mean:.3e} (bound {MEAN_ABS})"
    return mx, mean
