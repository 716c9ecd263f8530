"""In-place attention route: stand-ins with vLLM's own signatures that send a decode-only call
to this build's paged decode and a call with prefill in it to the paged prefill, both on the
engine's own cache, and everything else back to the engine's kernel, counted.

The decode half of hk-dsl's route (python/hk/integration/vllm_prefill.py:937-1095 for
`unified_attention`, :1287-1376 for `chunked_prefill_paged_decode`):

* a call is taken only if a predicate finds nothing it cannot serve (`d_why_not`,
  `rd_why_not`): decode-only, every feature the kernels do not implement off, every argument
  this module does not know at its default, bf16 queries, head size with a kernel, pages a
  multiple of 16, a GQA group of at most 16, contiguous int32 metadata, a cache layout the
  kernels can stride over (`layout_why_not`);
* anything else is `PATCH.count("fallback")` and the original function, which `apply()`
  kept when it rebound the name by identity in every imported vLLM module. The original is
  the ENGINE's code, not a second implementation of ours; without one, the call raises;
* decided on the batch alone, never on its lengths, and nothing is read back, so a captured
  CUDA graph replays what was decided at capture (`PATCH.guard`).

Unlike the reference, whose walk needs one of three exact cache orders (`_flash_kv`,
:599-628), the kernels here take the key and value caches as strided
`(blocks, page, kv_heads, head_dim)` views, so planes / tokens / heads orders and K|V side
by side are all read in place; fp8-e4m3 caches with per-tensor descales are taken too.
Switches: HK_VLLM_DECODE ("" or 1 = on, 0 = off), HK_VLLM_ROCM_DECODE (chunked_prefill_paged_decode, 1 = on).
"""

from __future__ import annotations

import inspect
import os
import sys
from typing import Callable, List, Optional

import torch

from ..ops import paged
from . import engine, switches
from ._common import rebind

PATCH = engine.Patch("vllm_prefill", ("prefill", "decode", "fallback"), graph="safe")

ARCHES = (switches.SM100,)

_ORIG_U: Optional[Callable] = None      # vLLM's unified_attention, kept by apply()
_U_SIG: Optional[inspect.Signature] = None
_ORIG_R: Optional[Callable] = None      # vLLM's chunked_prefill_paged_decode
_R_SIG: Optional[inspect.Signature] = None
_SCRATCH: dict = {}


def decode_switches(env: str):
    """(decode on at all, asked for explicitly) for an HK_VLLM_DECODE value."""
    v = (env or "").strip().lower()
    return v not in switches.OFF, v in switches.ON


DECODE, DECODE_ASKED = decode_switches(os.environ.get("HK_VLLM_DECODE", ""))
ROCM_DECODE = os.environ.get("HK_VLLM_ROCM_DECODE", "").strip().lower() in switches.ON

#: unified_attention's arguments that must be off for a call to be taken: name -> the test
_U_OFF = {
    "alibi_slopes": lambda v: v is None, "sinks": lambda v: v is None,
    "output_scale": lambda v: v is None, "qq_bias": lambda v: v is None,
    "mm_prefix_range": lambda v: v is None, "softcap": lambda v: not v,
    "q_descale": lambda v: v is None,
    "window_size": lambda v: v is None or tuple(v) == (-1, -1),
}

#: arguments this module reads, or that change nothing it computes (vLLM's own split-softmax
#: scratch for its 3-D kernel). Any other argument must be at its default, or the call falls back.
_U_READ = frozenset((
    "q", "k", "v", "out", "cu_seqlens_q", "max_seqlen_q", "seqused_k", "max_seqlen_k", "softmax_scale",
    "causal", "block_table", "k_descale", "v_descale", "seq_threshold_3D", "num_par_softmax_segments",
    "softmax_segm_output", "softmax_segm_max", "softmax_segm_expsum"))


def _unknown_set(a: dict, sig: Optional[inspect.Signature], known) -> str:
    """The first argument neither read nor tested that is not at its default, or ""."""
    for name, val in a.items():
        if name in known:
            continue
        p = sig.parameters.get(name) if sig is not None else None
        default = p.default if p is not None else None
        if val is default:
            continue
        try:
            if not hasattr(val, "shape") and val == default:
                continue
        except Exception:  # noqa: BLE001 -- an uncomparable value is a set one
            pass
        return name
    return ""


def page_why_not(page: int) -> str:
    return "" if page > 0 and page % 16 == 0 else f"page size {page} (a multiple of 16 needed)"


def layout_why_not(k, v) -> str:
    """Why the kernels cannot stride over these key / value cache views, or ""."""
    if k.dim() != 4 or v.shape != k.shape or v.dtype != k.dtype:
        return f"key/value caches {tuple(k.shape)} / {tuple(v.shape)}: not two (blocks, page, kv_heads, head_dim) views"
    if k.stride(-1) != 1 or v.stride(-1) != 1:
        return "key/value caches: head_dim not contiguous"
    es = k.element_size()
    for t in (k, v):
        if any((s * es) % 16 for s in t.stride()[:3]) or t.data_ptr() % 16:
            return "key/value caches: rows not 16-byte aligned (padded block?)"
    return ""


def _dtype_why_not(q, out, k, k_descale, v_descale) -> str:
    if q.dtype not in paged.ACT_DTYPES or out.dtype != q.dtype:
        return f"dtype {q.dtype} (bfloat16 or float16 queries only)"
    if k.dtype == q.dtype:
        return ""
    if k.dtype in paged._FP8_DTYPES:
        if q.dtype != torch.bfloat16:
            return f"fp8 cache with {q.dtype} queries (bfloat16 only)"
        for s in (k_descale, v_descale):
            if not isinstance(s, torch.Tensor) or s.numel() != 1 or s.dtype != torch.float32:
                return "fp8 cache without per-tensor float32 k/v descale"
        return ""
    return f"cache dtype {k.dtype}"


def _common_why_not(q, out, k, v, block_table, seq_lens, q_start, k_descale, v_descale) -> str:
    why = _dtype_why_not(q, out, k, k_descale, v_descale)
    if why:
        return why
    if q.dim() != 3 or q.shape[-1] not in paged.HEAD_DIMS:
        return f"head size {q.shape[-1]}"
    if k.dim() != 4:
        return f"cache {tuple(k.shape)}"
    why = page_why_not(int(k.shape[1]))
    if why:
        return why
    if q.shape[1] % k.shape[2] or q.shape[1] // k.shape[2] > paged.Q_TILE:
        return "query heads not a multiple of kv heads, or more than 16 a kv head"
    for t in (block_table, seq_lens, q_start):
        if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
            return "metadata not contiguous int32"
    if q.stride(-1) != 1 or out.stride(-1) != 1 or out.shape != q.shape:
        return "q / output head_dim not contiguous"
    return layout_why_not(k, v)


def d_why_not(a: dict) -> str:
    """Why this decode-only unified_attention call is not taken, or ""."""
    if switches.arch() not in ARCHES:
        return f"arch {switches.arch()}"
    if int(a.get("max_seqlen_q", 1)) != 1:
        return "not decode-only"
    for name, ok in _U_OFF.items():
        if name in a and not ok(a[name]):
            return f"{name} set"
    unknown = _unknown_set(a, _U_SIG, _U_READ | _U_OFF.keys())
    if unknown:
        return f"{unknown} set (an argument hk does not know)"
    return _common_why_not(a["q"], a["out"], a["k"], a["v"], a["block_table"], a["seqused_k"],
                           a.get("cu_seqlens_q"), a.get("k_descale"), a.get("v_descale"))


def _scratch(device, rows: int, hq: int, d: int):
    """The split partials, kept across calls (a captured graph holds them); grown outside a
    capture only -- None if a capture needs more than there is."""
    key = (str(device), hq, d)
    got = _SCRATCH.get(key)
    if got is None or got[0].shape[0] < rows:
        if engine.capturing():
            return None
        got = _SCRATCH[key] = paged.split_scratch(max(rows, 256), hq, d, 1, device)
    return got


def _decode(q, out, k, v, block_table, seq_lens, q_start, scale, k_descale, v_descale) -> bool:
    """This build's split decode on a decode-only batch; False if it cannot (falls back)."""
    n, hq, d = q.shape
    reqs = seq_lens.shape[0]
    hkv, page = int(k.shape[2]), int(k.shape[1])
    splits = paged.plan_splits(reqs, hkv, block_table.shape[1] * (page // 16), device=q.device)
    scratch = _scratch(q.device, reqs * splits, hq, d) if splits > 1 else None
    if splits > 1 and scratch is None:
        return False
    fp8 = k.dtype not in paged.ACT_DTYPES
    paged.paged_attention_decode(out, q, k, v, block_table, seq_lens, d ** -0.5 if scale is None else float(scale),
                                 "fp8" if fp8 else "auto", k_descale if fp8 else None, v_descale if fp8 else None,
                                 num_splits=splits, scratch=scratch, query_start_loc=q_start)
    return True


def u_why_not(a: dict) -> str:
    """Why this unified_attention call WITH prefill in it is not taken, or "". The same checks as
    a decode-only call, minus decode-only, plus: never under capture (the grid follows query
    lengths read on the host)."""
    if switches.arch() not in ARCHES:
        return f"arch {switches.arch()}"
    if engine.capturing():
        return "being captured (a mixed batch's grid follows its query lengths)"
    for name, ok in _U_OFF.items():
        if name in a and not ok(a[name]):
            return f"{name} set"
    if not a.get("causal", True):
        return "not causal"
    unknown = _unknown_set(a, _U_SIG, _U_READ | _U_OFF.keys())
    if unknown:
        return f"{unknown} set (an argument hk does not know)"
    return _common_why_not(a["q"], a["out"], a["k"], a["v"], a["block_table"], a["seqused_k"],
                           a.get("cu_seqlens_q"), a.get("k_descale"), a.get("v_descale"))


def _prefill(a: dict) -> bool:
    """The paged prefill on a batch with prefill in it (decodes included as one-row tiles)."""
    q, out, k = a["q"], a["out"], a["k"]
    hq, d = q.shape[1], q.shape[2]
    starts = a["cu_seqlens_q"].tolist()           # a host read: mixed batches are never captured
    reqs = len(starts) - 1
    work = paged.work_list([(r, starts[r + 1] - starts[r]) for r in range(reqs)],
                           paged.prefill_tile_rows(hq, int(k.shape[2])), q.device)
    sc = a.get("softmax_scale")
    fp8 = k.dtype not in paged.ACT_DTYPES
    paged.paged_prefill(out, q, k, a["v"], a["block_table"], a["seqused_k"], a["cu_seqlens_q"], work,
                        d ** -0.5 if sc is None else float(sc), "fp8" if fp8 else "auto",
                        a.get("k_descale") if fp8 else None, a.get("v_descale") if fp8 else None)
    return True


#: HK_VLLM_PREFILL_SHADOW=1 (the reference's switch, python/hk/integration/vllm_prefill.py:236-275):
#: after every call this module takes, the engine's own kernel runs on the same arguments into a
#: scratch output and the two are compared row by row in bf16 ulps of the row's largest value --
#: the in-situ check of a drop-in. It reads the device every call and doubles the attention work:
#: a diagnostic, never a serving mode, and skipped while a CUDA graph is being captured.
SHADOW = os.environ.get("HK_VLLM_PREFILL_SHADOW", "").strip().lower() not in ("", "0", "off", "false", "no")
SHADOW_STATS = {"calls": 0, "rows": 0, "worst_ulps": 0.0, "worst_call": -1, "over_4": 0}


def shadow_compare(ours: torch.Tensor, ref: torch.Tensor, stats: dict = SHADOW_STATS) -> float:
    """Worst row of `ours` against `ref`, (rows, heads, head_dim) each, in bf16 ulps of the
    reference row's largest magnitude (4 is the reference's own bound for this path,
    tests/hk/gpu/_attn_ref.py:43-44); counted into `stats`."""
    stats["calls"] += 1
    if ours.numel() == 0:
        return 0.0
    a, b = ours.float(), ref.float()
    top = b.abs().amax(dim=-1).clamp_min(1e-30)
    ulp = torch.exp2(torch.floor(torch.log2(top)) - 7)
    err = float(((a - b).abs().amax(dim=-1) / ulp).max())
    stats["rows"] += ours.shape[0]
    if err > stats["worst_ulps"]:
        stats["worst_ulps"], stats["worst_call"] = err, stats["calls"]
    if err > 4:
        stats["over_4"] += 1
    if err > 4 or stats["calls"] % 500 == 0:
        print(f"[hk] attention shadow: {stats}", file=sys.stderr, flush=True)
    return err


def _shadow(orig, a: dict, out_name: str, starts_name: str) -> None:
    if orig is None or engine.capturing():
        return
    ours = a[out_name]
    again = dict(a)
    again[out_name] = torch.empty_like(ours)
    orig(**again)
    starts = a.get(starts_name)
    live = int(starts[-1]) if starts is not None else ours.shape[0]      # a host read: diagnostic mode
    shadow_compare(ours[:live], again[out_name][:live], SHADOW_STATS)


def _fallback(orig, args, kwargs, why: str):
    PATCH.count("fallback")
    if orig is None:
        raise RuntimeError(f"hk vllm_prefill: call not taken ({why}) and there is no engine function to fall "
                           f"back to (apply() was not run inside an engine); this build has no second path")
    return orig(*args, **kwargs)


def unified_attention(*args, **kwargs):
    """vLLM's unified_attention (its signature, set on apply): a call with prefill in it goes to
    the paged prefill (python/hk/integration/vllm_prefill.py:1096-1163 of the reference), a
    decode-only call to the paged decode, anything the kernels do not take to the original."""
    a = kwargs if not args else _U_SIG.bind(*args, **kwargs).arguments
    if int(a.get("max_seqlen_q", 1)) > 1:
        why = u_why_not(a)
        if not why and _prefill(a):
            PATCH.count("prefill")
            if SHADOW:
                _shadow(_ORIG_U, dict(a), "out", "cu_seqlens_q")
            return None
        return _fallback(_ORIG_U, args, kwargs, why)
    why = "decode route off (HK_VLLM_DECODE=0)"
    if DECODE:
        why = d_why_not(a)
        if not why:
            if _decode(a["q"], a["out"], a["k"], a["v"], a["block_table"], a["seqused_k"], a.get("cu_seqlens_q"),
                       a.get("softmax_scale"), a.get("k_descale"), a.get("v_descale")):
                PATCH.count("decode")
                if SHADOW:
                    _shadow(_ORIG_U, dict(a), "out", "cu_seqlens_q")
                return None
            why = "scratch would grow under capture"
    return _fallback(_ORIG_U, args, kwargs, why)


#: chunked_prefill_paged_decode's arguments that must be off
_R_OFF = {
    "alibi_slopes": lambda v: v is None, "sliding_window": lambda v: not v or v < 0,
    "output_scale": lambda v: v is None, "sinks": lambda v: v is None,
    "is_block_table_ptr": lambda v: not v,
}
_R_READ = frozenset(("query", "key", "value", "output", "kv_cache_dtype", "key_cache", "value_cache", "block_table",
                     "query_start_loc", "seq_lens", "max_seq_len", "max_query_len", "k_scale", "v_scale",
                     "sm_scale", "causal"))


def _x_split_why_not(q, out, kc, vc, block_table, seq_lens, q_start) -> str:
    """The decode-only checks for ROCM_ATTN's own cache pair -- K (blocks, kv_heads, head_dim / x,
    page, x), V (blocks, kv_heads, head_dim, page) -- which the walk reads in place
    (python/hk/integration/vllm_prefill.py:1287-1330 of the reference)."""
    if q.dim() != 3:
        return f"query {tuple(q.shape)}"
    if q.dtype not in paged.ACT_DTYPES or out.dtype != q.dtype:
        return f"query / output {q.dtype} / {out.dtype}"
    why = paged.x_split_why_not(kc, vc, int(q.shape[-1]))
    if why:
        return why
    if kc.dtype != q.dtype:
        return f"x-split cache {kc.dtype} under {q.dtype} activations"
    if q.shape[1] % kc.shape[1] or q.shape[1] // kc.shape[1] > paged.Q_TILE:
        return "query heads not a multiple of kv heads, or more than 16 a kv head"
    if seq_lens.shape[0] > 2048:
        return f"{seq_lens.shape[0]} sequences (the x-split walk takes 2048)"
    for t in (block_table, seq_lens, q_start):
        if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
            return "metadata not contiguous int32"
    if q.stride(-1) != 1 or out.stride(-1) != 1 or out.shape != q.shape:
        return "q / output head_dim not contiguous"
    return ""


def _x_split_decode(q, out, kc, vc, block_table, seq_lens, q_start, scale) -> bool:
    """The split decode over x-split caches; False if its scratch would have to grow under capture."""
    n, hq, d = q.shape
    reqs = seq_lens.shape[0]
    hkv, page = int(kc.shape[1]), int(kc.shape[3])
    splits = max(2, paged.plan_splits(reqs, hkv, block_table.shape[1] * (page // 16), device=q.device))
    scratch = _scratch(q.device, reqs * splits, hq, d)
    if scratch is None:
        return False
    paged.paged_attention_decode_xsplit(out, q, kc, vc, block_table, seq_lens, d ** -0.5 if scale is None else float(scale),
                                        num_splits=splits, scratch=scratch, query_start_loc=q_start)
    return True


def rd_why_not(a: dict) -> str:
    """Why this decode-only chunked_prefill_paged_decode call is not taken, or ""."""
    if not ROCM_DECODE:
        return "HK_VLLM_ROCM_DECODE not set"
    if switches.arch() not in ARCHES:
        return f"arch {switches.arch()}"
    if int(a.get("max_query_len", 1)) != 1:
        return "not decode-only"
    for name, ok in _R_OFF.items():
        if name in a and not ok(a[name]):
            return f"{name} set"
    unknown = _unknown_set(a, _R_SIG, _R_READ | _R_OFF.keys())
    if unknown:
        return f"{unknown} set (an argument hk does not know)"
    kc, vc = a["key_cache"], a["value_cache"]
    if kc.dim() == 5:
        return _x_split_why_not(a["query"], a["output"], kc, vc, a["block_table"], a["seq_lens"],
                                a.get("query_start_loc"))
    return _common_why_not(a["query"], a["output"], kc, vc, a["block_table"], a["seq_lens"],
                           a.get("query_start_loc"), a.get("k_scale"), a.get("v_scale"))


def chunked_prefill_paged_decode(*args, **kwargs):
    """vLLM's chunked_prefill_paged_decode: a decode-only call on 4-D (blocks, page, kv_heads,
    head_dim) caches, or on its own x-split K / V^T pair, goes to the paged decode, anything else
    to the original."""
    a = kwargs if not args else _R_SIG.bind(*args, **kwargs).arguments
    why = rd_why_not(a)
    if not why:
        if a["key_cache"].dim() == 5:
            ran = _x_split_decode(a["query"], a["output"], a["key_cache"], a["value_cache"], a["block_table"],
                                  a["seq_lens"], a.get("query_start_loc"), a.get("sm_scale"))
        else:
            ran = _decode(a["query"], a["output"], a["key_cache"], a["value_cache"], a["block_table"], a["seq_lens"],
                          a.get("query_start_loc"), a.get("sm_scale"), a.get("k_scale"), a.get("v_scale"))
        if ran:
            PATCH.count("decode")
            if SHADOW:
                _shadow(_ORIG_R, dict(a), "output", "query_start_loc")
            return None
        why = "scratch would grow under capture"
    return _fallback(_ORIG_R, args, kwargs, why)


_GUARDED_U = PATCH.guard(unified_attention)
_GUARDED_R = PATCH.guard(chunked_prefill_paged_decode)
_REBOUND: List[tuple] = []


def apply() -> str:
    """Rebind vLLM's functions, by identity, in every vLLM module already imported. Run after
    vLLM's modules are imported and before a model runs. Returns a report line."""
    global _ORIG_U, _U_SIG, _ORIG_R, _R_SIG
    notes = []
    try:
        from vllm.v1.attention.ops import triton_unified_attention as tua  # noqa: PLC0415

        if tua.unified_attention is not _GUARDED_U:
            _ORIG_U = tua.unified_attention
            _U_SIG = inspect.signature(_ORIG_U)
            tua.unified_attention = _GUARDED_U
            names = rebind(("vllm",), _ORIG_U, _GUARDED_U)
            _REBOUND.append((tua, "unified_attention", _ORIG_U, _GUARDED_U))
            notes.append(f"unified_attention ({len(names)} imports rebound)")
    except Exception as e:  # noqa: BLE001 -- another vLLM: the route stays off, the engine is untouched
        notes.append(f"unified_attention not found ({type(e).__name__})")
    try:
        from vllm.v1.attention.ops import chunked_prefill_paged_decode as cpd  # noqa: PLC0415

        if cpd.chunked_prefill_paged_decode is not _GUARDED_R:
            _ORIG_R = cpd.chunked_prefill_paged_decode
            _R_SIG = inspect.signature(_ORIG_R)
            cpd.chunked_prefill_paged_decode = _GUARDED_R
            names = rebind(("vllm",), _ORIG_R, _GUARDED_R)
            _REBOUND.append((cpd, "chunked_prefill_paged_decode", _ORIG_R, _GUARDED_R))
            notes.append(f"chunked_prefill_paged_decode ({len(names)} imports rebound)")
    except Exception as e:  # noqa: BLE001
        notes.append(f"chunked_prefill_paged_decode not found ({type(e).__name__})")
    return "decode-only attention calls -> hk: " + "; ".join(notes)


def revert() -> None:
    """Put the engine's functions back."""
    for mod, name, orig, ours in _REBOUND:
        setattr(mod, name, orig)
        rebind(("vllm",), ours, orig)
    _REBOUND.clear()
