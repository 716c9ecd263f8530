"""The decoder attention backend: cache write + paged GQA decode on this build's kernels.

The shape of hk-dsl's backend (python/hk/integration/vllm_backend.py:532-781) with B200
kernels behind it:

* the cache is head-major, `(2, num_blocks, num_kv_heads, block_size, head_size)`, so one
  page of one head is 4 KB contiguous (bf16) -- the layout the walk streams best -- and the
  cache write reaches it through a `(blocks, block, heads, d)` transposed view (:582-599);
* `forward` writes the step's K/V, and a pure-decode step (max_query_len == 1, known on the
  host) runs the walk and, when the plan cuts the KV axis, the merge -- reading the query and
  writing the answer where the engine keeps them, with no copy, no sync and no allocation
  after the first call (:613-636, 700-728);
* the split count is a function of the batch size and max_model_len only, a power of two,
  so a CUDA graph captured on one batch is right for every replay (:137-151);
* what it does not implement raises with a sentence (:538-556): ALiBi, sliding windows,
  sinks, softcap, fused output quantisation, head sizes without a kernel. Unlike the
  reference it accepts an fp8-e4m3 KV cache with per-tensor k_scale / v_scale.
* a batch with prefill in it runs ONE paged-prefill launch over a host-built work list, decodes
  included (:637-698); it is never captured (its grid follows host-read query lengths).

`HKAttentionImplCore` has no vLLM import, so it is constructed and driven in tests with
plain tensors; `register()` wraps it in vLLM's classes when vLLM is importable.
"""

from __future__ import annotations

import os
from types import SimpleNamespace
from typing import Optional

import torch

from ..ops import paged
from . import engine

NAME = "HK_ATTN"

#: the enum member registered under: vLLM reserves CUSTOM for third-party backends and the
#: CUDA platform accepts it (`--attention-backend CUSTOM`); HK_VLLM_BACKEND_SLOT or a value in
#: HK_VLLM_BACKEND names another member to override instead.
SLOT = "CUSTOM"
_SLOT_NAME = SLOT

PATCH = engine.Patch("vllm_backend", ("decode", "prefill"), graph="safe")

#: decode scratch, one set per (device, q heads, head_dim) for every layer (layers run one
#: after another on one stream), allocated at its largest on first use so that a captured
#: graph's pointers stay valid
_SCRATCH: dict = {}
_UNIT: dict = {}


def _engine_limits():
    """(max_model_len, max_num_seqs) of the engine being built, or vLLM's defaults outside one."""
    try:
        from vllm.config import get_current_vllm_config  # noqa: PLC0415

        cfg = get_current_vllm_config()
        return int(cfg.model_config.max_model_len), int(cfg.scheduler_config.max_num_seqs)
    except Exception:  # noqa: BLE001 -- no engine: a bench, a test
        return 40960, 256


def _unit_scale(device):
    t = _UNIT.get(device)
    if t is None:
        t = _UNIT[device] = torch.ones((), device=device, dtype=torch.float32)
    return t


def _kv_scales(layer, device):
    """(k_scale, v_scale) tensors of the layer (vLLM keeps `_k_scale` / `_v_scale`), else 1."""
    ks = getattr(layer, "_k_scale", None)
    vs = getattr(layer, "_v_scale", None)
    one = _unit_scale(device)
    return (ks if isinstance(ks, torch.Tensor) else one), (vs if isinstance(vs, torch.Tensor) else one)


def _scratch(device, n_q_heads: int, head_dim: int, rows: int):
    key = (device, n_q_heads, head_dim)
    got = _SCRATCH.get(key)
    if got is None or got[0].shape[0] < rows:
        if engine.capturing():
            raise engine.GraphCaptureError(
                f"{NAME}: the decode scratch would have to grow to {rows} rows under CUDA-graph capture")
        got = _SCRATCH[key] = paged.split_scratch(rows, n_q_heads, head_dim, 1, device)
    return got


def decode_splits(n: int, n_kv_heads: int, pages_cap: int, device=None) -> int:
    """The decode's split count for `n` requests: a function of the batch size and of
    max_model_len (through `pages_cap`, in 16-token tiles), never of a step's lengths, and
    a power of two."""
    return paged.plan_splits(n, n_kv_heads, pages_cap, device=device)


def joined_step() -> bool:
    """HK_VLLM_JOINED_STEP=0 keeps the cache write of a decode step a launch of its own."""
    return os.environ.get("HK_VLLM_JOINED_STEP", "1") not in ("0", "false", "off", "no")


class HKAttentionImplCore:
    """vLLM's AttentionImpl constructor and forward, on plain tensors."""

    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int, alibi_slopes=None,
                 sliding_window=None, kv_cache_dtype: str = "auto", logits_soft_cap=None, attn_type=None,
                 kv_sharing_target_layer_name=None, sinks=None, **kw) -> None:
        unsupported = {"alibi_slopes": alibi_slopes, "sliding_window": sliding_window, "sinks": sinks}
        bad = [k for k, v in unsupported.items() if v is not None and v is not False and (
            not isinstance(v, (tuple, list)) or tuple(v) != (-1, -1))]
        if bad:
            raise NotImplementedError(
                f"{NAME} does not implement {', '.join(bad)}. The kernel is plain causal decode attention; "
                f"anything that changes the mask needs the mask written, not a flag threaded.")
        if logits_soft_cap:
            raise NotImplementedError(f"{NAME} has no logits_soft_cap")
        name = (kv_cache_dtype or "auto").lower()
        if not (name.startswith("auto") or name in ("fp8", "fp8_e4m3", "bfloat16", "float16", "half")):
            raise NotImplementedError(
                f"{NAME} keeps the cache in the model's 16-bit dtype (bfloat16 or float16) or in fp8-e4m3 "
                f"(per-tensor scales, bfloat16 models), not {kv_cache_dtype}")
        if kv_sharing_target_layer_name is not None:
            raise NotImplementedError(f"{NAME} has no cross-layer KV sharing")
        if num_heads % num_kv_heads or num_heads // num_kv_heads > paged.Q_TILE:
            raise ValueError(f"{NAME}: {num_heads} query heads over {num_kv_heads} kv heads: the GQA group "
                             f"must be a whole number of at most {paged.Q_TILE}")
        validate_head_size(head_size)
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = float(scale)
        self.num_kv_heads = num_kv_heads
        self.group = num_heads // num_kv_heads
        self.kv_cache_dtype = "fp8" if name.startswith("fp8") else "auto"
        self._checked = False
        max_len, max_seqs = _engine_limits()
        self._pages_cap = -(-max_len // 16)
        self._max_seqs = max_seqs
        self._splits: dict = {}
        self._rows: Optional[int] = None

    def _plan(self, n: int, device=None) -> int:
        s = self._splits.get(n)
        if s is None:
            s = self._splits[n] = decode_splits(n, self.num_kv_heads, self._pages_cap, device)
        return s

    def _scratch_rows(self, device) -> int:
        if self._rows is None:
            self._rows = max(self._max_seqs,
                             max(m * self._plan(m, device) for m in range(1, self._max_seqs + 1)))
        return self._rows

    # -- the cache ---------------------------------------------------------------------

    def _kv(self, kv_cache):
        """(k_cache, v_cache), each (blocks, kv_heads, block, head_dim): the (2, ...) tensor of
        `get_kv_cache_shape`, or [B, H, N, 2C] with K and V side by side in the last axis."""
        if kv_cache.dim() == 5:
            return kv_cache[0], kv_cache[1]
        d = self.head_size
        return kv_cache[..., :d], kv_cache[..., d:2 * d]

    def _update_cache(self, layer, key, value, k_cache, v_cache, slot_mapping):
        """The cache write into head-major pages through the (blocks, block, heads, d) view; slot
        -1 -- a CUDA graph's padding token -- is skipped."""
        ks, vs = _kv_scales(layer, key.device)
        paged.reshape_and_cache(key, value, k_cache.transpose(1, 2), v_cache.transpose(1, 2), slot_mapping,
                                self.kv_cache_dtype, ks, vs)

    # -- the launch --------------------------------------------------------------------

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        if attn_metadata is None:                 # profiling run
            return output.fill_(0)
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError(f"{NAME} has no fused output quant")
        n = attn_metadata.num_actual_tokens
        k_cache, v_cache = self._kv(kv_cache)
        decode_only = attn_metadata.max_query_len == 1      # a host int: no device read
        new = None
        if key is not None and value is not None:
            if decode_only and joined_step():
                # one token a request: the walk writes each request's new row itself, just before it
                # reads the tile the row lands in (two launches a layer instead of three)
                new = (key[:n], value[:n], attn_metadata.slot_mapping[:n])
            else:
                self._update_cache(layer, key[:n], value[:n], k_cache, v_cache, attn_metadata.slot_mapping[:n])
        if decode_only:
            self._decode_all(query, output, k_cache, v_cache, attn_metadata, n, layer, new)
            return output
        if engine.capturing():
            raise engine.GraphCaptureError(
                f"{NAME} is being captured on a batch with prefill in it. It claims "
                f"UNIFORM_SINGLE_TOKEN_DECODE: a prefill step reads its query lengths on the host, which a "
                f"replay would not repeat.")
        # A step with prefill in it: every new token's K/V is in the cache by now, so ONE paged
        # prefill launch over a host-built work list serves the whole batch -- chunks, cached
        # prefixes and the one-token decodes riding along (a lone token is a one-row tile).
        self._prefill(query, output, k_cache, v_cache, attn_metadata, n, layer)
        PATCH.count("prefill")
        return output

    def _prefill(self, query, output, k_cache, v_cache, attn_metadata, n, layer=None):
        """The batch's rows as (tokens, heads, head_dim); the work list comes from the metadata
        builder (`hk_prefill_work`, built on the host where the query lengths already are) or, for
        a caller without one, from query_start_loc read back here (never under capture)."""
        hq, d = self.num_heads, self.head_size
        work = getattr(attn_metadata, "hk_prefill_work", None)
        qsl = attn_metadata.query_start_loc
        reqs = qsl.shape[0] - 1
        if not self._checked:
            self._check(attn_metadata.block_table[:reqs], attn_metadata.seq_lens[:reqs])
        if work is None:
            starts = qsl.tolist()
            work = paged.work_list([(r, starts[r + 1] - starts[r]) for r in range(reqs)],
                                   paged.prefill_tile_rows(hq, self.num_kv_heads), query.device)
        paged.paged_prefill(output[:n].view(n, hq, d), query[:n].view(n, hq, d), k_cache.transpose(1, 2),
                            v_cache.transpose(1, 2), attn_metadata.block_table, attn_metadata.seq_lens, qsl, work,
                            self.scale, self.kv_cache_dtype, *_kv_scales(layer, query.device))

    def _decode_all(self, query, output, k_cache, v_cache, attn_metadata, n, layer=None, new=None):
        """Every request has exactly one token: the walk and its merge, reading the query and
        writing the answer where the engine keeps them. `new`: (key, value, slot_mapping) of the
        step when the cache write rides in the walk."""
        hq, d = self.num_heads, self.head_size
        q = query[:n].view(n, hq, d)
        out = output[:n].view(n, hq, d)
        table = attn_metadata.block_table[:n]
        lens = attn_metadata.seq_lens[:n]
        if not self._checked and not engine.capturing():
            self._check(table, lens, k_cache.shape[2])       # head-major cache: (blocks, kv_heads, page, d)
        splits = self._plan(n, query.device)
        scratch = None
        if splits > 1:
            po, pl = _scratch(query.device, hq, d, self._scratch_rows(query.device))
            scratch = (po, pl)
        ks, vs = _kv_scales(layer, query.device)
        if new is not None:
            paged.decode_step(out, q, new[0], new[1], k_cache.transpose(1, 2), v_cache.transpose(1, 2), new[2], table,
                              lens, self.scale, self.kv_cache_dtype, ks, vs, num_splits=splits, scratch=scratch)
        else:
            paged.paged_attention_decode(out, q, k_cache.transpose(1, 2), v_cache.transpose(1, 2), table, lens,
                                         self.scale, self.kv_cache_dtype, ks, vs, num_splits=splits, scratch=scratch)
        PATCH.count("decode")

    def _check(self, table, lens, block_size: int = paged.KV_BLOCK):
        """Once per layer object, never under capture: it reads the device. The kernel reads
        these two as int32 and indexes memory with the result. `block_size` is the page size of
        the cache in hand (16, 32, 64 or a hybrid model's larger page): a table column is one such
        page. The reference counts with its constant because it refuses any page but 16
        (python/hk/integration/vllm_backend.py:490, 731-753)."""
        self._checked = True
        for name, t in (("block_table", table), ("seq_lens", lens)):
            if t.dtype != torch.int32 or t.stride(-1) != 1:
                raise TypeError(f"{NAME}: {name} is {t.dtype} strides {t.stride()} {tuple(t.shape)}; the kernel "
                                f"reads it as int32 with contiguous rows.")
        if lens.numel():
            mx = int(lens.max())
            cols = table.shape[-1]
            need = -(-mx // max(1, int(block_size)))
            if need > cols:
                raise ValueError(f"{NAME}: seq_len {mx} needs {need} pages of {block_size} tokens but block_table "
                                 f"has {cols} columns.")


def validate_head_size(head_size: int) -> None:
    if head_size not in paged.HEAD_DIMS:
        raise ValueError(f"{NAME} has kernels for head_size {list(paged.HEAD_DIMS)}, not {head_size}.")


def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                       cache_dtype_str: str = "auto") -> tuple:
    """Head-major pages: (2, num_blocks, num_kv_heads, block_size, head_size)."""
    if block_size % 16:
        raise ValueError(f"{NAME} needs a block_size that is a multiple of 16, got {block_size}")
    return (2, num_blocks, num_kv_heads, block_size, head_size)


def metadata(num_actual_tokens, slot_mapping, block_table, seq_lens, max_query_len=1, query_start_loc=None,
             max_seq_len=0):
    """The fields of vLLM's attention metadata this backend reads
    (tests/hk/engines/test_vllm_contract.py:241-257), for callers outside an engine."""
    return SimpleNamespace(num_actual_tokens=num_actual_tokens, slot_mapping=slot_mapping, block_table=block_table,
                           seq_lens=seq_lens, max_query_len=max_query_len, query_start_loc=query_start_loc,
                           max_seq_len=max_seq_len)


# --------------------------------------------------------------------------- vLLM classes

_BUILT: list = []


def _build():
    """(HKAttentionBackend, HKAttentionImpl) as vLLM subclasses; needs vLLM."""
    if _BUILT:
        return _BUILT[0]
    from typing import ClassVar  # noqa: PLC0415

    from vllm.v1.attention.backend import AttentionBackend, AttentionImpl  # noqa: PLC0415

    class HKAttentionImpl(HKAttentionImplCore, AttentionImpl):
        pass

    class HKAttentionBackend(AttentionBackend):
        accept_output_buffer: bool = True
        supported_dtypes: ClassVar[list] = [torch.bfloat16, torch.float16]
        supported_kv_cache_dtypes: ClassVar[list] = ["auto", "bfloat16", "float16", "fp8", "fp8_e4m3"]

        @staticmethod
        def get_name() -> str:
            return _SLOT_NAME

        @staticmethod
        def get_impl_cls():
            return HKAttentionImpl

        @staticmethod
        def get_builder_cls():
            # block_table, seq_lens, slot_mapping, query_start_loc, max_query_len are exactly
            # what vLLM's Triton backend's builder already assembles
            from vllm.v1.attention.backends.triton_attn import TritonAttentionMetadataBuilder  # noqa: PLC0415

            rows = paged.prefill_tile_rows

            class HKAttentionMetadataBuilder(TritonAttentionMetadataBuilder):
                """vLLM's builder plus the prefill work list, made on the host where vLLM already
                has the query lengths (python/hk/integration/vllm_backend.py:447-471 of the
                reference does the same in its builder)."""

                def build(self, common_prefix_len, common_attn_metadata, fast_build=False):
                    md = super().build(common_prefix_len, common_attn_metadata, fast_build)
                    md.hk_prefill_work = None
                    if getattr(common_attn_metadata, "max_query_len", 1) > 1:
                        qs = common_attn_metadata.query_start_loc_cpu.tolist()
                        spec = getattr(self, "kv_cache_spec", None)
                        hkv = getattr(spec, "num_kv_heads", None)
                        hq = getattr(self, "num_heads_q", None)
                        if hkv and hq:
                            md.hk_prefill_work = paged.work_list(
                                [(r, qs[r + 1] - qs[r]) for r in range(len(qs) - 1)], rows(hq, hkv), self.device)
                    return md

            return HKAttentionMetadataBuilder

        @staticmethod
        def get_supported_kernel_block_sizes():
            return [16, 32, 64]

        @classmethod
        def get_supported_head_sizes(cls) -> list:
            return list(paged.HEAD_DIMS)

        @staticmethod
        def get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size, cache_dtype_str="auto"):
            return get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size, cache_dtype_str)

        @classmethod
        def validate_head_size(cls, head_size: int) -> None:
            validate_head_size(head_size)

        @staticmethod
        def use_cascade_attention(*args, **kwargs) -> bool:
            return False

    _BUILT.append((HKAttentionBackend, HKAttentionImpl))
    return _BUILT[0]


def register(slot: Optional[str] = None) -> str:
    """Register the backend with vLLM. Idempotent."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend  # noqa: PLC0415

    want = slot or os.environ.get("HK_VLLM_BACKEND_SLOT", SLOT)
    globals()["_SLOT_NAME"] = want
    backend, impl = _build()
    globals()["HKAttentionBackend"] = backend
    globals()["HKAttentionImpl"] = impl
    member = getattr(AttentionBackendEnum, want, None)
    if member is None:
        raise RuntimeError(f"this vLLM has no AttentionBackendEnum.{want}; the members it has are "
                           f"{sorted(m.name for m in AttentionBackendEnum)}. Set HK_VLLM_BACKEND_SLOT to one of them.")
    register_backend(member, f"{__name__}.HKAttentionBackend")
    return f"{NAME} registered over {want} (--attention-backend {want})"
