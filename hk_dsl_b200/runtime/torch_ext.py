"""The kernels as `torch.ops.hk.*`: opaque custom ops with out-parameters that return `()`.

hk-dsl exposes every compiled kernel as `torch.ops.hk.<name>` whose schema is the kernel's
tensors in declaration order, written tensors marked `(a!)`, returning nothing
(python/hk/codegen/scaffold.py:264-275, python/hk/runtime/torch_ext.py:102-174,
python/hk/runtime/codeobj.py:582-629), and calls them directly in eager code. There every
(head_dim, splits) pair is its own compiled kernel and so its own op name; here the same
names are registered on demand onto ONE runtime-parameterised C entry point:

    hk::reshape_and_cache(key, value, key_cache!, value_cache!, slot_mapping, kv_cache_dtype, k_scale, v_scale)
    hk::paged_attention_decode(out!, query, key_cache, value_cache, block_tables, seq_lens, scale,
                               kv_cache_dtype, k_scale, v_scale, num_splits, part_out!, part_lse!)
    hk::paged_decode_step(out!, query, key, value, key_cache!, value_cache!, slot_mapping, block_tables, seq_lens,
                          scale, kv_cache_dtype, k_scale, v_scale, num_splits, part_out!, part_lse!)
    hk::paged_decode_fused_d{D}_s{S}(q, k_cache, v_cache, block_table, seq_lens, out!, o_part!, ml_part!)
    hk::paged_merge_d{D}_s{S}(seq_lens, out!, o_part, ml_part)
    hk::paged_prefill_d{D}_g{G}(q, k_cache, v_cache, block_table, seq_lens, q_start, tiles, out!)

The split scratch (`o_part`, `ml_part`) is this build's: fp32 normalised partials and their
natural-log lse (`hk_dsl_b200.ops.paged.fused_scratch`), caller-owned and allocated once.
"""

from __future__ import annotations

from typing import Callable, Dict

import torch

from ..integration import engine
from ..ops import paged

NS = "hk"
_OPS: Dict[str, engine.Op] = {}


def _nothing(*args, **kwargs):
    return None


def _define(name: str, schema: str, impl: Callable) -> engine.Op:
    op = _OPS.get(name)
    if op is None:
        op = engine.Op(f"{NS}::{name}", f"{name}{schema}", _nothing, ("launch",))
        op.define(impl, dispatch="CUDA")
        _OPS[name] = op
    return op


def _reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale):
    paged.reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale)


def _paged_attention_decode(out, query, key_cache, value_cache, block_tables, seq_lens, scale, kv_cache_dtype,
                            k_scale, v_scale, num_splits, part_out, part_lse):
    paged.paged_attention_decode(out, query, key_cache, value_cache, block_tables, seq_lens, scale,
                                 kv_cache_dtype, k_scale, v_scale, num_splits=num_splits,
                                 scratch=(part_out, part_lse) if num_splits > 1 else None)


def _paged_decode_step(out, query, key, value, key_cache, value_cache, slot_mapping, block_tables, seq_lens, scale,
                       kv_cache_dtype, k_scale, v_scale, num_splits, part_out, part_lse):
    paged.decode_step(out, query, key, value, key_cache, value_cache, slot_mapping, block_tables, seq_lens, scale,
                      kv_cache_dtype, k_scale, v_scale, num_splits=num_splits,
                      scratch=(part_out, part_lse) if num_splits > 1 else None)


def paged_decode_step_op() -> engine.Op:
    """The cache write of a decode step and its attention as one op: the walk writes the new rows
    (two launches where `reshape_and_cache` + `paged_attention_decode` are three)."""
    return _define(
        "paged_decode_step",
        "(Tensor(a!) out, Tensor query, Tensor key, Tensor value, Tensor(b!) key_cache, Tensor(c!) value_cache, "
        "Tensor slot_mapping, Tensor block_tables, Tensor seq_lens, float scale, str kv_cache_dtype, Tensor k_scale, "
        "Tensor v_scale, int num_splits, Tensor(d!) part_out, Tensor(e!) part_lse) -> ()", _paged_decode_step)


def reshape_and_cache_op() -> engine.Op:
    return _define(
        "reshape_and_cache",
        "(Tensor key, Tensor value, Tensor(a!) key_cache, Tensor(b!) value_cache, Tensor slot_mapping, "
        "str kv_cache_dtype, Tensor k_scale, Tensor v_scale) -> ()", _reshape_and_cache)


def paged_attention_decode_op() -> engine.Op:
    return _define(
        "paged_attention_decode",
        "(Tensor(a!) out, Tensor query, Tensor key_cache, Tensor value_cache, Tensor block_tables, "
        "Tensor seq_lens, float scale, str kv_cache_dtype, Tensor k_scale, Tensor v_scale, int num_splits, "
        "Tensor(b!) part_out, Tensor(c!) part_lse) -> ()", _paged_attention_decode)


def fused_walk_op(head_dim: int, splits: int) -> engine.Op:
    """`hk::paged_decode_fused_d{D}_s{S}` (python/hk/ops/paged.py:544-547, 706-708): the walk on
    engine views; with one split it writes the answer, with more the partials."""
    if head_dim not in paged.DECODE_HEAD_DIMS:
        raise ValueError(f"hk.ops.paged: no walk for head_dim {head_dim} (have {paged.DECODE_HEAD_DIMS})")

    def impl(q, k_cache, v_cache, block_table, seq_lens, out, o_part, ml_part):
        paged.even_heads(q, "q")
        paged.even_heads(out, "out")
        reqs, hkv, g, d = q.shape
        hq = hkv * g
        q3 = q.as_strided((reqs, hq, d), (q.stride(0), paged._row_stride(q), 1))
        o3 = out.as_strided((reqs, hq, d), (out.stride(0), paged._row_stride(out), 1))
        if k_cache.dtype not in paged.ACT_DTYPES:
            # the reference's schema has no room for scales: an fp8 cache goes through the flat op
            raise TypeError(f"hk::paged_decode_fused_d{head_dim}_s{splits} reads bfloat16 or float16 caches; an "
                            f"fp8 cache ({k_cache.dtype}) needs k_scale / v_scale: use hk::paged_attention_decode")
        paged.paged_attention_decode(
            o3, q3, k_cache.transpose(1, 2), v_cache.transpose(1, 2), block_table, seq_lens[:reqs], d ** -0.5,
            "auto", None, None, num_splits=splits,
            scratch=(o_part.view(-1, hq, d), ml_part.view(-1, hq)) if splits > 1 else None, merge=False)

    return _define(f"paged_decode_fused_d{head_dim}_s{splits}",
                   "(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_table, Tensor seq_lens, "
                   "Tensor(a!) out, Tensor(b!) o_part, Tensor(c!) ml_part) -> ()", impl)


def merge_op(head_dim: int, splits: int) -> engine.Op:
    """`hk::paged_merge_d{D}_s{S}` (python/hk/ops/paged.py:482-483, 727-729)."""

    def impl(seq_lens, out, o_part, ml_part):
        reqs = out.shape[0]
        paged.merge_splits(o_part[: reqs * splits], ml_part[: reqs * splits], splits, out)

    return _define(f"paged_merge_d{head_dim}_s{splits}",
                   "(Tensor seq_lens, Tensor(a!) out, Tensor o_part, Tensor ml_part) -> ()", impl)


def prefill_op(head_dim: int, group: int) -> engine.Op:
    """`hk::paged_prefill_d{D}_g{G}(q, k_cache, v_cache, block_table, seq_lens, q_start, tiles, out!)`:
    the reference's prefill launch and argument order (tests/hk/gpu/test_paged_prefill.py:80-82;
    python/hk/ops/paged_prefill.py kernel_for) on 2-D (tokens, heads * head_dim) q / out rows and
    hk's (blocks, kv_heads, page, head_dim) caches; `tiles` from `hk_dsl_b200.ops.paged.work_list`."""

    def impl(q, k_cache, v_cache, block_table, seq_lens, q_start, tiles, out):
        n = q.shape[0]
        hq = k_cache.shape[1] * group
        for name, t in (("q", q), ("out", out)):
            if t.dim() != 2 or t.shape[1] != hq * head_dim or t.stride(1) != 1:
                raise ValueError(f"hk::paged_prefill_d{head_dim}_g{group}: {name} is {tuple(t.shape)} strides "
                                 f"{tuple(t.stride())}; (tokens, {hq * head_dim}) rows with contiguous columns needed")
        paged.paged_prefill(out.as_strided((n, hq, head_dim), (out.stride(0), head_dim, 1)),
                            q.as_strided((n, hq, head_dim), (q.stride(0), head_dim, 1)), k_cache.transpose(1, 2),
                            v_cache.transpose(1, 2), block_table, seq_lens, q_start, tiles, head_dim ** -0.5)

    return _define(f"paged_prefill_d{head_dim}_g{group}",
                   "(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_table, Tensor seq_lens, Tensor q_start, "
                   "Tensor tiles, Tensor(a!) out) -> ()", impl)


def launcher(kind: str, head_dim: int, splits: int) -> engine.Op:
    """The decode launches by kind, as python/hk/integration/vllm_backend.py:154-163 asks for
    them: "walk" or "merge"."""
    return fused_walk_op(head_dim, splits) if kind == "walk" else merge_op(head_dim, splits)
