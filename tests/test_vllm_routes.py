"""The in-place route's predicates and fallback accounting, and the backend's constructor
refusals -- host logic on CPU tensors, the engine replaced by stubs with vLLM's signatures
(tests/hk/ir/test_vllm_prefill_route.py and tests/hk/gpu/test_paged_decode.py:329-424 of the
reference do the same: a stub that records or raises if the call falls back)."""

import inspect

import pytest
import torch

from hk_dsl_b200.integration import engine, switches, vllm_backend, vllm_prefill


def _stub_unified(q, k, v, out, cu_seqlens_q, max_seqlen_q, seqused_k, max_seqlen_k, softmax_scale, causal,
                  window_size, block_table, softcap, q_descale, k_descale, v_descale, alibi_slopes=None,
                  output_scale=None, qq_bias=None, sinks=None, new_feature=None):
    _stub_unified.calls += 1
    return "engine"


_stub_unified.calls = 0


def _args(reqs=3, hq=8, hkv=2, d=128, page=16, blocks=12, dtype=torch.bfloat16, **over):
    k = torch.zeros(blocks, page, hkv, d, dtype=dtype)
    a = dict(q=torch.zeros(reqs, hq, d, dtype=torch.bfloat16), k=k, v=k.clone(),
             out=torch.zeros(reqs, hq, d, dtype=torch.bfloat16),
             cu_seqlens_q=torch.arange(reqs + 1, dtype=torch.int32), max_seqlen_q=1,
             seqused_k=torch.ones(reqs, dtype=torch.int32), max_seqlen_k=64, softmax_scale=d ** -0.5, causal=True,
             window_size=(-1, -1), block_table=torch.zeros(reqs, 4, dtype=torch.int32), softcap=0.0,
             q_descale=None, k_descale=None, v_descale=None)
    a.update(over)
    return a


@pytest.fixture
def on_b200(monkeypatch):
    monkeypatch.setenv("HK_ARCH", "sm_100")
    monkeypatch.setattr(vllm_prefill, "_ORIG_U", _stub_unified)
    monkeypatch.setattr(vllm_prefill, "_U_SIG", inspect.signature(_stub_unified))
    monkeypatch.setattr(vllm_prefill, "DECODE", True)
    vllm_prefill.PATCH.reset()
    _stub_unified.calls = 0


def test_a_plain_decode_call_is_taken(on_b200):
    assert vllm_prefill.d_why_not(_args()) == ""
    assert vllm_prefill.d_why_not(_args(page=48)) == ""
    fp8 = _args(dtype=torch.float8_e4m3fn, k_descale=torch.ones(1), v_descale=torch.ones(1))
    assert vllm_prefill.d_why_not(fp8) == ""


@pytest.mark.parametrize("over,word", [
    (dict(max_seqlen_q=7), "not decode-only"),
    (dict(softcap=30.0), "softcap set"),
    (dict(window_size=(127, 0)), "window_size set"),
    (dict(alibi_slopes=torch.zeros(8)), "alibi_slopes set"),
    (dict(sinks=torch.zeros(8)), "sinks set"),
    (dict(q_descale=torch.ones(1)), "q_descale set"),
    (dict(new_feature=3), "new_feature set (an argument hk does not know)"),
    (dict(q=torch.zeros(3, 8, 128, dtype=torch.float16), out=torch.zeros(3, 8, 128, dtype=torch.float16)), "dtype"),
    (dict(q=torch.zeros(3, 8, 96, dtype=torch.bfloat16), out=torch.zeros(3, 8, 96, dtype=torch.bfloat16)), "head size"),
    (dict(block_table=torch.zeros(3, 4, dtype=torch.int64)), "metadata not contiguous int32"),
    (dict(seqused_k=torch.ones(6, dtype=torch.int32)[::2]), "metadata not contiguous int32"),
])
def test_refusal_reasons(on_b200, over, word):
    assert word in vllm_prefill.d_why_not(_args(**over))


def test_layouts(on_b200):
    assert "page size" in vllm_prefill.d_why_not(_args(page=24))
    assert "more than 16" in vllm_prefill.d_why_not(_args(hq=34, hkv=2, reqs=1))
    # K|V side by side in the last axis, head-major storage: read in place through strides
    both = torch.zeros(12, 2, 16, 256, dtype=torch.bfloat16)
    k, v = both[..., :128].transpose(1, 2), both[..., 128:].transpose(1, 2)
    assert vllm_prefill.layout_why_not(k, v) == ""
    # a padded block whose rows lose 16-byte alignment is refused
    padded = torch.zeros(12, 16, 2, 132, dtype=torch.bfloat16)[..., :128]
    assert "16-byte" in vllm_prefill.layout_why_not(padded, padded)
    assert "fp8 cache without" in vllm_prefill.d_why_not(_args(dtype=torch.float8_e4m3fn))


def test_arch_gate(monkeypatch, on_b200):
    monkeypatch.setenv("HK_ARCH", "sm_90")
    assert vllm_prefill.d_why_not(_args()) == "arch sm_90"


def test_untaken_calls_fall_back_to_the_engine_and_are_counted(on_b200):
    a = _args(softcap=30.0)
    assert vllm_prefill.unified_attention(**a) == "engine"
    assert vllm_prefill.unified_attention(*a.values()) == "engine"            # positional, as vLLM calls it
    assert _stub_unified.calls == 2
    assert vllm_prefill.PATCH.stats == {"prefill": 0, "decode": 0, "fallback": 2}


def test_switch_off_sends_everything_back(on_b200, monkeypatch):
    monkeypatch.setattr(vllm_prefill, "DECODE", False)
    assert vllm_prefill.unified_attention(**_args()) == "engine"
    assert vllm_prefill.PATCH.stats["fallback"] == 1


def test_without_an_engine_an_untaken_call_raises(on_b200, monkeypatch):
    monkeypatch.setattr(vllm_prefill, "_ORIG_U", None)
    with pytest.raises(RuntimeError, match="no engine function"):
        vllm_prefill.unified_attention(**_args(softcap=30.0))


def test_a_taken_call_never_reaches_the_engine_and_has_no_cpu_path(on_b200):
    """CPU tensors pass the predicate (it reads metadata only); the launch then refuses them:
    there is no CPU implementation to fall into."""
    with pytest.raises(RuntimeError, match="no CPU path"):
        vllm_prefill.unified_attention(**_args())
    assert _stub_unified.calls == 0


def test_prefill_calls_are_judged_by_their_own_predicate(on_b200):
    a = _args(max_seqlen_q=7)
    assert vllm_prefill.u_why_not(a) == ""
    assert "softcap set" in vllm_prefill.u_why_not(_args(max_seqlen_q=7, softcap=30.0))
    assert "not causal" in vllm_prefill.u_why_not(_args(max_seqlen_q=7, causal=False))
    fp8 = _args(max_seqlen_q=7, dtype=torch.float8_e4m3fn, k_descale=torch.ones(1), v_descale=torch.ones(1))
    assert vllm_prefill.u_why_not(fp8) == ""
    assert "fp8 cache without" in vllm_prefill.u_why_not(_args(max_seqlen_q=7, dtype=torch.float8_e4m3fn))
    assert vllm_prefill.unified_attention(**_args(max_seqlen_q=7, softcap=30.0)) == "engine"
    assert vllm_prefill.PATCH.stats == {"prefill": 0, "decode": 0, "fallback": 1}
    with pytest.raises(RuntimeError, match="no CPU path"):      # taken: the launch refuses CPU tensors
        vllm_prefill.unified_attention(**a)


def test_work_list_orders_long_tiles_first():
    from hk_dsl_b200.ops import paged

    assert paged.prefill_tile_rows(32, 8) == 64 and paged.prefill_tile_rows(8, 8) == 256
    assert paged.prefill_tile_rows(64, 8) == 32 and paged.prefill_tile_rows(6, 2) == 256
    w = paged.work_list([(0, 40), (2, 70)], 32, "cpu").tolist()
    assert sorted(w) == [[0, 0], [0, 32], [2, 0], [2, 32], [2, 64]]
    w = paged.work_list([(0, 40), (1, 33)], 32, "cpu", seq_lens=[40, 1033]).tolist()
    assert w[0] == [1, 32] and w[1] == [1, 0]                       # the tiles that see the most keys lead
    lib_rows = __import__("hk_dsl_b200.runtime.lib", fromlist=["load"]).load().hkb_prefill_tile_rows
    for hq, hkv in ((32, 8), (8, 8), (64, 8), (6, 2), (24, 8), (16, 1)):
        assert lib_rows(hq, hkv) == paged.prefill_tile_rows(hq, hkv)
    assert lib_rows(7, 2) == 0


def test_decode_switch_parsing():
    assert vllm_prefill.decode_switches("") == (True, False)
    assert vllm_prefill.decode_switches("1") == (True, True)
    assert vllm_prefill.decode_switches("0") == (False, False)
    assert vllm_prefill.decode_switches(" OFF ") == (False, False)


def _stub_chunked(query, key, value, output, kv_cache_dtype, key_cache, value_cache, block_table, query_start_loc,
                  seq_lens, max_seq_len, max_query_len, k_scale, v_scale, alibi_slopes=None, sliding_window=None,
                  sm_scale=None, output_scale=None, sinks=None, is_block_table_ptr=False, causal=True):
    return "engine"


def test_chunked_prefill_paged_decode_route(monkeypatch):
    monkeypatch.setenv("HK_ARCH", "sm_100")
    monkeypatch.setattr(vllm_prefill, "_ORIG_R", _stub_chunked)
    monkeypatch.setattr(vllm_prefill, "_R_SIG", inspect.signature(_stub_chunked))
    kc = torch.zeros(12, 16, 2, 128, dtype=torch.bfloat16)
    a = dict(query=torch.zeros(3, 8, 128, dtype=torch.bfloat16), key=None, value=None,
             output=torch.zeros(3, 8, 128, dtype=torch.bfloat16), kv_cache_dtype="auto", key_cache=kc,
             value_cache=kc.clone(), block_table=torch.zeros(3, 4, dtype=torch.int32),
             query_start_loc=torch.arange(4, dtype=torch.int32), seq_lens=torch.ones(3, dtype=torch.int32),
             max_seq_len=64, max_query_len=1, k_scale=torch.ones(1), v_scale=torch.ones(1))
    monkeypatch.setattr(vllm_prefill, "ROCM_DECODE", False)
    assert vllm_prefill.rd_why_not(a) == "HK_VLLM_ROCM_DECODE not set"
    assert vllm_prefill.chunked_prefill_paged_decode(**a) == "engine"
    monkeypatch.setattr(vllm_prefill, "ROCM_DECODE", True)
    assert vllm_prefill.rd_why_not(a) == ""
    assert "sliding_window set" in vllm_prefill.rd_why_not(dict(a, sliding_window=128))
    # ROCM_ATTN's own pair -- K (blocks, kv_heads, head_dim / 8, page, 8), V (blocks, kv_heads, head_dim, page) -- is
    # read in place; anything that only looks like it is named
    k5, v4 = torch.zeros(12, 2, 16, 16, 8, dtype=torch.bfloat16), torch.zeros(12, 2, 128, 16, dtype=torch.bfloat16)
    assert vllm_prefill.rd_why_not(dict(a, key_cache=k5, value_cache=v4)) == ""
    assert "beside K" in vllm_prefill.rd_why_not(dict(a, key_cache=k5))
    assert "x = 8" in vllm_prefill.rd_why_not(dict(a, key_cache=torch.zeros(12, 2, 8, 16, 16, dtype=torch.bfloat16),
                                                   value_cache=v4))
    assert "not contiguous" in vllm_prefill.rd_why_not(dict(a, key_cache=k5.transpose(2, 3).contiguous().transpose(2, 3),
                                                            value_cache=v4))
    assert "16-bit" in vllm_prefill.rd_why_not(dict(a, key_cache=k5.to(torch.float8_e4m3fn),
                                                    value_cache=v4.to(torch.float8_e4m3fn)))
    assert "under" in vllm_prefill.rd_why_not(dict(a, key_cache=k5.half(), value_cache=v4.half()))
    assert "not decode-only" in vllm_prefill.rd_why_not(dict(a, max_query_len=5))


def test_rebind_by_identity():
    import sys
    import types

    from hk_dsl_b200.integration._common import rebind

    def old():
        return 0

    def new():
        return 1

    m1, m2 = types.ModuleType("fakeengine.a"), types.ModuleType("fakeengine.b")
    m1.fn, m1.other = old, new
    m2.alias = old
    sys.modules["fakeengine.a"], sys.modules["fakeengine.b"] = m1, m2
    try:
        hits = rebind(("fakeengine",), old, new)
        assert sorted(hits) == ["fakeengine.a.fn", "fakeengine.b.alias"] and m1.fn is new and m2.alias is new
    finally:
        del sys.modules["fakeengine.a"], sys.modules["fakeengine.b"]


# ------------------------------------------------------------------------------ backend

def _impl(**over):
    kw = dict(num_heads=32, head_size=128, scale=128 ** -0.5, num_kv_heads=8, alibi_slopes=None, sliding_window=None,
              kv_cache_dtype="auto")
    kw.update(over)
    return vllm_backend.HKAttentionImplCore(**kw)


def test_backend_refuses_what_it_does_not_implement():
    _impl()
    _impl(kv_cache_dtype="fp8")
    _impl(kv_cache_dtype="fp8_e4m3")
    for bad in (dict(alibi_slopes=[0.1] * 32), dict(sliding_window=4096), dict(sinks=torch.zeros(32))):
        with pytest.raises(NotImplementedError, match="does not implement"):
            _impl(**bad)
    with pytest.raises(NotImplementedError, match="logits_soft_cap"):
        _impl(logits_soft_cap=30.0)
    with pytest.raises(NotImplementedError, match="fp8_e5m2"):
        _impl(kv_cache_dtype="fp8_e5m2")
    with pytest.raises(ValueError, match="head_size"):
        _impl(head_size=96)
    with pytest.raises(ValueError, match="GQA group"):
        _impl(num_heads=34, num_kv_heads=1)


def test_backend_cache_shape_and_views():
    assert vllm_backend.get_kv_cache_shape(100, 16, 8, 128) == (2, 100, 8, 16, 128)
    with pytest.raises(ValueError):
        vllm_backend.get_kv_cache_shape(100, 20, 8, 128)
    impl = _impl()
    five = torch.zeros(2, 10, 8, 16, 128, dtype=torch.bfloat16)
    k, v = impl._kv(five)
    assert k.shape == (10, 8, 16, 128) and v.data_ptr() != k.data_ptr()
    side = torch.zeros(10, 8, 16, 256, dtype=torch.bfloat16)
    k, v = impl._kv(side)
    assert k.shape == (10, 8, 16, 128) and v.storage_offset() - k.storage_offset() == 128


def test_backend_plan_depends_on_batch_only_and_is_a_power_of_two(monkeypatch):
    monkeypatch.delenv("HK_SPLITS", raising=False)
    impl = _impl()
    plans = [impl._plan(n) for n in (1, 4, 8, 16, 32, 64, 128, 256)]
    assert all(p & (p - 1) == 0 for p in plans) and plans == sorted(plans, reverse=True)
    assert impl._plan(64) == impl._plan(64)


def test_backend_prefill_batches_raise_and_checks_metadata():
    impl = _impl()
    md = vllm_backend.metadata(4, torch.zeros(4, dtype=torch.int64), torch.zeros(2, 8, dtype=torch.int32),
                               torch.ones(2, dtype=torch.int32), max_query_len=3)
    kv = torch.zeros(2, 4, 8, 16, 128, dtype=torch.bfloat16)
    md.query_start_loc = torch.tensor([0, 3, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):          # a prefill batch is taken; CPU tensors are not
        impl.forward(None, torch.zeros(4, 32 * 128, dtype=torch.bfloat16), None, None, kv, md,
                     output=torch.zeros(4, 32 * 128, dtype=torch.bfloat16))

    with pytest.raises(NotImplementedError, match="output quant"):
        impl.forward(None, None, None, None, kv, md, output=None, output_scale=torch.ones(1))
    with pytest.raises(TypeError, match="int32"):
        impl._check(torch.zeros(2, 8, dtype=torch.int64), torch.ones(2, dtype=torch.int32))
    with pytest.raises(ValueError, match="pages of 16 tokens but block_table"):
        impl._check(torch.zeros(2, 2, dtype=torch.int32), torch.tensor([10, 100], dtype=torch.int32))
    out = torch.ones(3, 8)
    assert impl.forward(None, None, None, None, kv, None, output=out) is out and (out == 0).all()   # profiling run


def test_register_with_an_installed_vllm_resolves_to_our_backend():
    """With vLLM importable, `register()` puts the backend under the chosen enum member and the
    classes it builds have vLLM's bases and this build's cache shape."""
    pytest.importorskip("vllm")
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum
    except Exception as e:  # noqa: BLE001 -- another vLLM layout: the plugin would report the route off
        pytest.skip(f"this vLLM has no v1 backend registry: {e}")
    msg = vllm_backend.register()
    assert "registered over CUSTOM" in msg
    backend = vllm_backend.HKAttentionBackend
    assert AttentionBackendEnum.CUSTOM.get_path().endswith("vllm_backend.HKAttentionBackend")
    assert backend.get_name() == "CUSTOM" and backend.get_impl_cls() is vllm_backend.HKAttentionImpl
    assert backend.get_kv_cache_shape(10, 16, 8, 128) == (2, 10, 8, 16, 128)
    assert issubclass(vllm_backend.HKAttentionImpl, vllm_backend.HKAttentionImplCore)
    with pytest.raises(RuntimeError, match="no AttentionBackendEnum"):
        vllm_backend.register("NOT_A_BACKEND")
    vllm_backend.register()     # idempotent, and restores the slot name


def test_shadow_compare_counts_rows_in_bf16_ulps():
    """The in-situ check's arithmetic (the reference's, python/hk/integration/vllm_prefill.py:258-275):
    a row's error in ulps of bf16 at the reference row's largest value; more than 4 is counted."""
    stats = {"calls": 0, "rows": 0, "worst_ulps": 0.0, "worst_call": -1, "over_4": 0}
    ref = torch.zeros(3, 2, 8)
    ref[..., 0] = 1.5                                  # largest value 1.5: one bf16 ulp there is 2^-7
    ours = ref.clone()
    assert vllm_prefill.shadow_compare(ours, ref, stats) == 0.0
    ours[1, 0, 3] = 2 * 2.0 ** -7
    assert vllm_prefill.shadow_compare(ours, ref, stats) == pytest.approx(2.0)
    assert stats == {"calls": 2, "rows": 6, "worst_ulps": pytest.approx(2.0), "worst_call": 2, "over_4": 0}
    ours[2, 1, 5] = 9 * 2.0 ** -7
    assert vllm_prefill.shadow_compare(ours, ref, stats) == pytest.approx(9.0)
    assert stats["over_4"] == 1 and stats["worst_call"] == 3
    assert vllm_prefill.shadow_compare(ours[:0], ref[:0], stats) == 0.0 and stats["calls"] == 4
