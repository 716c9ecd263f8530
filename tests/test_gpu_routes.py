"""The engine-facing surfaces on a GPU: the in-place route stand-ins called as vLLM calls them,
the backend's forward (cache write + decode) on plain tensors, the torch custom ops, the
CUDA-graph contract, and guard bands around everything the kernels write.

Reference cases: tests/hk/gpu/test_paged_decode.py:329-424 (stand-ins with a stub that raises
if the call falls back; fallback counted), tests/hk/gpu/test_engine.py:35-75 (a host sync in a
"safe" patch raises under capture, naming it), python/hk/ops/paged.py:897-900 (guard pages
either side of the outputs stay untouched; here canaries checked on the host, no faulting
allocator).
"""

import inspect

import pytest
import torch

from oracle import paged_oracle as orc

pytestmark = pytest.mark.gpu


def _case(lens, hkv=2, group=4, d=128, page=16, seed=0, fp8=False):
    g = torch.Generator().manual_seed(seed)
    pages = [max(1, -(-n // page)) for n in lens]
    nb = sum(pages) + 3
    k = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16)
    v = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nb, generator=g)
    table = torch.zeros(len(lens), max(pages), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages):
        table[i, :n] = perm[at:at + n].to(torch.int32)
        at += n
    q = torch.randn(len(lens), hkv * group, d, generator=g).to(torch.bfloat16)
    return q, k, v, table, torch.tensor(lens, dtype=torch.int32)


def _stub_raises(q, k, v, out, cu_seqlens_q, max_seqlen_q, seqused_k, max_seqlen_k, softmax_scale, causal,
                 window_size, block_table, softcap, q_descale, k_descale, v_descale, alibi_slopes=None,
                 output_scale=None, qq_bias=None, sinks=None):
    raise AssertionError("the call fell back to the engine's kernel")


@pytest.fixture
def route(monkeypatch):
    from hk_dsl_b200.integration import vllm_prefill

    monkeypatch.setattr(vllm_prefill, "_ORIG_U", _stub_raises)
    monkeypatch.setattr(vllm_prefill, "_U_SIG", inspect.signature(_stub_raises))
    monkeypatch.setattr(vllm_prefill, "DECODE", True)
    vllm_prefill.PATCH.reset()
    return vllm_prefill


@pytest.mark.parametrize("order", ["nhd", "hnd", "side_by_side"])
@pytest.mark.parametrize("group", [4, 8])
def test_unified_attention_stand_in_as_vllm_calls_it(route, order, group):
    lens = [1, 33, 1000, 2063]
    q, k, v, table, lens_t = _case(lens, group=group, seed=group)
    want = orc.paged_decode_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t)
    if order == "nhd":
        kc, vc = k.transpose(1, 2).contiguous().cuda(), v.transpose(1, 2).contiguous().cuda()
    elif order == "hnd":
        kc, vc = k.cuda().transpose(1, 2), v.cuda().transpose(1, 2)
    else:
        both = torch.cat([k, v], dim=-1).cuda()
        kc, vc = both[..., :128].transpose(1, 2), both[..., 128:].transpose(1, 2)
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
    n = len(lens)
    route.unified_attention(q.cuda(), kc, vc, out, torch.arange(n + 1, dtype=torch.int32, device="cuda"), 1,
                            lens_t.cuda(), max(lens), 128 ** -0.5, True, (-1, -1), table.cuda(), 0.0, None, None,
                            None)
    orc.check(out, want)
    assert route.PATCH.stats == {"prefill": 0, "decode": 1, "fallback": 0}


def _stub_chunked_raises(query, key, value, output, kv_cache_dtype, key_cache, value_cache, block_table,
                         query_start_loc, seq_lens, max_seq_len, max_query_len, k_scale, v_scale, alibi_slopes=None,
                         sliding_window=None, sm_scale=None, output_scale=None, sinks=None, is_block_table_ptr=False,
                         causal=True):
    raise AssertionError("the call fell back to the engine's kernel")


@pytest.mark.parametrize("page", [16, 32])
def test_chunked_prefill_paged_decode_stand_in_on_x_split_caches(route, page, monkeypatch):
    """ROCM_ATTN's own cache pair, read in place (python/hk/integration/vllm_prefill.py:1332-1356)."""
    from hk_dsl_b200.ops import paged

    monkeypatch.setattr(route, "_ORIG_R", _stub_chunked_raises)
    monkeypatch.setattr(route, "_R_SIG", inspect.signature(_stub_chunked_raises))
    monkeypatch.setattr(route, "ROCM_DECODE", True)
    lens = [1, 33, 1000, 2063]
    q, k, v, table, lens_t = _case(lens, group=4, page=page, seed=page)
    want = orc.paged_decode_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t)
    k5, v4 = paged.x_split_caches(k.transpose(1, 2).cuda(), v.transpose(1, 2).cuda())
    assert k5.shape == (k.shape[0], 2, 16, page, 8) and v4.shape == (k.shape[0], 2, 128, page)
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
    n = len(lens)
    route.chunked_prefill_paged_decode(q.cuda(), None, None, out, "auto", k5, v4, table.cuda(),
                                       torch.arange(n + 1, dtype=torch.int32, device="cuda"), lens_t.cuda(),
                                       max(lens), 1, None, None, sm_scale=128 ** -0.5)
    orc.check(out, want)
    assert route.PATCH.stats == {"prefill": 0, "decode": 1, "fallback": 0}


def test_the_stand_in_under_graph_capture_and_padding(route):
    """Captured once, replayed with other lengths; requests without a query write nothing."""
    lens = [500, 33, 0, 0]
    q, k, v, table, lens_t = _case([500, 33, 700, 64], seed=5)
    lens_dev = torch.tensor(lens, dtype=torch.int32, device="cuda")
    q_start = torch.tensor([0, 1, 2, 2, 2], dtype=torch.int32, device="cuda")
    kc, vc, tb, qd = k.cuda().transpose(1, 2), v.cuda().transpose(1, 2), table.cuda(), q.cuda()
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)

    def call():
        route._GUARDED_U(qd, kc, vc, out, q_start, 1, lens_dev, 2048, 128 ** -0.5, True, (-1, -1), tb, 0.0, None,
                         None, None)

    call()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call()
    assert route.PATCH.captured["decode"] == 1
    out.fill_(7.0)
    lens_dev.copy_(torch.tensor([64, 500, 0, 0], dtype=torch.int32))
    graph.replay()
    torch.cuda.synchronize()
    want = orc.paged_decode_ref(q, k.transpose(1, 2), v.transpose(1, 2), table,
                                torch.tensor([64, 500, 0, 0], dtype=torch.int32), None, None, None, q_start.cpu())
    orc.check(out[:2], want[:2])
    assert (out[2:] == 7.0).all()


def test_a_host_sync_inside_a_safe_patch_raises_under_capture_naming_it():
    from hk_dsl_b200.integration import engine

    p = engine.Patch("t_sync", ("a",))
    x = torch.ones(4, device="cuda")
    f = p.guard(lambda t: t.sum().item())
    assert f(x) == 4.0
    graph = torch.cuda.CUDAGraph()
    with pytest.raises(engine.GraphCaptureError, match="t_sync"):
        with torch.cuda.graph(graph):
            f(x)
    torch.cuda.synchronize()
    never = engine.Patch("t_never_gpu", ("a",), graph="never", why="plans on lengths read back")
    h = never.guard(lambda t: t + 1)
    with pytest.raises(engine.GraphCaptureError, match="plans on lengths read back"):
        with torch.cuda.graph(torch.cuda.CUDAGraph()):
            h(x)
    torch.cuda.synchronize()


@pytest.mark.parametrize("d", [128, 64, 256])
@pytest.mark.parametrize("kv_cache_dtype", ["auto", "fp8"])
@pytest.mark.parametrize("layout", ["five", "side_by_side"])
def test_backend_forward_writes_the_cache_then_decodes(kv_cache_dtype, layout, d, monkeypatch):
    """One decode step as the engine drives it: new K/V rows scattered by slot, then attention
    over the updated cache; and the same step replayed from a CUDA graph. Head sizes 64, 128 and 256,
    16-bit and fp8 caches."""
    from hk_dsl_b200.integration import vllm_backend

    monkeypatch.delenv("HK_SPLITS", raising=False)
    hq, hkv, page = 32, 8, 16
    lens = [17, 700, 1, 2063, 256]
    n = len(lens)
    q, k, v, table, lens_t = _case(lens, hkv=hkv, group=4, d=d, seed=21)
    g = torch.Generator().manual_seed(99)
    key = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    value = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    slots = torch.tensor([int(table[i, (s - 1) // page]) * page + (s - 1) % page for i, s in enumerate(lens)])
    fp8 = kv_cache_dtype == "fp8"
    ks, vs = torch.tensor([0.02]), torch.tensor([0.017])

    # the oracle's cache after the write
    want_k, want_v = k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous()
    if fp8:
        want_k, want_v = orc.quantize_fp8(want_k, ks), orc.quantize_fp8(want_v, vs)
    orc.reshape_and_cache_ref(key, value, want_k, want_v, slots, kv_cache_dtype, ks, vs)
    want = orc.paged_decode_ref(q, want_k, want_v, table, lens_t, None, ks if fp8 else None, vs if fp8 else None)

    nb = k.shape[0]
    cdt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    k0 = orc.quantize_fp8(k, ks) if fp8 else k
    v0 = orc.quantize_fp8(v, vs) if fp8 else v
    if layout == "five":
        kv = torch.zeros(2, nb, hkv, page, d, dtype=torch.bfloat16).to(cdt).cuda()
        kv[0].view(torch.uint8 if fp8 else cdt).copy_(k0.view(torch.uint8 if fp8 else cdt))
        kv[1].view(torch.uint8 if fp8 else cdt).copy_(v0.view(torch.uint8 if fp8 else cdt))
    else:
        kv = torch.cat([k0.view(torch.uint8) if fp8 else k0, v0.view(torch.uint8) if fp8 else v0], dim=-1).cuda()
        if fp8:
            kv = kv.view(cdt)
    impl = vllm_backend.HKAttentionImplCore(hq, d, d ** -0.5, hkv, None, None, kv_cache_dtype)
    layer = type("Layer", (), {})()
    layer._k_scale, layer._v_scale = ks.cuda(), vs.cuda()
    md = vllm_backend.metadata(n, slots.cuda(), table.cuda(), lens_t.cuda(), max_query_len=1)
    query = q.cuda().view(n, hq * d)
    out = torch.full((n, hq * d), 7.0, device="cuda", dtype=torch.bfloat16)
    vllm_backend.PATCH.reset()
    key_d, value_d = key.cuda(), value.cuda()
    impl.forward(layer, query, key_d, value_d, kv, md, output=out)
    torch.cuda.synchronize()
    orc.check(out.view(n, hq, d), want)
    orc.check_baseline(out.view(n, hq, d), want)
    kc, vc = impl._kv(kv)
    assert torch.equal(kc.transpose(1, 2).contiguous().view(torch.uint8).cpu(), want_k.view(torch.uint8))
    assert torch.equal(vc.transpose(1, 2).contiguous().view(torch.uint8).cpu(), want_v.view(torch.uint8))
    assert vllm_backend.PATCH.stats["decode"] == 1
    # the whole step captured and replayed: same bits
    first = out.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        impl.forward(layer, query, key_d, value_d, kv, md, output=out)
    out.fill_(0)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), first.view(torch.int16))


def test_torch_ops_surface():
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import torch_ext

    lens = [1, 31, 32, 33, 200, 1000]
    q, k, v, table, lens_t = _case(lens, hkv=8, group=4, seed=31)
    want = orc.paged_decode_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t)
    n, hq, d = q.shape
    qd, kd, vd, td, ld = q.cuda(), k.cuda(), v.cuda(), table.cuda(), lens_t.cuda()
    one = torch.ones(1, device="cuda")

    torch_ext.paged_attention_decode_op()
    torch_ext.reshape_and_cache_op()
    out = torch.empty_like(qd)
    po, pl = paged.split_scratch(n, hq, d, 4, "cuda")
    r = torch.ops.hk.paged_attention_decode(out, qd, kd.transpose(1, 2), vd.transpose(1, 2), td, ld, d ** -0.5, "auto",
                                            one, one, 4, po, pl)
    assert r is None
    orc.check(out, want)

    # the reference's per-(head_dim, splits) names, registered on demand
    splits = 4
    walk, merge = torch_ext.launcher("walk", d, splits), torch_ext.launcher("merge", d, splits)
    assert walk.name == "hk::paged_decode_fused_d128_s4" and merge.name == "hk::paged_merge_d128_s4"
    o_part, ml_part = paged.fused_scratch(n * splits, 8, d, "cuda", group=4)
    out4 = torch.empty(n, 8, 4, d, device="cuda", dtype=torch.bfloat16)
    walk(qd.view(n, 8, 4, d), kd, vd, td, ld, out4, o_part, ml_part)
    merge(ld, out4, o_part, ml_part)
    orc.check(out4.view(n, hq, d), want)
    out4.zero_()
    torch.ops.hk.paged_decode_fused_d128_s4(qd.view(n, 8, 4, d), kd, vd, td, ld, out4, o_part, ml_part)
    torch.ops.hk.paged_merge_d128_s4(ld, out4, o_part, ml_part)
    orc.check(out4.view(n, hq, d), want)

    # the same names on a float16 cache (a model served in float16) ...
    out16 = torch.empty(n, 8, 4, d, device="cuda", dtype=torch.float16)
    walk(qd.half().view(n, 8, 4, d), kd.half(), vd.half(), td, ld, out16, o_part, ml_part)
    merge(ld, out16, o_part, ml_part)
    want16 = orc.paged_decode_ref(q.half(), k.half().transpose(1, 2), v.half().transpose(1, 2), table, lens_t)
    orc.check(out16.view(n, hq, d), want16)
    # ... an fp8 cache is refused by name (the reference's schema has no scales); the flat op takes it
    k8 = orc.quantize_fp8(k, torch.tensor([0.02])).cuda()
    v8 = orc.quantize_fp8(v, torch.tensor([0.02])).cuda()
    with pytest.raises(TypeError, match="hk::paged_attention_decode"):
        walk(qd.view(n, 8, 4, d), k8, v8, td, ld, out4, o_part, ml_part)
    s8 = torch.full((1,), 0.02, device="cuda")
    torch.ops.hk.paged_attention_decode(out, qd, k8.transpose(1, 2), v8.transpose(1, 2), td, ld, d ** -0.5, "fp8", s8, s8,
                                        4, po, pl)
    orc.check(out, orc.paged_decode_ref(q, k8.cpu().transpose(1, 2), v8.cpu().transpose(1, 2), table, lens_t, None,
                                        s8.cpu(), s8.cpu()))
    # a view whose heads are not evenly strided is refused, not read at the wrong elements
    with pytest.raises(ValueError, match="evenly strided"):
        walk(torch.zeros(n, 8, d, 4, device="cuda", dtype=torch.bfloat16).transpose(2, 3), kd, vd, td, ld, out4, o_part, ml_part)

    # the cache write as an op
    key = torch.randn(n, 8, d, device="cuda").to(torch.bfloat16)
    slots = torch.arange(n, device="cuda") * 16
    kc2, vc2 = torch.zeros_like(kd), torch.zeros_like(vd)
    torch.ops.hk.reshape_and_cache(key, key, kc2.transpose(1, 2), vc2.transpose(1, 2), slots, "auto", one, one)
    assert torch.equal(kc2[torch.arange(n), :, 0], key)


@pytest.mark.parametrize("group", [4, 8])
@pytest.mark.parametrize("splits", [1, 8])
def test_guard_bands_around_everything_written(group, splits):
    """Output, split scratch and cache sit inside larger buffers filled with a canary; after
    the calls every margin byte is untouched. The cache has no spare blocks, so the last page
    is the cache's end (tests/hk/gpu/test_fenced.py:424-533 of the reference uses a faulting
    allocator for this; a fault is never provoked here)."""
    from hk_dsl_b200.ops import paged

    lens = [1, 15, 16, 17, 1000, 33]
    g = torch.Generator().manual_seed(77)
    hkv, d, page = 2, 128, 16
    pages = [-(-n // page) for n in lens]
    nb = sum(pages)                                    # no spare blocks
    n, hq = len(lens), hkv * group
    CAN = 0x5A

    def banded(numel, dtype, margin=4096):
        raw = torch.full((numel * dtype.itemsize + 2 * margin,), CAN, dtype=torch.uint8, device="cuda")
        return raw, raw[margin:margin + numel * dtype.itemsize].view(dtype)

    raw_k, kf = banded(nb * hkv * page * d, torch.bfloat16)
    raw_v, vf = banded(nb * hkv * page * d, torch.bfloat16)
    kc, vc = kf.view(nb, hkv, page, d), vf.view(nb, hkv, page, d)
    kc.copy_(torch.randn(kc.shape, generator=g).to(torch.bfloat16))
    vc.copy_(torch.randn(vc.shape, generator=g).to(torch.bfloat16))
    table = torch.zeros(n, max(pages), dtype=torch.int32)
    perm = torch.randperm(nb, generator=g)
    at = 0
    for i, p in enumerate(pages):
        table[i, :p] = perm[at:at + p].to(torch.int32)
        at += p
    raw_o, of = banded(n * hq * d, torch.bfloat16)
    raw_po, pof = banded(n * splits * hq * d, torch.float32)
    raw_pl, plf = banded(n * splits * hq, torch.float32)
    out = of.view(n, hq, d)
    scratch = (pof.view(n * splits, hq, d), plf.view(n * splits, hq))
    q = torch.randn(n, hq, d, generator=g).to(torch.bfloat16).cuda()
    key = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16).cuda()
    slots = torch.tensor([int(table[i, (s - 1) // page]) * page + (s - 1) % page for i, s in enumerate(lens)]).cuda()
    lens_t = torch.tensor(lens, dtype=torch.int32)
    for _ in range(3):
        paged.reshape_and_cache(key, key, kc.transpose(1, 2), vc.transpose(1, 2), slots)
        paged.paged_attention_decode(out, q, kc.transpose(1, 2), vc.transpose(1, 2), table.cuda(), lens_t.cuda(),
                                     d ** -0.5, num_splits=splits, scratch=scratch if splits > 1 else None)
    torch.cuda.synchronize()
    for raw in (raw_k, raw_v, raw_o, raw_po, raw_pl):
        assert (raw[:4096] == CAN).all() and (raw[-4096:] == CAN).all()
    want = orc.paged_decode_ref(q.cpu(), kc.cpu().transpose(1, 2), vc.cpu().transpose(1, 2), table, lens_t)
    orc.check(out, want)


def _mixed_case(reqs, hkv=8, group=4, d=128, page=16, seed=0):
    """reqs: [(ctx, q_len)]; the whole sequence of each is in the cache, the last q_len tokens query."""
    g = torch.Generator().manual_seed(seed)
    seq = [c + n for c, n in reqs]
    pages = [max(1, -(-s // page)) for s in seq]
    nb = sum(pages) + 3
    k = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16)
    v = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nb, generator=g)
    table = torch.zeros(len(reqs), max(pages), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages):
        table[i, :n] = perm[at:at + n].to(torch.int32)
        at += n
    n_tok = sum(n for _, n in reqs)
    q = torch.randn(n_tok, hkv * group, d, generator=g).to(torch.bfloat16)
    starts = [0]
    for _, n in reqs:
        starts.append(starts[-1] + n)
    return q, k, v, table, torch.tensor(seq, dtype=torch.int32), torch.tensor(starts, dtype=torch.int32)


def test_backend_forward_on_a_batch_with_prefill_in_it():
    """Decodes first, then a chunk with a cached prefix and a fresh prompt: the step's K/V rows are
    written by slot, then one prefill launch serves every request (a decode is a one-row tile)."""
    from hk_dsl_b200.integration import vllm_backend

    hq, hkv, d, page = 32, 8, 128, 16
    reqs = [(700, 1), (33, 1), (1000, 77), (0, 300)]
    q, k, v, table, lens, q_start = _mixed_case(reqs, hkv=hkv, seed=41)
    n = q.shape[0]
    g = torch.Generator().manual_seed(43)
    key = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    value = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    slots = []
    for i, (ctx, ql) in enumerate(reqs):
        pos = torch.arange(ctx, ctx + ql)
        slots.append(table[i, pos // page].long() * page + pos % page)
    slots = torch.cat(slots)
    want_k, want_v = k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous()
    orc.reshape_and_cache_ref(key, value, want_k, want_v, slots)
    want = orc.paged_prefill_ref(q, want_k, want_v, table, lens, q_start)

    kv = torch.stack([k, v]).cuda()
    impl = vllm_backend.HKAttentionImplCore(hq, d, d ** -0.5, hkv, None, None, "auto")
    md = vllm_backend.metadata(n, slots.cuda(), table.cuda(), lens.cuda(), max_query_len=300,
                               query_start_loc=q_start.cuda())
    out = torch.full((n, hq * d), 7.0, device="cuda", dtype=torch.bfloat16)
    vllm_backend.PATCH.reset()
    impl.forward(None, q.cuda().view(n, hq * d), key.cuda(), value.cuda(), kv, md, output=out)
    torch.cuda.synchronize()
    orc.check(out.view(n, hq, d), want)
    assert vllm_backend.PATCH.stats == {"decode": 0, "prefill": 1}
    # a prefill step is never captured: it reads query lengths on the host
    from hk_dsl_b200.integration import engine
    qd = q.cuda().view(n, hq * d)
    with pytest.raises(engine.GraphCaptureError, match="prefill"):
        with torch.cuda.graph(torch.cuda.CUDAGraph()):
            impl.forward(None, qd, None, None, kv, md, output=out)
    torch.cuda.synchronize()


def test_unified_attention_stand_in_takes_a_batch_with_prefill(route):
    reqs = [(64, 100), (300, 1), (0, 200)]
    q, k, v, table, lens, q_start = _mixed_case(reqs, hkv=2, group=8, seed=44)
    want = orc.paged_prefill_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens, q_start)
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
    route.unified_attention(q.cuda(), k.cuda().transpose(1, 2), v.cuda().transpose(1, 2), out, q_start.cuda(), 200,
                            lens.cuda(), 300, 128 ** -0.5, True, (-1, -1), table.cuda(), 0.0, None, None, None)
    torch.cuda.synchronize()
    orc.check(out, want)
    assert route.PATCH.stats == {"prefill": 1, "decode": 0, "fallback": 0}


def test_prefill_torch_op():
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import torch_ext

    reqs = [(100, 90), (0, 33)]
    q, k, v, table, lens, q_start = _mixed_case(reqs, hkv=2, group=4, seed=45)
    want = orc.paged_prefill_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens, q_start)
    n, hq, d = q.shape
    op = torch_ext.prefill_op(d, 4)
    assert op.name == "hk::paged_prefill_d128_g4"
    tiles = paged.work_list([(0, 90), (1, 33)], paged.prefill_tile_rows(hq, 2), "cuda")
    out = torch.empty(n, hq * d, device="cuda", dtype=torch.bfloat16)
    torch.ops.hk.paged_prefill_d128_g4(q.cuda().view(n, hq * d), k.cuda(), v.cuda(), table.cuda(), lens.cuda(),
                                       q_start.cuda(), tiles, out)
    orc.check(out.view(n, hq, d), want)


def test_shadow_mode_runs_the_engines_kernel_beside_ours(route, monkeypatch):
    """HK_VLLM_PREFILL_SHADOW: after a taken call the engine's function runs on the same arguments
    into a scratch output and the rows are compared. The "engine" here is this build's one-split
    kernel (another code path to the same answer), then one that is wrong on purpose."""
    from hk_dsl_b200.ops import paged

    lens = [1, 33, 1000, 2063]
    q, k, v, table, lens_t = _case(lens, group=4, seed=12)
    kc, vc = k.cuda().transpose(1, 2), v.cuda().transpose(1, 2)
    n = len(lens)
    seen = []

    def engine_kernel(q, k, v, out, cu_seqlens_q, max_seqlen_q, seqused_k, max_seqlen_k, softmax_scale, causal,
                      window_size, block_table, softcap, q_descale, k_descale, v_descale, alibi_slopes=None,
                      output_scale=None, qq_bias=None, sinks=None):
        seen.append(out.data_ptr())
        paged.paged_attention_decode(out, q, k, v, block_table, seqused_k, softmax_scale, num_splits=1)
        if len(seen) > 1:
            out.add_(0.5)

    stats = {"calls": 0, "rows": 0, "worst_ulps": 0.0, "worst_call": -1, "over_4": 0}
    monkeypatch.setattr(route, "_ORIG_U", engine_kernel)
    monkeypatch.setattr(route, "SHADOW", True)
    monkeypatch.setattr(route, "SHADOW_STATS", stats)
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
    args = (q.cuda(), kc, vc, out, torch.arange(n + 1, dtype=torch.int32, device="cuda"), 1, lens_t.cuda(), max(lens),
            128 ** -0.5, True, (-1, -1), table.cuda(), 0.0, None, None, None)
    route.unified_attention(*args)
    assert seen and seen[0] != out.data_ptr(), "the engine's kernel writes a scratch output, not ours"
    assert stats["calls"] == 1 and stats["rows"] == n and stats["worst_ulps"] <= 4 and stats["over_4"] == 0
    want = orc.paged_decode_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t)
    orc.check(out, want)                      # our answer is what the caller gets
    route.unified_attention(*args)            # the second "engine" answer is off by 0.5
    assert stats["calls"] == 2 and stats["over_4"] == 1 and stats["worst_call"] == 2
    orc.check(out, want)
    assert route.PATCH.stats == {"prefill": 0, "decode": 2, "fallback": 0}
