"""Paged GQA decode attention (walk + LSE merge) against the float64 oracle, through the
C ABI. The cases are the reference's, one for one:

  tests/hk/gpu/test_paged.py        lengths 1 / PAGE-1 / PAGE+1 / 3 PAGE+7, ragged batches, scrambled
                                    tables, poison past the end, splits 1/2/4/8 and more splits than pages
  tests/hk/gpu/test_paged_fused.py  lens [1,31,32,33,200,1000] x splits, 64 and 256 splits, determinism,
                                    a padded request answers zero, graph replay over new lengths / a new table
  tests/hk/gpu/test_paged_decode.py LENS [1,15,16,33,1000,2063,4100], GQA shapes, V == 1 gives exactly 1,
                                    NaN past the end, graph padding writes nothing, strided q, 200 calls
                                    over NaN-poisoned scratch on a side stream, bad shapes refused

Tolerances: the reference's own (worst row within 4 bf16 ulps of its largest value, and
max|err| / max|ref| < 2^-6; tests/hk/gpu/_attn_ref.py:43-44) AND this build's stated bound
(max-abs <= 2e-2, mean-abs <= 2e-3), both against the float64 softmax.
"""

import pytest
import torch

from oracle import paged_oracle as orc

pytestmark = pytest.mark.gpu

LENS = [1, 15, 16, 33, 1000, 2063, 4100]


def _paged():
    from hk_dsl_b200.ops import paged
    return paged


def _case(lens, *, head_dim=128, h_kv=2, group=8, page=16, seed=0, v_ones=False, nan_tail=False, pad=0,
          strided_q=False, layout="hnd", fp8=False, spare=3):
    """The reference's case generator (tests/hk/gpu/test_paged_decode.py:40-74): a scrambled page
    table so that `i` for `table[i]` is wrong, not lucky; `pad` requests with no query after the
    real ones (a CUDA graph's padding: query_start_loc repeats, seq_lens 0)."""
    g = torch.Generator().manual_seed(seed)
    r = len(lens)
    pages = [max(1, -(-n // page)) for n in lens]
    nb = sum(pages) + spare
    k = torch.randn(nb, h_kv, page, head_dim, generator=g).to(torch.bfloat16)
    v = torch.ones_like(k) if v_ones else torch.randn(k.shape, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nb, generator=g)
    table = torch.zeros(r + pad, max(pages), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages):
        table[i, :n] = perm[at:at + n].to(torch.int32)
        at += n
    lens_t = torch.tensor(list(lens) + [0] * pad, dtype=torch.int32)
    if nan_tail:
        live = torch.zeros(nb, page, dtype=torch.bool)
        for i, s in enumerate(lens):
            for j in range(-(-s // page)):
                live[int(table[i, j]), : min(page, s - j * page)] = True
        dead = ~live[:, None, :, None]
        k, v = k.masked_fill(dead, float("nan")), v.masked_fill(dead, float("nan"))
    h = h_kv * group
    if strided_q:
        qkv = torch.randn(r + pad, (h + 2 * h_kv) * head_dim, generator=g).to(torch.bfloat16)
        q = qkv[:, : h * head_dim].view(r + pad, h, head_dim)
    else:
        q = torch.randn(r + pad, h, head_dim, generator=g).to(torch.bfloat16)
    q_start = torch.tensor(list(range(r + 1)) + [r] * pad, dtype=torch.int32)
    ks = vs = None
    if fp8:
        ks, vs = torch.tensor([0.0125]), torch.tensor([0.011])
        k, v = orc.quantize_fp8(k, ks), orc.quantize_fp8(v, vs)
    if layout == "nhd":
        k, v = k.transpose(1, 2).contiguous().transpose(1, 2), v.transpose(1, 2).contiguous().transpose(1, 2)
    return dict(q=q, k=k, v=v, table=table, lens=lens_t, q_start=q_start, ks=ks, vs=vs, group=group)


def _cuda(c):
    return {n: (t.cuda() if isinstance(t, torch.Tensor) else t) for n, t in c.items()}


def _reference(c, with_q_start=False):
    return orc.paged_decode_ref(c["q"], c["k"].transpose(1, 2), c["v"].transpose(1, 2), c["table"], c["lens"],
                                None, c["ks"], c["vs"], c["q_start"] if with_q_start else None)


def _run(c, splits=None, out=None, scratch=None, with_q_start=False):
    paged = _paged()
    g = _cuda(c) if not c["q"].is_cuda else c
    if c["q"].is_cuda is False and c["q"].stride(0) != c["q"].shape[1] * c["q"].shape[2]:
        # keep the fused-qkv striding on the device too
        base = torch.empty(c["q"].shape[0], c["q"].stride(0), dtype=torch.bfloat16, device="cuda")
        g["q"] = base[:, : c["q"].shape[1] * c["q"].shape[2]].view(c["q"].shape)
        g["q"].copy_(c["q"])
    o = torch.empty(g["q"].shape, device="cuda", dtype=torch.bfloat16) if out is None else out
    n = g["lens"].shape[0]
    paged.paged_attention_decode(
        o, g["q"], g["k"].transpose(1, 2), g["v"].transpose(1, 2), g["table"], g["lens"],
        g["q"].shape[-1] ** -0.5, "fp8" if c["ks"] is not None else "auto", g["ks"], g["vs"],
        num_splits=splits, scratch=scratch, query_start_loc=g["q_start"] if with_q_start else None)
    return o


def _check(got, want):
    orc.check(got, want)
    orc.check_baseline(got, want)


# ---------------------------------------------------------------- lengths, tables, splits

@pytest.mark.parametrize("n", [1, 15, 17, 3 * 16 + 7])
def test_single_request_lengths(n):
    c = _case([n], h_kv=8, group=4)
    _check(_run(c, splits=1), _reference(c))


def test_ragged_batch_scrambled_table():
    c = _case([5, 700, 33, 2048, 1, 16], h_kv=8, group=4)
    _check(_run(c, splits=1), _reference(c))


@pytest.mark.parametrize("splits", [1, 2, 3, 8, 32])
@pytest.mark.parametrize("group,h_kv", [(4, 8), (8, 2)])
def test_lens_by_splits(splits, group, h_kv):
    c = _case(LENS, h_kv=h_kv, group=group, seed=splits)
    _check(_run(c, splits=splits), _reference(c))


@pytest.mark.parametrize("splits", [64, 256])
def test_many_more_splits_than_pages(splits):
    c = _case([1, 31, 32, 33, 200, 1000], h_kv=2, group=4, seed=7)
    _check(_run(c, splits=splits), _reference(c))


@pytest.mark.parametrize("h_kv,group", [(1, 16), (2, 8), (4, 6), (8, 4), (2, 1), (2, 2), (2, 3), (1, 5), (1, 7),
                                        (1, 12)])
def test_gqa_shapes(h_kv, group):
    c = _case([1, 33, 1000, 2063], h_kv=h_kv, group=group, seed=group)
    want = _reference(c)
    _check(_run(c, splits=1), want)
    _check(_run(c, splits=4), want)


@pytest.mark.parametrize("group", [4, 8])
def test_head_dim_64(group):
    c = _case([1, 33, 1000], head_dim=64, h_kv=2, group=group, seed=3)
    want = _reference(c)
    _check(_run(c, splits=1), want)
    _check(_run(c, splits=4), want)


@pytest.mark.parametrize("page", [32, 48])
@pytest.mark.parametrize("group", [4, 8])
def test_pages_of_a_multiple_of_16(page, group):
    c = _case([1, 47, 48, 49, 1000], h_kv=2, group=group, page=page, seed=page)
    want = _reference(c)
    _check(_run(c, splits=1), want)
    _check(_run(c, splits=4), want)


@pytest.mark.parametrize("group", [4, 8])
def test_vllm_nhd_layout(group):
    c = _case([1, 33, 1000, 2063], h_kv=4, group=group, layout="nhd", seed=5)
    assert c["k"].stride(2) != c["k"].shape[3]          # really token-major storage
    want = _reference(c)
    _check(_run(c, splits=1), want)
    _check(_run(c, splits=8), want)


# ------------------------------------------------------------------------- known answers

@pytest.mark.parametrize("group", [4, 8])
@pytest.mark.parametrize("splits", [1, 8])
def test_v_of_ones_gives_exactly_one(group, splits):
    c = _case(LENS, h_kv=2, group=group, v_ones=True)
    got = _run(c, splits=splits)
    assert (got.float() == 1.0).all()


@pytest.mark.parametrize("group", [4, 8])
@pytest.mark.parametrize("splits", [1, 4])
def test_nan_past_the_end_is_never_read_into_the_answer(group, splits):
    c = _case([1, 15, 17, 33, 1000], h_kv=2, group=group, nan_tail=True, seed=2)
    clean = _case([1, 15, 17, 33, 1000], h_kv=2, group=group, nan_tail=False, seed=2)
    got = _run(c, splits=splits)
    assert torch.isfinite(got.float()).all()
    _check(got, _reference(clean))


@pytest.mark.parametrize("group", [4, 8])
def test_poison_past_the_end_changes_no_bit(group):
    lens = [1, 15, 17, 3 * 16 + 7]
    c = _case(lens, h_kv=2, group=group, seed=4)
    a = _run(c, splits=1).clone()
    k, v = c["k"].clone(), c["v"].clone()
    for i, s in enumerate(lens):
        j = (s - 1) // 16
        k[int(c["table"][i, j]), :, s - j * 16:] = 1e4
        v[int(c["table"][i, j]), :, s - j * 16:] = 1e4
    c2 = dict(c, k=k, v=v)
    b = _run(c2, splits=1)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_a_padded_request_reads_nothing_and_answers_zero():
    c = _case([40, 0, 200, 0], h_kv=2, group=4, seed=6)
    for splits in (1, 4):
        out = torch.full(c["q"].shape, 7.0, device="cuda", dtype=torch.bfloat16)
        got = _run(c, splits=splits, out=out)
        assert (got[1] == 0).all() and (got[3] == 0).all()
        _check(got, _reference(c))


@pytest.mark.parametrize("group", [4, 8])
def test_graph_padding_writes_nothing(group):
    """Requests with no query (query_start_loc repeats) leave their output rows untouched."""
    c = _case([33, 1000], h_kv=2, group=group, pad=3, seed=8)
    for splits in (1, 4):
        out = torch.full(c["q"].shape, 7.0, device="cuda", dtype=torch.bfloat16)
        got = _run(c, splits=splits, out=out, with_q_start=True)
        assert (got[2:] == 7.0).all()
        _check(got[:2], _reference(c, with_q_start=True)[:2])


def test_strided_q_of_a_fused_qkv():
    c = _case([33, 1000, 5], h_kv=2, group=4, strided_q=True, seed=9)
    _check(_run(c, splits=2), _reference(c))


@pytest.mark.parametrize("group", [4, 8])
def test_two_hundred_calls_over_poisoned_scratch_are_bitwise_equal_on_a_side_stream(group):
    paged = _paged()
    c = _cuda(_case(LENS, h_kv=2, group=group, seed=10))
    n, h, d = c["q"].shape
    splits = 8
    scratch = paged.split_scratch(n, h, d, splits, "cuda")
    first = None
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for it in range(200):
            scratch[0].fill_(float("nan"))
            scratch[1].fill_(float("nan"))
            out = torch.full((n, h, d), float("nan"), device="cuda", dtype=torch.bfloat16)
            _run(c, splits=splits, out=out, scratch=scratch)
            if first is None:
                first = out.clone()
            else:
                assert torch.equal(out.view(torch.int16), first.view(torch.int16)), f"call {it} differs"
    side.synchronize()
    assert torch.isfinite(first.float()).all()


@pytest.mark.parametrize("group", [4, 8])
def test_split_and_unsplit_agree(group):
    c = _case([700, 33, 2048], h_kv=2, group=group, seed=12)
    a, b = _run(c, splits=1).float(), _run(c, splits=8).float()
    assert (a - b).abs().max().item() < 2e-2


# ---------------------------------------------------------------------------------- fp8

@pytest.mark.parametrize("group", [4, 8, 16])
@pytest.mark.parametrize("splits", [1, 4])
def test_fp8_cache_against_the_dequantised_oracle(group, splits):
    c = _case([1, 15, 33, 1000, 2063], h_kv=2, group=group, fp8=True, seed=13)
    _check(_run(c, splits=splits), _reference(c))


@pytest.mark.parametrize("head_dim", [64, 256])
@pytest.mark.parametrize("group,h_kv", [(1, 2), (4, 2), (8, 1), (16, 1)])
@pytest.mark.parametrize("splits", [1, 4, 32])
def test_fp8_cache_at_head_sizes_64_and_256(head_dim, group, h_kv, splits):
    """fp8 rows of 64 and 256 bytes: one split (the fixed grid, tiles widened in shared memory) and the
    balanced stream (fragments built from the fp8 tile in its 32-byte-unit layout)."""
    c = _case(LENS, head_dim=head_dim, h_kv=h_kv, group=group, fp8=True, seed=head_dim + group)
    _check(_run(c, splits=splits), _reference(c))


@pytest.mark.parametrize("head_dim", [64, 256])
def test_fp8_pages_of_64_tokens_at_head_sizes_64_and_256(head_dim):
    c = _case([1, 63, 65, 700, 2063], head_dim=head_dim, h_kv=2, group=4, page=64, fp8=True, seed=head_dim)
    _check(_run(c, splits=8), _reference(c))


# --------------------------------------------------------------------------- CUDA graphs

@pytest.mark.parametrize("group", [4, 8])
def test_captured_graph_replays_over_new_lengths_and_a_flipped_table(group):
    paged = _paged()
    c = _cuda(_case([1000, 33, 2063, 500], h_kv=2, group=group, seed=14))
    n, h, d = c["q"].shape
    splits = 4
    scratch = paged.split_scratch(n, h, d, splits, "cuda")
    out = torch.empty(n, h, d, device="cuda", dtype=torch.bfloat16)
    _run(c, splits=splits, out=out, scratch=scratch)       # warm up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        _run(c, splits=splits, out=out, scratch=scratch)
    graph.replay()
    torch.cuda.synchronize()
    cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    _check(out, _reference(cpu))
    # new lengths and a flipped table, written in place; the replay must follow them
    c["lens"].copy_(torch.tensor([17, 1000, 1, 333], dtype=torch.int32))
    c["table"].copy_(c["table"].flip(0))
    graph.replay()
    torch.cuda.synchronize()
    cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    _check(out, _reference(cpu))


# ---------------------------------------------------------------------------- refusals

def test_bad_shapes_are_refused_before_launch():
    paged = _paged()
    c = _cuda(_case([33], h_kv=2, group=4))
    o = torch.empty_like(c["q"])
    kc, vc = c["k"].transpose(1, 2), c["v"].transpose(1, 2)
    with pytest.raises(ValueError):
        paged.paged_attention_decode(o[:, :4], c["q"], kc, vc, c["table"], c["lens"], 0.1)
    with pytest.raises(TypeError):
        paged.paged_attention_decode(o, c["q"], kc, vc, c["table"].long(), c["lens"], 0.1)
    with pytest.raises(TypeError):
        paged.paged_attention_decode(o, c["q"], kc, vc, c["table"], c["lens"].long(), 0.1)
    with pytest.raises(ValueError):
        paged.paged_attention_decode(o, c["q"], kc[..., :64], vc[..., :64], c["table"], c["lens"], 0.1)
    with pytest.raises(ValueError):
        paged.paged_attention_decode(o, c["q"].float(), kc, vc, c["table"], c["lens"], 0.1)
    from hk_dsl_b200.runtime.lib import HkbError
    with pytest.raises(HkbError):      # 3 q heads over 2 kv heads: refused by the C ABI, nothing launched
        paged.paged_attention_decode(o[:, :3], c["q"][:, :3], kc, vc, c["table"], c["lens"], 0.1, num_splits=1)
    with pytest.raises(HkbError):
        paged.paged_attention_decode(o, c["q"], kc, vc, c["table"], c["lens"], 0.1, num_splits=1000)


# ------------------------------------------------------------------- hk's own call form

@pytest.mark.parametrize("splits", [1, 4])
def test_hk_form_decode_and_merge(splits):
    """`decode(q, k_cache, v_cache, block_table, seq_lens, out, scratch, splits)` on
    (requests, kv_heads, group, d) views, as python/hk/integration/vllm_backend.py:715-728 calls it."""
    paged = _paged()
    c = _case([1, 31, 32, 33, 200, 1000], h_kv=8, group=4, seed=15)
    g = _cuda(c)
    n, h, d = c["q"].shape
    q4, out = g["q"].view(n, 8, 4, d), torch.empty(n, h, d, device="cuda", dtype=torch.bfloat16)
    scratch = paged.fused_scratch(n * splits, 8, d, "cuda", group=4)
    paged.decode(q4, g["k"], g["v"], g["table"], g["lens"], out.view(n, 8, 4, d), scratch, splits)
    _check(out, _reference(c))


# ---------------------------------------------------------------- head_dim 256 (decode only)

@pytest.mark.parametrize("splits", [1, 4, 32])
@pytest.mark.parametrize("group,h_kv", [(2, 4), (8, 1), (16, 1)])
def test_head_dim_256(splits, group, h_kv):
    """512-byte rows (the reference lists D=256 among the shapes beside its D=128 route,
    python/hk/ops/paged_decode.py:17-20): the tensor-core worker at every group, one split and the stream."""
    c = _case(LENS, head_dim=256, h_kv=h_kv, group=group, seed=7 + splits)
    _check(_run(c, splits=splits), _reference(c))


def test_head_dim_256_step_writes_the_cache():
    paged = _paged()
    c = _case([5, 700, 33, 2048], head_dim=256, h_kv=2, group=4, seed=3)
    g = _cuda(c)
    n, hkv, d = 4, 2, 256
    gen = torch.Generator().manual_seed(11)
    key = torch.randn(n, hkv, d, generator=gen).to(torch.bfloat16)
    value = torch.randn(n, hkv, d, generator=gen).to(torch.bfloat16)
    slots = torch.tensor([int(c["table"][i, (s - 1) // 16]) * 16 + (s - 1) % 16 for i, s in enumerate([5, 700, 33, 2048])])
    k_want, v_want = c["k"].clone(), c["v"].clone()
    k_want[slots // 16, :, slots % 16] = key
    v_want[slots // 16, :, slots % 16] = value
    out = torch.empty_like(g["q"])
    paged.decode_step(out, g["q"], key.cuda(), value.cuda(), g["k"].transpose(1, 2), g["v"].transpose(1, 2), slots.cuda(),
                      g["table"], g["lens"], d ** -0.5, num_splits=8)
    assert torch.equal(g["k"].cpu(), k_want) and torch.equal(g["v"].cpu(), v_want)
    want = orc.paged_decode_ref(c["q"], k_want.transpose(1, 2), v_want.transpose(1, 2), c["table"], c["lens"])
    _check(out.cpu(), want)


# ---------------------------------------------------------------- hybrid page sizes

@pytest.mark.parametrize("page", [544, 784, 2064])
@pytest.mark.parametrize("group,h_kv,fp8", [(4, 2, False), (8, 1, False), (4, 2, True)])
def test_hybrid_page_sizes_with_nan_past_the_end(page, group, h_kv, fp8):
    """Pages of 544 / 784 / 2064 tokens -- the sizes vLLM gives a hybrid model's attention layers,
    with NaN in the unused tail of the last page (python/hk/ops/paged_decode.py:17-20, 93-94):
    34 / 49 / 129 16-token tiles a page, lengths that end inside, at and just past a page."""
    lens = [1, page - 1, page, page + 1, 2 * page + 17]
    c = _case(lens, h_kv=h_kv, group=group, page=page, seed=page, nan_tail=not fp8, fp8=fp8, spare=1)
    _check(_run(c, splits=4), _reference(c))
    _check(_run(c, splits=1), _reference(c))


def test_read_probe_runs_and_reads_at_a_plausible_rate():
    """hkb_hbm_read_probe through the C ABI: it launches, touches nothing but its sink, and a 256 MB
    read lands between 1 and 12 TB/s on an HBM3e part (a sanity band, not a benchmark)."""
    from hk_dsl_b200.runtime import lib as hkb

    lib = hkb.load()
    nbytes = 256 << 20
    buf = torch.full((nbytes + 64,), 0x5a, dtype=torch.uint8, device="cuda")
    sink = torch.zeros(4, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    best = 0.0
    for ctas, inflight in ((2, 4), (4, 8)):
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            assert lib.hkb_hbm_read_probe(buf.data_ptr(), nbytes, ctas, inflight, sink.data_ptr(), st) == 0
            b.record()
            torch.cuda.synchronize()
            best = max(best, nbytes / (a.elapsed_time(b) * 1e-3) / 1e9)
    assert 1000.0 < best < 12000.0, best
    assert (buf[nbytes:] == 0x5a).all() and (sink == 0).all()
    assert lib.hkb_hbm_read_probe(buf.data_ptr(), nbytes, 2, 3, sink.data_ptr(), st) == -9       # loads in flight: 1, 2, 4, 8, 16


def test_the_environment_switches_are_read_at_every_call(monkeypatch):
    """`HKB_MMA_MIN_GROUP` moves the worker bound between two calls of one process."""
    from hk_dsl_b200.runtime import lib as hkb

    lib = hkb.load()
    monkeypatch.delenv("HKB_MMA_MIN_GROUP", raising=False)
    assert lib.hkb_walk_uses_mma(4, 0) == 1 and lib.hkb_walk_uses_mma(3, 0) == 0
    monkeypatch.setenv("HKB_MMA_MIN_GROUP", "8")
    assert lib.hkb_walk_uses_mma(4, 0) == 0 and lib.hkb_walk_uses_mma(8, 1) == 1 and lib.hkb_walk_uses_mma(4, 1) == 0
    c = _case([700, 33, 1500], group=4, h_kv=2, seed=3)
    want = _reference(c)
    _check(_run(c, splits=4), want)               # the CUDA-core worker
    monkeypatch.setenv("HKB_FIXED_SPLITS", "1")
    _check(_run(c, splits=4), want)               # on the fixed-split grid
    monkeypatch.delenv("HKB_FIXED_SPLITS")
    monkeypatch.delenv("HKB_MMA_MIN_GROUP")
    _check(_run(c, splits=4), want)               # the default worker again
