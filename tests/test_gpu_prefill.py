"""Paged prefill against the float64 oracle, through the C ABI. Cases are those of the reference's
tests/hk/gpu/test_paged_prefill.py:86-125: no prefix with a short second tile, a cached prefix with
a chunk shorter than a tile, a tile that runs into the next request, a ragged batch with a
one-token request, requests outside the work list untouched, every GQA group, head_dim 64 -- plus
NaN past the ends, vLLM's NHD layout, pages of 32, and a long prompt."""

import pytest
import torch

from oracle import paged_oracle as orc

pytestmark = pytest.mark.gpu
PAGE = 16


def _case(reqs, head_dim=128, h_kv=2, group=4, seed=0, page=PAGE, nan_past=False, layout="hnd"):
    """reqs: [(ctx, q_len)]. Every request's whole sequence is in the cache; its last q_len tokens
    are the queries (tests/hk/gpu/test_paged_prefill.py:30-51)."""
    g = torch.Generator().manual_seed(seed)
    r = len(reqs)
    seq = [c + n for c, n in reqs]
    max_pages = max(1, max(-(-s // page) for s in seq))
    nb = r * max_pages + 5
    k = torch.randn(nb, h_kv, page, head_dim, generator=g).to(torch.bfloat16)
    v = torch.randn(nb, h_kv, page, head_dim, generator=g).to(torch.bfloat16)
    table = torch.randperm(nb, generator=g)[: r * max_pages].reshape(r, max_pages).to(torch.int32).contiguous()
    if nan_past:
        live = torch.zeros(nb, page, dtype=torch.bool)
        for i, s in enumerate(seq):
            for j in range(-(-s // page)):
                live[int(table[i, j]), : min(page, s - j * page)] = True
        dead = ~live[:, None, :, None]
        k, v = k.masked_fill(dead, float("nan")), v.masked_fill(dead, float("nan"))
    n_tok = sum(n for _, n in reqs)
    q = torch.randn(n_tok, h_kv * group, head_dim, generator=g).to(torch.bfloat16)
    starts = [0]
    for _, n in reqs:
        starts.append(starts[-1] + n)
    if layout == "nhd":
        k, v = k.transpose(1, 2).contiguous().transpose(1, 2), v.transpose(1, 2).contiguous().transpose(1, 2)
    return q, k, v, table, torch.tensor(seq, dtype=torch.int32), torch.tensor(starts, dtype=torch.int32)


def _run(reqs, prefill=None, **kw):
    from hk_dsl_b200.ops import paged

    q, k, v, table, lens, q_start = _case(reqs, **kw)
    clean = _case(reqs, **dict(kw, nan_past=False)) if kw.get("nan_past") else (q, k, v, table, lens, q_start)
    n_tok, h, d = q.shape
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
    which = range(len(reqs)) if prefill is None else prefill
    rows = paged.prefill_tile_rows(h, k.shape[1])
    work = paged.work_list([(r, reqs[r][1]) for r in which], rows, "cuda", seq_lens=lens.tolist())
    paged.paged_prefill(out, q.cuda(), k.cuda().transpose(1, 2), v.cuda().transpose(1, 2), table.cuda(), lens.cuda(),
                        q_start.cuda(), work, d ** -0.5)
    torch.cuda.synchronize()
    want = orc.paged_prefill_ref(clean[0], clean[1].transpose(1, 2), clean[2].transpose(1, 2), table, lens, q_start)
    return out, want, q_start


def test_no_prefix_two_tiles_the_second_short():
    got, want, _ = _run([(0, 300)])
    orc.check(got, want)


def test_a_cached_prefix_and_a_chunk_shorter_than_a_tile():
    got, want, _ = _run([(1000, 77)])
    orc.check(got, want)


def test_a_tile_that_runs_into_the_next_request():
    got, want, _ = _run([(64, 100), (300, 50), (0, 200)])
    orc.check(got, want)


def test_ragged_batch_with_a_one_token_request():
    got, want, _ = _run([(0, 192), (500, 5), (40, 600), (33, 1)])
    orc.check(got, want)
    orc.check_baseline(got, want)


def test_rows_of_requests_not_in_the_work_list_are_untouched():
    reqs = [(0, 40), (128, 70), (10, 30)]
    got, want, q_start = _run(reqs, prefill=[1])
    a, b = int(q_start[1]), int(q_start[2])
    orc.check(got[a:b], want[a:b])
    assert (got[:a] == 7.0).all() and (got[b:] == 7.0).all()


@pytest.mark.parametrize("group", [1, 2, 3, 4, 6, 8, 16])
def test_every_gqa_group(group):
    got, want, _ = _run([(37, 150), (0, 17), (260, 1)], group=group, seed=group)
    orc.check(got, want)


def test_head_dim_64():
    got, want, _ = _run([(100, 90), (0, 33)], head_dim=64, group=4, seed=3)
    orc.check(got, want)


def test_nan_past_the_ends_never_reaches_the_answer():
    got, want, _ = _run([(0, 300), (1000, 77), (5, 1), (16, 16)], nan_past=True, seed=5)
    assert torch.isfinite(got.float()).all()
    orc.check(got, want)


@pytest.mark.parametrize("page", [32, 48])
def test_pages_of_a_multiple_of_16(page):
    got, want, _ = _run([(100, 90), (0, 130)], page=page, seed=page)
    orc.check(got, want)


def test_vllm_nhd_layout():
    got, want, _ = _run([(64, 100), (0, 200)], layout="nhd", h_kv=4, seed=6)
    orc.check(got, want)


def test_a_long_prompt_and_a_long_prefix():
    got, want, _ = _run([(0, 2100), (4000, 300)], h_kv=1, group=4, seed=7)
    orc.check(got, want)


def test_refusals():
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime.lib import HkbError

    q, k, v, table, lens, q_start = _case([(0, 40)])
    kw = dict(block_tables=table.cuda(), seq_lens=lens.cuda(), query_start_loc=q_start.cuda(),
              work=paged.work_list([(0, 40)], 32, "cuda"), scale=0.1)
    out = torch.empty_like(q).cuda()
    with pytest.raises(TypeError):
        paged.paged_prefill(out, q.cuda(), k.cuda().transpose(1, 2), v.cuda().transpose(1, 2),
                            **dict(kw, seq_lens=lens.long().cuda()))
    with pytest.raises(ValueError):
        paged.paged_prefill(out, q.cuda().float(), k.cuda().transpose(1, 2), v.cuda().transpose(1, 2), **kw)
    k8 = k.cuda().to(torch.float8_e4m3fn).transpose(1, 2)
    with pytest.raises(ValueError, match="k_scale"):          # an fp8 cache needs its scales
        paged.paged_prefill(out, q.cuda(), k8, k8, kv_cache_dtype="fp8", **kw)


@pytest.mark.parametrize("head_dim", [64, 256])
@pytest.mark.parametrize("group", [1, 4, 8])
def test_fp8_cache_at_head_sizes_64_and_256(head_dim, group):
    from hk_dsl_b200.ops import paged

    reqs = [(0, 300), (1000, 77), (33, 1), (64, 100)]
    q, k, v, table, lens, q_start = _case(reqs, head_dim=head_dim, group=group, seed=40 + group)
    ks, vs = torch.tensor([0.0125]), torch.tensor([0.011])
    k8, v8 = orc.quantize_fp8(k, ks), orc.quantize_fp8(v, vs)
    want = orc.paged_prefill_ref(q, orc.dequantize_fp8(k8, ks).transpose(1, 2), orc.dequantize_fp8(v8, vs).transpose(1, 2),
                                 table, lens, q_start)
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
    work = paged.work_list([(r, n) for r, (_, n) in enumerate(reqs)], paged.prefill_tile_rows(q.shape[1], 2), "cuda")
    paged.paged_prefill(out, q.cuda(), k8.cuda().transpose(1, 2), v8.cuda().transpose(1, 2), table.cuda(), lens.cuda(),
                        q_start.cuda(), work, head_dim ** -0.5, "fp8", ks.cuda(), vs.cuda())
    torch.cuda.synchronize()
    orc.check(out, want)


@pytest.mark.parametrize("group", [1, 4, 8])
def test_fp8_cache_against_the_dequantised_oracle(group):
    from hk_dsl_b200.ops import paged

    reqs = [(0, 300), (1000, 77), (33, 1), (64, 100)]
    q, k, v, table, lens, q_start = _case(reqs, group=group, seed=20 + group)
    ks, vs = torch.tensor([0.0125]), torch.tensor([0.011])
    k8, v8 = orc.quantize_fp8(k, ks), orc.quantize_fp8(v, vs)
    want = orc.paged_prefill_ref(q, orc.dequantize_fp8(k8, ks).transpose(1, 2), orc.dequantize_fp8(v8, vs).transpose(1, 2),
                                 table, lens, q_start)
    out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
    work = paged.work_list([(r, n) for r, (_, n) in enumerate(reqs)], paged.prefill_tile_rows(q.shape[1], 2), "cuda")
    paged.paged_prefill(out, q.cuda(), k8.cuda().transpose(1, 2), v8.cuda().transpose(1, 2), table.cuda(), lens.cuda(),
                        q_start.cuda(), work, 128 ** -0.5, "fp8", ks.cuda(), vs.cuda())
    torch.cuda.synchronize()
    orc.check(out, want)
    orc.check_baseline(out, want)


@pytest.mark.parametrize("page", [16, 64])
def test_fp8_cache_on_both_kernel_forms(page, monkeypatch):
    """An fp8 cache on the tensor-memory kernel (the producers widen e4m3 to f16 on the way into the
    ring) and on the mma.sync one: both within the oracle's bounds of the dequantised reference, and
    within three bf16 ulps of each other; a long prompt, so the ring of slots laps, a cached prefix,
    a chunk that ends inside a key block, and garbage past the end of the last page."""
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb

    reqs = [(0, 1500), (700, 333), (129, 1)]
    q, k, v, table, lens, q_start = _case(reqs, group=4, seed=31, page=page)
    ks, vs = torch.tensor([0.02]), torch.tensor([0.015])
    k8, v8 = orc.quantize_fp8(k, ks), orc.quantize_fp8(v, vs)
    want = orc.paged_prefill_ref(q, orc.dequantize_fp8(k8, ks).transpose(1, 2), orc.dequantize_fp8(v8, vs).transpose(1, 2),
                                 table, lens, q_start)
    # bytes past each request's last token: 0x7f is NaN in e4m3
    k8d, v8d = k8.cuda(), v8.cuda()
    for r, (c, n) in enumerate(reqs):
        last = c + n
        blk, off = int(table[r, (last - 1) // page]), (last - 1) % page + 1
        k8d.view(torch.uint8)[blk, :, off:] = 0x7f
        v8d.view(torch.uint8)[blk, :, off:] = 0x7f
    work = paged.work_list([(r, n) for r, (_, n) in enumerate(reqs)], paged.prefill_tile_rows(q.shape[1], 2), "cuda")
    outs = []
    for sync in ("0", "1"):
        monkeypatch.setenv("HKB_PREFILL_MMA_SYNC", sync)
        out = torch.full(q.shape, 7.0, device="cuda", dtype=torch.bfloat16)
        paged.paged_prefill(out, q.cuda(), k8d.transpose(1, 2), v8d.transpose(1, 2), table.cuda(), lens.cuda(),
                            q_start.cuda(), work, 128 ** -0.5, "fp8", ks.cuda(), vs.cuda())
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        orc.check(out, want)
        outs.append(out)
    assert orc.ulps(outs[0], outs[1].float()) <= 3.0
    assert hkb.load().hkb_prefill_tc_error(0) == 0


@pytest.mark.parametrize("seed", range(8))
def test_many_items_a_cta_in_every_mix(seed):
    """More work items than SMs, so a persistent CTA walks several in a row: items whose second query tile
    is empty beside items with both, one-block items beside long ones, one-token requests, prefixes that
    end inside a key block -- the barrier phases must carry over every such sequence of items. Seeded
    random batches (six of the eight hold more items than a B200 has SMs), NaN past the ends in half of them."""
    import random

    from hk_dsl_b200.runtime import lib as hkb

    rng = random.Random(100 + seed)
    group = rng.choice([1, 2, 4, 8])
    h_kv = rng.choice([2, 4, 8]) if group <= 4 else rng.choice([1, 2])
    page = rng.choice([16, 16, 32, 64])
    reqs = []
    for _ in range(rng.randint(12, 40)):
        kind = rng.random()
        if kind < 0.2:
            reqs.append((rng.randint(0, 700), 1))                       # a decode inside the batch
        elif kind < 0.6:
            reqs.append((rng.choice([0, 0, 17, 128, 300]), rng.randint(2, 140)))   # short chunks: second tile often empty
        else:
            reqs.append((rng.randint(0, 900), rng.randint(141, 520)))
    got, want, _ = _run(reqs, h_kv=h_kv, group=group, page=page, seed=200 + seed, nan_past=(seed % 2 == 0))
    assert torch.isfinite(got.float()).all()
    orc.check(got, want)
    assert hkb.load().hkb_prefill_tc_error(0) == 0


def test_which_kernel_runs_and_that_no_wait_ran_out(monkeypatch):
    """head_dim 128 on a 16-bit cache runs the tcgen05 / tensor-memory kernel, everything else (and
    HKB_PREFILL_MMA_SYNC=1) the mma.sync one; both give the oracle's answer on the same inputs and
    each other's within three bf16 ulps of the row maximum; the tensor-memory kernel's bounded waits
    left no error code behind -- in this test or in any that ran before it in this process."""
    from hk_dsl_b200.runtime import lib as hkb

    lib = hkb.load()
    monkeypatch.delenv("HKB_PREFILL_MMA_SYNC", raising=False)
    assert lib.hkb_prefill_uses_tcgen05(128, hkb.KV_BF16) == 1 and lib.hkb_prefill_uses_tcgen05(128, hkb.KV_F16) == 1
    assert lib.hkb_prefill_uses_tcgen05(128, hkb.KV_FP8_E4M3) == 1 and lib.hkb_prefill_uses_tcgen05(64, hkb.KV_BF16) == 0
    assert lib.hkb_prefill_uses_tcgen05(256, hkb.KV_F16) == 0
    reqs = [(0, 700), (900, 300), (17, 1), (2048, 130)]
    new, want, _ = _run(reqs, h_kv=2, group=4, seed=11)
    orc.check(new, want)
    orc.check_baseline(new, want)
    monkeypatch.setenv("HKB_PREFILL_MMA_SYNC", "1")
    assert lib.hkb_prefill_uses_tcgen05(128, hkb.KV_BF16) == 0
    old, _, _ = _run(reqs, h_kv=2, group=4, seed=11)
    orc.check(old, want)
    assert orc.ulps(new, old.float()) <= 3.0
    monkeypatch.delenv("HKB_PREFILL_MMA_SYNC")
    assert lib.hkb_prefill_tc_error(0) == 0


@pytest.mark.parametrize("group,h_kv", [(1, 2), (2, 2), (4, 8), (8, 1), (16, 1), (6, 2)])
def test_tensor_memory_kernel_tile_shapes(group, h_kv):
    """Every way the 256 rows of a work item divide into tokens x heads (a group of 8 or 16: 32 tokens,
    4: 64, 2 or 6: 128, 1: 256), with a cached prefix, a chunk that ends inside the first query tile and
    one that ends inside the second."""
    from hk_dsl_b200.runtime import lib as hkb

    got, want, _ = _run([(100, 40), (0, 290), (515, 70), (64, 3)], h_kv=h_kv, group=group, seed=group)
    orc.check(got, want)
    assert hkb.load().hkb_prefill_tc_error(0) == 0


def test_tensor_memory_kernel_long_prompt_and_big_pages():
    """A 5000-token prompt (79 key blocks: the ring of slots laps ten times) and pages of 64 tokens."""
    got, want, _ = _run([(0, 5000)], h_kv=1, group=4, seed=3)
    orc.check(got, want)
    got, want, _ = _run([(300, 500), (0, 129)], h_kv=2, group=4, seed=4, page=64)
    orc.check(got, want)
