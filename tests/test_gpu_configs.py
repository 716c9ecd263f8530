"""The five measured configurations: parity against the float64 oracle where the oracle
finishes in seconds (c1 in full; c2-c5 on a slice of their sequences with their real shapes
and dtypes), EVERY sequence of the full-size c2 / c3 / c4 batches against the oracle's fp32
evaluation, one full 131072-token c5 sequence against the float64 oracle, and at FULL size
through properties that need no oracle: a cache of V == 1
answers exactly 1, split and unsplit walks agree, a kv-head shard equals the same heads of the
whole, a KV split over emulated ranks folds back to the single-GPU answer, the cache write is
an exact round trip, and a step leaves every other slot of the cache untouched."""

import pytest
import torch

from hk_dsl_b200 import workloads as W
from oracle import paged_oracle as orc

pytestmark = pytest.mark.gpu


def _paged():
    from hk_dsl_b200.ops import paged
    return paged


def _decode(st, splits=None, l=0, out=None):
    out = torch.empty_like(st.out) if out is None else out
    _paged().paged_attention_decode(out, st.query, st.k_caches[l], st.v_caches[l], st.block_table, st.seq_lens,
                                    st.scale, st.spec.kv_cache_dtype, st.k_scale, st.v_scale, num_splits=splits)
    return out


def _oracle(st, rows=None):
    n = len(st.lens)
    rows = range(n) if rows is None else rows
    want = torch.zeros(n, st.q_heads, st.spec.head_dim)
    bs = st.spec.block_size
    for i in rows:
        s = st.lens[i]
        pages = st.block_table[i, : -(-s // bs)].long()
        kc, vc = st.k_caches[0][pages].cpu(), st.v_caches[0][pages].cpu()
        table = torch.arange(kc.shape[0], dtype=torch.int32)[None]
        want[i] = orc.paged_decode_ref(st.query[i:i + 1].cpu(), kc, vc, table, torch.tensor([s], dtype=torch.int32),
                                       st.scale, st.k_scale.cpu() if st.k_scale is not None else None,
                                       st.v_scale.cpu() if st.v_scale is not None else None)[0]
    return want


def test_c1_in_full_cache_write_and_decode():
    spec = W.CONFIGS["c1"]
    st = W.build_step(spec, "cuda")
    kc, vc = st.k_caches[0], st.v_caches[0]
    want_k, want_v = kc.cpu().clone(), vc.cpu().clone()
    _paged().reshape_and_cache(st.key, st.value, kc, vc, st.slot_mapping, "auto")
    orc.reshape_and_cache_ref(st.key.cpu(), st.value.cpu(), want_k, want_v, st.slot_mapping.cpu())
    assert torch.equal(kc.cpu(), want_k) and torch.equal(vc.cpu(), want_v)
    want = orc.paged_decode_ref(st.query.cpu(), want_k, want_v, st.block_table.cpu(), st.seq_lens.cpu(), st.scale)
    for splits in (None, 1, 2, 8):
        got = _decode(st, splits)
        orc.check(got, want)
        orc.check_baseline(got, want)


@pytest.mark.parametrize("name,take", [("c2", 3), ("c3", 4), ("c4", 6), ("c5", 1)])
def test_config_slices_against_the_oracle(name, take):
    """The first `take` sequences of the config (c5: one sequence cut to 16384 tokens), with the
    config's head counts, dtype and scales."""
    spec = W.CONFIGS[name]
    lens = W.seq_lens_of(spec)[:take]
    if name == "c5":
        lens = [16384 + 5]
    st = W.build_step(spec, "cuda", lens=lens)
    _paged().reshape_and_cache(st.key, st.value, st.k_caches[0], st.v_caches[0], st.slot_mapping,
                               spec.kv_cache_dtype, st.k_scale, st.v_scale)
    want = _oracle(st)
    for splits in (None, 1, 4):
        got = _decode(st, splits)
        orc.check(got, want)
        orc.check_baseline(got, want)


@pytest.mark.parametrize("name", ["c2", "c3", "c4", "c5"])
def test_full_size_properties(name):
    spec = W.CONFIGS[name]
    st = W.build_step(spec, "cuda")
    paged = _paged()
    n = len(st.lens)
    kc, vc = st.k_caches[0], st.v_caches[0]

    # (1) the step's cache write: exact round trip of the new rows, nothing else touched
    before_k = kc.clone()
    paged.reshape_and_cache(st.key, st.value, kc, vc, st.slot_mapping, spec.kv_cache_dtype, st.k_scale, st.v_scale)
    slots = st.slot_mapping
    blk, off = slots // spec.block_size, slots % spec.block_size
    if spec.fp8:
        want_rows = orc.quantize_fp8(st.key.cpu(), st.k_scale.cpu()).view(torch.uint8)
        got_rows = kc[blk, off].view(torch.uint8).cpu()
    else:
        want_rows, got_rows = st.key.cpu(), kc[blk, off].cpu()
    assert torch.equal(got_rows, want_rows)
    changed = (kc.view(torch.uint8) != before_k.view(torch.uint8)).any(dim=-1).any(dim=-1)      # (blocks, block)
    mask = torch.zeros_like(changed)
    mask[blk, off] = True
    assert not (changed & ~mask).any()

    # (2) split and unsplit walks agree, and the planner's choice with them
    a = _decode(st, 1).float()
    planned = _decode(st, None).float()
    b = _decode(st, 8).float()
    assert torch.isfinite(a).all()
    assert (a - b).abs().max().item() < 2e-2 and (a - planned).abs().max().item() < 2e-2
    assert (a - b).abs().mean().item() < 2e-3

    # (3) spot check of the two shortest sequences against the oracle at full batch
    order = sorted(range(n), key=lambda i: st.lens[i])[:2] if name != "c5" else []
    if order:
        want = _oracle(st, order)
        orc.check(planned[order], want[order])

    # (4) a kv-head shard computes exactly the bits of those heads in the whole
    if spec.kv_heads >= 2:
        hkv, g = spec.kv_heads, spec.q_heads // spec.kv_heads
        lo, hi = hkv // 2, hkv
        out_sh = torch.empty(n, (hi - lo) * g, spec.head_dim, device="cuda", dtype=torch.bfloat16)
        paged.paged_attention_decode(out_sh, st.query[:, lo * g:hi * g], kc[:, :, lo:hi], vc[:, :, lo:hi],
                                     st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype, st.k_scale,
                                     st.v_scale, num_splits=1)
        whole = _decode(st, 1)
        assert torch.equal(out_sh.view(torch.int16), whole[:, lo * g:hi * g].contiguous().view(torch.int16))

    # (5) V == 1 answers exactly 1 (bf16 caches)
    if not spec.fp8:
        ones = torch.ones_like(vc)
        out = torch.empty_like(st.out)
        for s in (1, None):
            paged.paged_attention_decode(out, st.query, kc, ones, st.block_table, st.seq_lens, st.scale,
                                         num_splits=s)
            assert (out.float() == 1.0).all()


def test_c5_kv_split_over_emulated_ranks_folds_to_the_single_gpu_answer():
    """Four 'ranks' run one after another on one GPU, each on its own token range with its own
    local lengths and table slice; their (out, lse) records are laid out as the all-gather lays
    them and folded by the merge kernel."""
    from hk_dsl_b200.ops import paged_dist

    paged = _paged()
    spec = W.CONFIGS["c5"]
    st = W.build_step(spec, "cuda", lens=[32768 + 40, 20000])
    whole = _decode(st, None).float()
    world = 4
    n, hq, d = st.query.shape
    decs = [paged_dist.SplitKVDecoder(n, hq, st.kv_heads, d, "cuda", local_splits=4) for _ in range(world)]
    bs = spec.block_size
    for r, dec in enumerate(decs):
        ranges = [paged_dist.kv_range(s, world, r, bs) for s in st.lens]
        local = torch.tensor([hi - lo for lo, hi in ranges], dtype=torch.int32, device="cuda")
        table = torch.zeros_like(st.block_table)
        for i, (lo, hi) in enumerate(ranges):
            p0, p1 = lo // bs, -(-hi // bs)
            table[i, : p1 - p0] = st.block_table[i, p0:p1]
        dec.local_partial(st.query, st.k_caches[0], st.v_caches[0], table, local, st.scale)
    last = decs[0]
    last.world = world
    last.all = torch.cat([dec.mine for dec in decs])
    out = torch.empty_like(st.out)
    last.merge(out)
    torch.cuda.synchronize()
    assert (out.float() - whole).abs().max().item() < 2e-2
    assert (out.float() - whole).abs().mean().item() < 2e-3
    want = _oracle(st, [1])
    orc.check(out[1:2], want[1:2])


def _whole_batch_fp32(st):
    """The oracle's vectorised fp32 evaluation of every sequence of the step, on the host."""
    ks = st.k_scale.cpu() if st.k_scale is not None else None
    vs = st.v_scale.cpu() if st.v_scale is not None else None
    return orc.paged_decode_ref_fp32(st.query.cpu(), st.k_caches[0].cpu(), st.v_caches[0].cpu(), st.block_table.cpu(),
                                     st.seq_lens.cpu(), st.scale, ks, vs)


@pytest.mark.parametrize("name", ["c2", "c3", "c4"])
def test_every_sequence_of_the_full_batch_against_the_oracle(name):
    """The whole batch at its full size (64 / 128 / 256 sequences), the step as the bench runs it
    (`decode_step`: the walk writes the new rows, then the merge), every output row held to the
    oracle: max-abs 2e-2, mean-abs 2e-3 and the reference's 4-ulp row bound. The fp32 oracle's own
    error (~1e-6) is far below a bf16 ulp, so it stands in for the float64 one at this size; the
    shortest, median and longest sequence are also checked against float64."""
    spec = W.CONFIGS[name]
    st = W.build_step(spec, "cuda")
    paged = _paged()
    for splits in (None, 1):
        out = torch.full_like(st.out, 7.0)
        if splits is None:
            paged.decode_step(out, st.query, st.key, st.value, st.k_caches[0], st.v_caches[0], st.slot_mapping,
                              st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype, st.k_scale, st.v_scale)
        else:
            out = _decode(st, 1)
        torch.cuda.synchronize()
        if splits is None:
            want = _whole_batch_fp32(st)       # after the step: the cache holds the new rows
        orc.check(out, want)
        mx, mean = orc.check_baseline(out, want)
    n = len(st.lens)
    order = sorted(range(n), key=lambda i: (st.lens[i], i))
    few = sorted({order[0], order[n // 2], order[-1]})
    want64 = _oracle(st, few)
    orc.check(out[few], want64[few])
    if spec.fp8:       # the config's scales are amax / 448 of what was quantised: the largest value maps to +-448
        for cache, scale in ((st.k_caches[0], st.k_scale), (st.v_caches[0], st.v_scale)):
            top = cache.view(torch.uint8).cpu().view(torch.float8_e4m3fn).float().abs().max().item()
            assert top == 448.0 and 5.0 / 448 < scale.item() < 7.0 / 448


@pytest.mark.parametrize("splits", [None, 256])
def test_c5_a_full_131072_token_sequence_against_the_float64_oracle(splits):
    """What c5 is about: 8192 tiles of one sequence through every slot the plan gives it (and
    through all 256, where the wide merge folds them), compared with float64 for the query heads
    of two kv heads (the other heads run the same code on other data)."""
    spec = W.CONFIGS["c5"]
    st = W.build_step(spec, "cuda", lens=[131072])
    paged = _paged()
    out = torch.empty_like(st.out)
    paged.decode_step(out, st.query, st.key, st.value, st.k_caches[0], st.v_caches[0], st.slot_mapping,
                      st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype, num_splits=splits)
    torch.cuda.synchronize()
    g = spec.q_heads // spec.kv_heads
    pages = st.block_table[0, : 131072 // spec.block_size].long()
    q = st.query.cpu()
    for kh in (0, spec.kv_heads - 1):
        kk = st.k_caches[0][pages][:, :, kh].reshape(-1, spec.head_dim).cpu()
        vv = st.v_caches[0][pages][:, :, kh].reshape(-1, spec.head_dim).cpu()
        hs = slice(kh * g, (kh + 1) * g)
        want = orc.softmax_v64(q[0, hs], kk, vv, st.scale)
        orc.check(out[0, hs], want)
        orc.check_baseline(out[0, hs], want)


def test_kv_split_step_writes_the_new_rows_on_the_rank_that_holds_them():
    """A KV-split step as two emulated ranks run one after the other on one GPU: the rank that holds
    the sequences' last position passes the step's new rows and its walk writes them (the same bits
    the cache-write kernel writes); the other passes none. The folded records equal the one-GPU
    step's answer within tolerance and the float64 oracle's within the row bound."""
    from hk_dsl_b200.ops import paged_dist

    paged = _paged()
    spec = W.CONFIGS["c5"]
    lens = [4096 + 33, 2048]
    st = W.build_step(spec, "cuda", lens=lens)
    ref = W.build_step(spec, "cuda", lens=lens)          # the same seeded tensors, for the separate launches
    paged.reshape_and_cache(ref.key, ref.value, ref.k_caches[0], ref.v_caches[0], ref.slot_mapping, "auto")
    whole = _decode(ref, None).float()
    world, bs = 2, spec.block_size
    n, hq, d = st.query.shape
    decs = [paged_dist.SplitKVDecoder(n, hq, st.kv_heads, d, "cuda", local_splits=4) for _ in range(world)]
    for r, dec in enumerate(decs):
        ranges = [paged_dist.kv_range(s, world, r, bs) for s in st.lens]
        local = torch.tensor([hi - lo for lo, hi in ranges], dtype=torch.int32, device="cuda")
        table = torch.zeros_like(st.block_table)
        slots = torch.full_like(st.slot_mapping, -1)
        for i, (lo, hi) in enumerate(ranges):
            p0, p1 = lo // bs, -(-hi // bs)
            table[i, : p1 - p0] = st.block_table[i, p0:p1]
            if hi == st.lens[i] and hi > lo:      # this rank holds the last position: the new row is its to write
                slots[i] = st.slot_mapping[i]
        new = dict(key=st.key, value=st.value, slot_mapping=slots) if (slots >= 0).any() else {}
        dec.local_partial(st.query, st.k_caches[0], st.v_caches[0], table, local, st.scale, **new)
    torch.cuda.synchronize()
    assert torch.equal(st.k_caches[0].view(torch.int16), ref.k_caches[0].view(torch.int16))
    assert torch.equal(st.v_caches[0].view(torch.int16), ref.v_caches[0].view(torch.int16))
    last = decs[0]
    last.world = world
    last.all = torch.cat([dec.mine for dec in decs])
    out = torch.empty_like(st.out)
    last.merge(out)
    torch.cuda.synchronize()
    assert (out.float() - whole).abs().max().item() < 2e-2
    want = _oracle(ref)
    orc.check(out, want)


@pytest.mark.parametrize("exchange", ["peer", "peer2"])
def test_peer_exchange_on_one_gpu_equals_the_step_and_replays_from_a_graph(exchange):
    """The exchange over peer memory with the rank as its own only peer: walk (writing the new rows),
    then the exchange in one launch (or push, merge) -- no collective -- gives the bits of the two-launch step when the
    walk and the fold are the same kernels' arithmetic (the fold order differs: tolerance), step after
    step (the gather halves and flags alternate by the step counter's parity), and from a CUDA graph."""
    from hk_dsl_b200.ops import paged_dist

    paged = _paged()
    spec = W.CONFIGS["c5"]
    lens = [3000 + 7, 1500]
    st = W.build_step(spec, "cuda", lens=lens)
    ref = W.build_step(spec, "cuda", lens=lens)
    n, hq, d = st.query.shape
    want = torch.empty_like(ref.out)
    paged.decode_step(want, ref.query, ref.key, ref.value, ref.k_caches[0], ref.v_caches[0], ref.slot_mapping,
                      ref.block_table, ref.seq_lens, ref.scale, num_splits=8)
    dec = paged_dist.SplitKVDecoder(n, hq, st.kv_heads, d, "cuda", local_splits=8, exchange=exchange)   # one launch / two
    assert dec.peer.world == 1 and dec.peer.error() == 0
    out = torch.full_like(st.out, 7.0)
    for step in range(3):                                   # parities 0, 1, 0
        out.fill_(7.0)
        dec.decode(out, st.query, st.k_caches[0], st.v_caches[0], st.block_table, st.seq_lens, st.scale,
                   key=st.key, value=st.value, slot_mapping=st.slot_mapping)
        torch.cuda.synchronize()
        assert dec.peer.error() == 0
        assert int(dec.peer.state[16].item()) == step + 1  # the step counter moved on
        orc.check(out, want.float())
    assert torch.equal(st.k_caches[0].view(torch.int16), ref.k_caches[0].view(torch.int16))   # the walk wrote the rows
    orc.check(out, _oracle(ref))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        dec.decode(out, st.query, st.k_caches[0], st.v_caches[0], st.block_table, st.seq_lens, st.scale)
    for _ in range(3):
        out.fill_(7.0)
        g.replay()
        torch.cuda.synchronize()
        orc.check(out, want.float())
    assert dec.peer.error() == 0


def test_peer_exchange_a_record_that_never_arrives_is_reported_not_waited_for():
    """The merge's wait is bounded: with no push before it (the flag of this step is never raised) it
    gives up after `spin_limit` polls, sets the error word to 1 + the missing rank, leaves `out`
    alone and returns; the GPU and the context stay usable, and after `reset` a whole step works."""
    from hk_dsl_b200.ops import paged_dist

    spec = W.CONFIGS["c5"]
    st = W.build_step(spec, "cuda", lens=[600, 100])
    n, hq, d = st.query.shape
    dec = paged_dist.SplitKVDecoder(n, hq, st.kv_heads, d, "cuda", local_splits=4, exchange="peer")
    out = torch.full_like(st.out, 7.0)
    dec.peer.merge(out, spin_limit=200)                     # nothing was pushed
    torch.cuda.synchronize()
    assert dec.peer.error() == 1                            # rank 0's record was the one missing
    assert (out == 7.0).all()
    dec.peer.reset()
    torch.cuda.synchronize()
    dec.decode(out, st.query, st.k_caches[0], st.v_caches[0], st.block_table, st.seq_lens, st.scale,
               key=st.key, value=st.value, slot_mapping=st.slot_mapping)
    torch.cuda.synchronize()
    assert dec.peer.error() == 0
    orc.check(out, _oracle(st))


def test_peer_exchange_in_one_launch_gives_up_on_rows_that_never_arrive():
    """hkb_kvsplit_exchange waits for a flag a (rank, row). Here this rank is told it is rank 0 of two whose
    second rank is itself (both peers' buffers are its own) -- so nobody ever raises rank 1's flags: every
    CTA gives up after `spin_limit` polls, the error word reads 1 + 1, `out` is untouched, the context stays
    usable, and after `reset` a whole step with the true single rank works."""
    from hk_dsl_b200.ops import paged_dist
    from hk_dsl_b200.runtime import lib as hkb

    spec = W.CONFIGS["c5"]
    st = W.build_step(spec, "cuda", lens=[600, 100])
    n, hq, d = st.query.shape
    dec = paged_dist.SplitKVDecoder(n, hq, st.kv_heads, d, "cuda", local_splits=4, exchange="peer")
    out = torch.full_like(st.out, 7.0)
    dec.walk(st.query, st.k_caches[0], st.v_caches[0], st.block_table, st.seq_lens, st.scale)
    lib = hkb.load()
    # a gather buffer sized for two ranks, beside a state block of its own
    gbytes = lib.hkb_exchange_gather_bytes(2, n, hq, d)
    sbytes = lib.hkb_exchange_state_bytes_rows(n, hq)
    buf = torch.zeros(gbytes + 256 + sbytes, dtype=torch.uint8, device="cuda")
    x = hkb.ExchangeT()
    x.world, x.rank = 2, 0
    for r in range(2):
        x.gather[r] = buf.data_ptr()
        x.state[r] = buf.data_ptr() + (gbytes + 255) // 256 * 256
    po, pl = dec.scratch
    rc = lib.hkb_kvsplit_exchange(x, po.data_ptr(), pl.data_ptr(), dec.local_splits, out.data_ptr(), out.stride(0),
                                  out.stride(1), 0, n, hq, d, 200, torch.cuda.current_stream().cuda_stream)
    hkb.check("hkb_kvsplit_exchange", rc)
    torch.cuda.synchronize()
    state = buf[(gbytes + 255) // 256 * 256:][:80].view(torch.int32)
    assert int(state[19].item()) == 2                       # rank 1's rows were the ones missing
    assert int(state[16].item()) == 1 and int(state[17].item()) == 0   # the step counter moved on, the CTA counter is back at zero
    assert (out == 7.0).all()
    dec.decode(out, st.query, st.k_caches[0], st.v_caches[0], st.block_table, st.seq_lens, st.scale,
               key=st.key, value=st.value, slot_mapping=st.slot_mapping)
    torch.cuda.synchronize()
    assert dec.peer.error() == 0
    orc.check(out, _oracle(st))
