"""The decode step in two launches or one (`paged.decode_step`: the cache write inside the walk;
with arrival counters the fold inside it too) against the separate launches and the float64 oracle.

hk-dsl's decode step is a cache write and two launches (python/hk/integration/vllm_backend.py:
582-599, 700-729) and its record lists joining them as what is left
(docs/history/17-the-decode-step-captured-whole.md:181-188); there is no reference test for the
joined form, so the cases here hold it to the separate form's results: the cache bit for bit
(tests/hk/gpu/test_vllm_backend_decode.py:44-49 is the scatter's specification), the output bit
for bit while a sequence has at most 16 pieces and within the decode tolerances beyond.
"""

import pytest
import torch

from oracle import paged_oracle as orc
from test_gpu_decode import _case, _check, _cuda

pytestmark = pytest.mark.gpu

PAGE = 16


def _paged():
    from hk_dsl_b200.ops import paged
    return paged


def _step_case(lens, seed=0, now=None, **kw):
    """A decode step over `_case`'s tables: the cache holds every position but the last of each
    sequence (poisoned there), and key/value/slots carry that last position. `now`: the lengths
    this step runs at, inside the tables built for `lens` (the same pool at other lengths)."""
    c = _case(lens, seed=seed, **kw)
    if now is not None:
        assert len(now) == len(lens) and all(a <= b for a, b in zip(now, lens))
        c["lens"][: len(now)] = torch.tensor(now, dtype=torch.int32)
        lens = now
    fp8 = c["ks"] is not None
    r = len(lens)
    hkv, d = c["k"].shape[1], c["k"].shape[3]
    g = torch.Generator().manual_seed(1000 + seed)
    n_rows = c["q"].shape[0]
    key = torch.randn(n_rows, hkv, d, generator=g).to(torch.bfloat16)
    value = torch.randn(n_rows, hkv, d, generator=g).to(torch.bfloat16)
    slots = torch.full((n_rows,), -1, dtype=torch.int64)
    for i, s in enumerate(lens):
        if s > 0:
            slots[i] = int(c["table"][i, (s - 1) // PAGE]) * PAGE + (s - 1) % PAGE
    # what the cache must hold after the step: the torch scatter of the reference's test
    k_want, v_want = c["k"].clone(), c["v"].clone()       # (blocks, kv heads, page, d) storage
    live = slots >= 0
    blk, off = slots[live] // PAGE, slots[live] % PAGE
    if fp8:
        k_want[blk, :, off] = orc.quantize_fp8(key[live], c["ks"])
        v_want[blk, :, off] = orc.quantize_fp8(value[live], c["vs"])
    else:
        k_want[blk, :, off] = key[live]
        v_want[blk, :, off] = value[live]
    # before the step those rows hold something else
    k0, v0 = c["k"].clone(), c["v"].clone()
    if fp8:
        k0.view(torch.uint8)[blk, :, off] = 0x55
        v0.view(torch.uint8)[blk, :, off] = 0x55
    else:
        k0[blk, :, off] = 7.0
        v0[blk, :, off] = -7.0
    c.update(key=key, value=value, slots=slots, k_want=k_want, v_want=v_want, k=k0, v=v0)
    return c


def _want(c):
    return orc.paged_decode_ref(c["q"], c["k_want"].transpose(1, 2), c["v_want"].transpose(1, 2), c["table"], c["lens"],
                                None, c["ks"], c["vs"], None)


def _separate(g, c, splits, with_q_start=False):
    paged = _paged()
    k, v = g["k"].clone(), g["v"].clone()
    kv = "fp8" if c["ks"] is not None else "auto"
    paged.reshape_and_cache(g["key"], g["value"], k.transpose(1, 2), v.transpose(1, 2), g["slots"], kv, g["ks"], g["vs"])
    o = torch.full(g["q"].shape, 3.0, device="cuda", dtype=torch.bfloat16)
    paged.paged_attention_decode(o, g["q"], k.transpose(1, 2), v.transpose(1, 2), g["table"], g["lens"],
                                 g["q"].shape[-1] ** -0.5, kv, g["ks"], g["vs"], num_splits=splits,
                                 query_start_loc=g["q_start"] if with_q_start else None)
    return o, k, v


def _joined(g, c, splits, with_q_start=False, arrivals=None, scratch=None, write=True, fold=True):
    paged = _paged()
    k, v = g["k"].clone(), g["v"].clone()
    kv = "fp8" if c["ks"] is not None else "auto"
    o = torch.full(g["q"].shape, 3.0, device="cuda", dtype=torch.bfloat16)
    n, hkv = g["lens"].shape[0], g["k"].shape[1]
    arrivals = paged.step_arrivals(n, hkv, "cuda") if arrivals is None and fold else arrivals
    paged.decode_step(o, g["q"], g["key"] if write else None, g["value"] if write else None, k.transpose(1, 2),
                      v.transpose(1, 2), g["slots"] if write else None, g["table"], g["lens"], g["q"].shape[-1] ** -0.5,
                      kv, g["ks"], g["vs"], num_splits=splits, scratch=scratch, arrivals=arrivals,
                      query_start_loc=g["q_start"] if with_q_start else None)
    torch.cuda.synchronize()
    assert arrivals is None or int(arrivals.abs().sum()) == 0, "the step must leave its counters zero"
    return o, k, v


def _bits(t):
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t.view(torch.int16)


LENS = [1, 15, 16, 33, 1000, 2063, 4100]


@pytest.mark.parametrize("splits", [2, 4, 16])
@pytest.mark.parametrize("group,h_kv,fp8", [(4, 8, False), (4, 2, True), (8, 2, False), (8, 1, True), (1, 4, False),
                                            (2, 4, False), (3, 2, False), (6, 2, False), (16, 1, False)])
def test_one_launch_equals_the_separate_launches(splits, group, h_kv, fp8):
    c = _step_case(LENS, seed=splits + group, h_kv=h_kv, group=group, fp8=fp8)
    g = _cuda(c)
    o1, k1, v1 = _separate(g, c, splits)
    assert torch.equal(_bits(k1), _bits(g["k_want"])) and torch.equal(_bits(v1), _bits(g["v_want"]))
    for fold in (False, True):       # two launches (write in the walk, merge kernel); one (fold on arrival too)
        o2, k2, v2 = _joined(g, c, splits, fold=fold)
        assert torch.equal(_bits(k2), _bits(g["k_want"])), "K cache after the joined step"
        assert torch.equal(_bits(v2), _bits(g["v_want"])), "V cache after the joined step"
        assert torch.equal(o1.view(torch.int16), o2.view(torch.int16)), "at most 16 pieces a sequence: the merge kernel's bits"
        _check(o2.cpu(), _want(c))


@pytest.mark.parametrize("head_dim", [64, 256])
@pytest.mark.parametrize("group,h_kv", [(4, 2), (8, 1)])
def test_fp8_step_at_head_sizes_64_and_256(head_dim, group, h_kv):
    """The step's quantised cache write inside the walk, and its answer, at fp8 rows of 64 and 256 bytes."""
    c = _step_case(LENS, seed=head_dim + group, head_dim=head_dim, h_kv=h_kv, group=group, fp8=True)
    g = _cuda(c)
    o1, k1, v1 = _separate(g, c, 4)
    assert torch.equal(_bits(k1), _bits(g["k_want"])) and torch.equal(_bits(v1), _bits(g["v_want"]))
    o2, k2, v2 = _joined(g, c, 4, fold=False)
    assert torch.equal(_bits(k2), _bits(g["k_want"])) and torch.equal(_bits(v2), _bits(g["v_want"]))
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
    _check(o2.cpu(), _want(c))


@pytest.mark.parametrize("splits", [64, 256])
@pytest.mark.parametrize("group,h_kv", [(4, 2), (8, 1)])
def test_many_pieces_fold_as_a_tree(splits, group, h_kv):
    """One long sequence over hundreds of rings: more than 16 pieces, so group folds then the fold of the groups."""
    c = _step_case([16 * 1024 + 5, 700], seed=splits, h_kv=h_kv, group=group)
    g = _cuda(c)
    o2, k2, v2 = _joined(g, c, splits)
    assert torch.equal(_bits(k2), _bits(g["k_want"])) and torch.equal(_bits(v2), _bits(g["v_want"]))
    _check(o2.cpu(), _want(c))
    o1, _, _ = _separate(g, c, splits)
    assert (o1.float() - o2.float()).abs().max() <= 2 ** -7, "tree fold against the flat merge: rounding only"


def test_counters_scratch_and_caches_are_reusable_step_after_step():
    paged = _paged()
    c = _step_case(LENS, seed=5, h_kv=8, group=4)
    g = _cuda(c)
    n, hq, d = g["q"].shape[0], g["q"].shape[1], g["q"].shape[2]
    arrivals = paged.step_arrivals(n, 8, "cuda")
    scratch = paged.split_scratch(n, hq, d, 8, "cuda")
    scratch[0].fill_(float("nan"))
    scratch[1].fill_(float("nan"))
    first = None
    for _ in range(20):
        o, k, v = _joined(g, c, 8, arrivals=arrivals, scratch=scratch)
        first = o if first is None else first
        assert torch.equal(o, first)
    _check(first.cpu(), _want(c))


def test_without_new_rows_only_the_fold_is_joined():
    c = _step_case(LENS, seed=9, h_kv=8, group=4)
    c["k"], c["v"] = c["k_want"].clone(), c["v_want"].clone()      # the engine wrote the cache itself
    g = _cuda(c)
    o, k, v = _joined(g, c, 8, write=False)
    assert torch.equal(_bits(k), _bits(g["k_want"]))
    _check(o.cpu(), _want(c))


def test_padding_and_empty_sequences():
    """Graph padding: requests with no query (query_start_loc repeats) write nothing; a sequence of
    length 0 with a query row answers zero; a slot of -1 leaves the cache alone."""
    c = _step_case([40, 0, 1000, 17], seed=3, h_kv=8, group=4, pad=3)
    g = _cuda(c)
    o, k, v = _joined(g, c, 4, with_q_start=True)
    assert torch.equal(_bits(k), _bits(g["k_want"])) and torch.equal(_bits(v), _bits(g["v_want"]))
    want = orc.paged_decode_ref(c["q"], c["k_want"].transpose(1, 2), c["v_want"].transpose(1, 2), c["table"], c["lens"],
                                None, None, None, c["q_start"])
    _check(o[[0, 2, 3]].cpu(), want[[0, 2, 3]])
    assert float(o[1].abs().max()) == 0.0
    assert torch.all(o[4:] == 3.0), "rows of padded requests are not written"


def test_vllm_layouts():
    """vLLM's token-major cache and its K|V side-by-side tensor, through strides."""
    paged = _paged()
    c = _step_case([5, 700, 33, 2048, 1, 16], seed=2, h_kv=8, group=4)
    g = _cuda(c)
    nb = g["k"].shape[0]
    both = torch.empty(2, nb, PAGE, 8, 128, device="cuda", dtype=torch.bfloat16)        # (2, blocks, block, heads, d)
    both[0].copy_(g["k"].transpose(1, 2))
    both[1].copy_(g["v"].transpose(1, 2))
    kc, vc = both.unbind(0)
    o = torch.empty_like(g["q"])
    paged.decode_step(o, g["q"], g["key"], g["value"], kc, vc, g["slots"].to(torch.int32), g["table"], g["lens"],
                      128 ** -0.5, num_splits=4)
    assert torch.equal(kc, g["k_want"].transpose(1, 2)) and torch.equal(vc, g["v_want"].transpose(1, 2))
    _check(o.cpu(), _want(c))


def test_one_split_and_bad_arguments():
    paged = _paged()
    c = _step_case([40, 300], seed=4, h_kv=2, group=4)
    g = _cuda(c)
    o, k, v = _joined(g, c, 1)                                   # one split: write launch + walk, no partials
    assert torch.equal(_bits(k), _bits(g["k_want"]))
    _check(o.cpu(), _want(c))
    with pytest.raises(ValueError, match="together"):
        paged.decode_step(o, g["q"], g["key"], None, k.transpose(1, 2), v.transpose(1, 2), g["slots"], g["table"],
                          g["lens"], 0.1)
    with pytest.raises(ValueError, match="arrivals"):
        paged.decode_step(o, g["q"], g["key"], g["value"], k.transpose(1, 2), v.transpose(1, 2), g["slots"], g["table"],
                          g["lens"], 0.1, num_splits=4, arrivals=torch.zeros(3, dtype=torch.int32, device="cuda"))


def test_captured_in_a_cuda_graph_and_replayed_over_new_lengths():
    paged = _paged()
    c = _step_case([100, 900, 33, 2000], seed=6, h_kv=8, group=4)
    g = _cuda(c)
    n, hq, d = g["q"].shape
    arrivals = paged.step_arrivals(n, 8, "cuda")
    scratch = paged.split_scratch(n, hq, d, 8, "cuda")
    k, v = g["k"].clone(), g["v"].clone()
    o = torch.empty_like(g["q"])
    lens, slots = g["lens"].clone(), g["slots"].clone()

    def step():
        paged.decode_step(o, g["q"], g["key"], g["value"], k.transpose(1, 2), v.transpose(1, 2), slots, g["table"], lens,
                          d ** -0.5, num_splits=8, scratch=scratch, arrivals=arrivals)

    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for now in (None, [64, 17, 20, 1999], [100, 1, 33, 16]):
        c2 = _step_case([100, 900, 33, 2000], seed=6, now=now, h_kv=8, group=4)   # same pool and tables
        g2 = _cuda(c2)
        k.copy_(g2["k"]); v.copy_(g2["v"])
        lens.copy_(g2["lens"]); slots.copy_(g2["slots"])
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(_bits(k), _bits(g2["k_want"])) and torch.equal(_bits(v), _bits(g2["v_want"]))
        _check(o.cpu(), _want(c2))
        assert int(arrivals.abs().sum()) == 0


def test_as_a_torch_op():
    """`torch.ops.hk.paged_decode_step`: the flat signature, caches and scratch as written arguments."""
    from hk_dsl_b200.runtime import torch_ext

    paged = _paged()
    torch_ext.paged_decode_step_op()
    c = _step_case([5, 700, 33, 2048], seed=8, h_kv=8, group=4)
    g = _cuda(c)
    n, hq, d = g["q"].shape
    po, pl = paged.split_scratch(n, hq, d, 4, "cuda")
    one = torch.ones(1, device="cuda")
    k, v = g["k"].clone(), g["v"].clone()
    o = torch.empty_like(g["q"])
    r = torch.ops.hk.paged_decode_step(o, g["q"], g["key"], g["value"], k.transpose(1, 2), v.transpose(1, 2), g["slots"],
                                       g["table"], g["lens"], d ** -0.5, "auto", one, one, 4, po, pl)
    assert r is None
    assert torch.equal(_bits(k), _bits(g["k_want"])) and torch.equal(_bits(v), _bits(g["v_want"]))
    _check(o.cpu(), _want(c))


@pytest.mark.parametrize("n", [2048, 2100])
def test_batches_at_and_past_the_streams_sequence_limit(n):
    """2048 sequences is the most the persistent stream keeps a prefix table for; one more batch
    size up, the same calls run on the fixed-split grid and the step on its three separate launches.
    Same answers, same cache, either side of the limit."""
    g0 = torch.Generator().manual_seed(n)
    lens = torch.randint(1, 48, (n,), generator=g0).tolist()
    c = _step_case(lens, seed=n % 97, h_kv=2, group=4)
    g = _cuda(c)
    o1, k1, v1 = _separate(g, c, 2)
    o2, k2, v2 = _joined(g, c, 2, fold=False)
    o3, k3, v3 = _joined(g, c, 2, fold=True)
    for k, v in ((k1, v1), (k2, v2), (k3, v3)):
        assert torch.equal(_bits(k), _bits(g["k_want"])) and torch.equal(_bits(v), _bits(g["v_want"]))
    want = _want(c)
    for o in (o1, o2, o3):
        _check(o.cpu(), want)


@pytest.mark.parametrize("name", ["c2", "c3", "c4"])
def test_full_size_configs_step_equals_separate_launches(name):
    """At the measured configurations' full sizes (no oracle needed): the two-launch step leaves the
    same cache and the same answer, bit for bit, as cache write + walk + merge launched separately."""
    from hk_dsl_b200 import workloads as W

    paged = _paged()
    spec = W.CONFIGS[name]
    st = W.build_step(spec, "cuda")
    k0, v0 = st.k_caches[0], st.v_caches[0]
    # the step's slots hold something else before it runs
    key = torch.randn(st.key.shape, device="cuda").to(torch.bfloat16)
    value = torch.randn(st.value.shape, device="cuda").to(torch.bfloat16)
    ka, va = k0.clone(), v0.clone()
    paged.reshape_and_cache(key, value, ka, va, st.slot_mapping, spec.kv_cache_dtype, st.k_scale, st.v_scale)
    o1 = torch.empty_like(st.out)
    paged.paged_attention_decode(o1, st.query, ka, va, st.block_table, st.seq_lens, st.scale, spec.kv_cache_dtype,
                                 st.k_scale, st.v_scale)
    o2 = torch.empty_like(st.out)
    paged.decode_step(o2, st.query, key, value, k0, v0, st.slot_mapping, st.block_table, st.seq_lens, st.scale,
                      spec.kv_cache_dtype, st.k_scale, st.v_scale)
    torch.cuda.synchronize()
    assert torch.equal(_bits(k0), _bits(ka)) and torch.equal(_bits(v0), _bits(va))
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16))
