"""Paged decode over vLLM's x-split caches, read in place: K (blocks, kv_heads, head_dim / 8, page, 8),
V (blocks, kv_heads, head_dim, page). The reference reads that pair through strided views
(python/hk/ops/paged_prefill.py:768-772) in its `_rocm_decode` route
(python/hk/integration/vllm_prefill.py:1332-1356); its cases are tests/hk/gpu/test_paged_decode.py's
"rocm" layout rows: the length list, GQA shapes, pages that are multiples of 16, NaN past the end.

Each case is also compared, bit for bit, with this build's walk over the same values in the usual
(blocks, page, kv_heads, head_dim) layout at the same split count: the two walks cut the same
tiles and do the same arithmetic in the same order, so a layout bug shows as a changed bit.
"""

import pytest
import torch

from oracle import paged_oracle as orc
from test_gpu_decode import LENS, _case, _check, _cuda, _reference

pytestmark = pytest.mark.gpu


def _both(c, splits, dtype=torch.bfloat16, with_q_start=False):
    from hk_dsl_b200.ops import paged

    g = _cuda(c)
    q = g["q"].to(dtype)
    k, v = g["k"].to(dtype).transpose(1, 2), g["v"].to(dtype).transpose(1, 2)
    k5, v4 = paged.x_split_caches(k, v)
    qs = g["q_start"] if with_q_start else None
    scale = q.shape[-1] ** -0.5
    a = torch.full(q.shape, 7.0, device="cuda", dtype=dtype)
    b = torch.full(q.shape, 7.0, device="cuda", dtype=dtype)
    paged.paged_attention_decode_xsplit(a, q, k5, v4, g["table"], g["lens"], scale, num_splits=splits,
                                        query_start_loc=qs)
    paged.paged_attention_decode(b, q, k, v, g["table"], g["lens"], scale, num_splits=splits, query_start_loc=qs)
    return a, b


@pytest.mark.parametrize("splits", [2, 3, 8, 32])
@pytest.mark.parametrize("group,h_kv", [(4, 8), (8, 2), (16, 1), (1, 2), (6, 2)])
def test_lens_by_splits(splits, group, h_kv):
    c = _case(LENS, h_kv=h_kv, group=group, seed=splits)
    a, b = _both(c, splits)
    _check(a, _reference(c))
    if group >= 4:      # below 4 the usual layout runs the CUDA-core worker: another order of sums
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("page", [32, 48, 64, 256])
def test_pages_of_a_multiple_of_16(page):
    c = _case([1, 33, page - 1, page + 1, 3 * page + 7, 2063], h_kv=2, group=4, page=page, seed=page)
    a, b = _both(c, 4)
    _check(a, _reference(c))
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("group", [4, 8])
def test_nan_past_the_end_is_never_read_into_the_answer(group):
    lens = [1, 7, 8, 9, 15, 17, 33, 1000]
    c = _case(lens, h_kv=2, group=group, nan_tail=True, seed=2)
    clean = _case(lens, h_kv=2, group=group, nan_tail=False, seed=2)
    a, _ = _both(c, 4)
    assert torch.isfinite(a.float()).all()
    _check(a, _reference(clean))


def test_v_of_ones_gives_exactly_one():
    c = _case(LENS, h_kv=2, group=8, v_ones=True)
    a, _ = _both(c, 8)
    assert (a.float() == 1.0).all()


def test_float16_and_graph_padding():
    c = _case([500, 33, 64], h_kv=2, group=4, pad=2, seed=9)
    a, b = _both(c, 4, dtype=torch.float16, with_q_start=True)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    want = orc.paged_decode_ref(c["q"].half(), c["k"].half().transpose(1, 2), c["v"].half().transpose(1, 2),
                                c["table"], c["lens"], None, None, None, c["q_start"])
    orc.check(a[:3], want[:3])
    assert (a[3:] == 7.0).all()        # requests without a query write nothing


def test_what_the_layout_does_not_take_is_refused_before_a_launch():
    from hk_dsl_b200.ops import paged

    c = _cuda(_case([40, 50], h_kv=2, group=4))
    k5, v4 = paged.x_split_caches(c["k"].transpose(1, 2), c["v"].transpose(1, 2))
    out = torch.empty_like(c["q"])
    with pytest.raises(ValueError, match="beside K"):
        paged.paged_attention_decode_xsplit(out, c["q"], k5, v4[:, :1], c["table"], c["lens"], 0.1)
    with pytest.raises(ValueError, match="not contiguous"):
        paged.paged_attention_decode_xsplit(out, c["q"], k5.transpose(2, 3).contiguous().transpose(2, 3), v4,
                                            c["table"], c["lens"], 0.1)
    with pytest.raises(ValueError, match="16-bit"):
        paged.paged_attention_decode_xsplit(out, c["q"], k5.to(torch.float8_e4m3fn), v4.to(torch.float8_e4m3fn),
                                            c["table"], c["lens"], 0.1)
    # a request for one split runs as two: the layout is served by the tile stream only
    paged.paged_attention_decode_xsplit(out, c["q"], k5, v4, c["table"], c["lens"], 128 ** -0.5, num_splits=1)
    orc.check(out, orc.paged_decode_ref(c["q"].cpu(), c["k"].cpu().transpose(1, 2), c["v"].cpu().transpose(1, 2),
                                        c["table"].cpu(), c["lens"].cpu()))
