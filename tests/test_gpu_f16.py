"""float16 throughout (a model served in float16: the reference's `_f16` kernel variants,
python/hk/ops/paged.py:706-729): the cache, the new rows, the query and the output are fp16. The
cache write is the same 16-bit copy, the walk runs on the tensor-core worker with f16 mma at every
GQA group, the merge and the prefill write fp16. Same oracle, same tolerances as bf16."""

import pytest
import torch

from oracle import paged_oracle as orc
from test_gpu_decode import LENS, _case, _check, _cuda

pytestmark = pytest.mark.gpu


def _paged():
    from hk_dsl_b200.ops import paged
    return paged


def _half(c):
    return {n: (t.to(torch.float16) if isinstance(t, torch.Tensor) and t.dtype == torch.bfloat16 else t) for n, t in c.items()}


@pytest.mark.parametrize("splits", [1, 4, 32])
@pytest.mark.parametrize("group,h_kv,d", [(1, 4, 128), (2, 4, 128), (4, 8, 128), (8, 2, 128), (16, 1, 128), (4, 2, 64), (2, 2, 256)])
def test_decode_in_float16(splits, group, h_kv, d):
    paged = _paged()
    c = _half(_case(LENS, head_dim=d, h_kv=h_kv, group=group, seed=splits + group))
    g = _cuda(c)
    out = torch.empty_like(g["q"])
    assert out.dtype == torch.float16
    paged.paged_attention_decode(out, g["q"], g["k"].transpose(1, 2), g["v"].transpose(1, 2), g["table"], g["lens"],
                                 d ** -0.5, "auto", num_splits=splits)
    want = orc.paged_decode_ref(c["q"], c["k"].transpose(1, 2), c["v"].transpose(1, 2), c["table"], c["lens"])
    _check(out.float().cpu(), want)


def test_step_in_float16_writes_the_cache_and_decodes():
    paged = _paged()
    lens = [5, 700, 33, 2048, 1, 16]
    c = _half(_case(lens, h_kv=8, group=4, seed=3))
    g = _cuda(c)
    n, hkv, d = len(lens), 8, 128
    gen = torch.Generator().manual_seed(5)
    key = torch.randn(n, hkv, d, generator=gen).to(torch.float16)
    value = torch.randn(n, hkv, d, generator=gen).to(torch.float16)
    slots = torch.tensor([int(c["table"][i, (s - 1) // 16]) * 16 + (s - 1) % 16 for i, s in enumerate(lens)])
    k_want, v_want = c["k"].clone(), c["v"].clone()
    k_want[slots // 16, :, slots % 16] = key
    v_want[slots // 16, :, slots % 16] = value
    # separate launches, then the joined step on a second copy of the cache
    k1, v1 = g["k"].clone(), g["v"].clone()
    paged.reshape_and_cache(key.cuda(), value.cuda(), k1.transpose(1, 2), v1.transpose(1, 2), slots.cuda(), "auto")
    assert torch.equal(k1.cpu(), k_want) and torch.equal(v1.cpu(), v_want)
    o1 = torch.empty_like(g["q"])
    paged.paged_attention_decode(o1, g["q"], k1.transpose(1, 2), v1.transpose(1, 2), g["table"], g["lens"], d ** -0.5,
                                 num_splits=8)
    o2 = torch.empty_like(g["q"])
    paged.decode_step(o2, g["q"], key.cuda(), value.cuda(), g["k"].transpose(1, 2), g["v"].transpose(1, 2), slots.cuda(),
                      g["table"], g["lens"], d ** -0.5, num_splits=8,
                      arrivals=paged.step_arrivals(n, hkv, "cuda"))      # counters given: fp16 keeps the merge launch
    assert torch.equal(g["k"].cpu(), k_want) and torch.equal(g["v"].cpu(), v_want)
    assert torch.equal(o1, o2)
    want = orc.paged_decode_ref(c["q"], k_want.transpose(1, 2), v_want.transpose(1, 2), c["table"], c["lens"])
    _check(o2.float().cpu(), want)


@pytest.mark.parametrize("group,h_kv,d", [(4, 2, 128), (8, 1, 128), (1, 2, 128), (2, 2, 64)])
def test_prefill_in_float16(group, h_kv, d):
    paged = _paged()
    reqs = [(0, 70), (100, 33), (513, 1), (0, 257)]
    page = 16
    gen = torch.Generator().manual_seed(group)
    seq = [c + n for c, n in reqs]
    pages = [-(-s // page) for s in seq]
    nb = sum(pages) + 3
    k = torch.randn(nb, h_kv, page, d, generator=gen).to(torch.float16)
    v = torch.randn(nb, h_kv, page, d, generator=gen).to(torch.float16)
    perm = torch.randperm(nb, generator=gen)
    table = torch.zeros(len(reqs), max(pages), dtype=torch.int32)
    at = 0
    for i, p in enumerate(pages):
        table[i, :p] = perm[at:at + p].to(torch.int32)
        at += p
    starts = [0]
    for _, n in reqs:
        starts.append(starts[-1] + n)
    q = torch.randn(starts[-1], h_kv * group, d, generator=gen).to(torch.float16)
    lens_t, qsl = torch.tensor(seq, dtype=torch.int32), torch.tensor(starts, dtype=torch.int32)
    out = torch.empty_like(q, device="cuda")
    work = paged.work_list([(r, n) for r, (_, n) in enumerate(reqs)], paged.prefill_tile_rows(h_kv * group, h_kv), "cuda")
    paged.paged_prefill(out, q.cuda(), k.cuda().transpose(1, 2), v.cuda().transpose(1, 2), table.cuda(), lens_t.cuda(),
                        qsl.cuda(), work, d ** -0.5)
    want = orc.paged_prefill_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t, qsl)
    _check(out.float().cpu(), want)


def test_float16_refusals():
    paged = _paged()
    c = _cuda(_half(_case([40, 300], h_kv=2, group=4)))
    out = torch.empty_like(c["q"])
    fp8 = torch.zeros(c["k"].shape, device="cuda", dtype=torch.uint8)
    one = torch.ones(1, device="cuda")
    with pytest.raises(TypeError, match="bfloat16 activations"):
        paged.paged_attention_decode(out, c["q"], fp8.transpose(1, 2), fp8.transpose(1, 2), c["table"], c["lens"], 0.1,
                                     "fp8", one, one)
    with pytest.raises(TypeError, match="keeps the cache in"):
        paged.paged_attention_decode(out, c["q"], c["k"].to(torch.bfloat16).transpose(1, 2),
                                     c["v"].to(torch.bfloat16).transpose(1, 2), c["table"], c["lens"], 0.1)
    with pytest.raises(ValueError, match="match query"):
        paged.paged_attention_decode(out.to(torch.bfloat16), c["q"], c["k"].transpose(1, 2), c["v"].transpose(1, 2),
                                     c["table"], c["lens"], 0.1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("group,h_kv", [(2, 2), (8, 1), (1, 2)])
def test_prefill_at_head_dim_256(dtype, group, h_kv):
    """512-byte rows in the prefill kernel: one (query tile, head) unit a warp, eight warps a CTA."""
    paged = _paged()
    d, page = 256, 16
    reqs = [(0, 70), (100, 33), (513, 1), (0, 257)]
    gen = torch.Generator().manual_seed(group)
    seq = [c + n for c, n in reqs]
    pages = [-(-s // page) for s in seq]
    nb = sum(pages) + 3
    k = torch.randn(nb, h_kv, page, d, generator=gen).to(dtype)
    v = torch.randn(nb, h_kv, page, d, generator=gen).to(dtype)
    perm = torch.randperm(nb, generator=gen)
    table = torch.zeros(len(reqs), max(pages), dtype=torch.int32)
    at = 0
    for i, p in enumerate(pages):
        table[i, :p] = perm[at:at + p].to(torch.int32)
        at += p
    starts = [0]
    for _, n in reqs:
        starts.append(starts[-1] + n)
    q = torch.randn(starts[-1], h_kv * group, d, generator=gen).to(dtype)
    lens_t, qsl = torch.tensor(seq, dtype=torch.int32), torch.tensor(starts, dtype=torch.int32)
    out = torch.empty_like(q, device="cuda")
    work = paged.work_list([(r, n) for r, (_, n) in enumerate(reqs)], paged.prefill_tile_rows(h_kv * group, h_kv), "cuda")
    paged.paged_prefill(out, q.cuda(), k.cuda().transpose(1, 2), v.cuda().transpose(1, 2), table.cuda(), lens_t.cuda(),
                        qsl.cuda(), work, d ** -0.5)
    want = orc.paged_prefill_ref(q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t, qsl)
    _check(out.float().cpu(), want)
