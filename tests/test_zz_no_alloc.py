"""The split decode on the library's built-in scratch (hkb_paged_decode_static), called through
the C ABI and held to the caller-scratch entry points on the same inputs.

That entry point exists for hosts that cannot allocate device memory when they decode: a
binding that only holds the pointers its engine gave it (no allocator bridge across cgo / JNI),
or a serving loop running after the engine has handed the whole GPU to its KV pool. The file
is named to be collected last, so a failure here cannot hide any other test's result, and it
keeps no state of its own: it passes alone in a fresh process and after the rest of the suite.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lens, hkv=2, group=4, d=128, page=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    pages = [max(1, -(-n // page)) for n in lens]
    nb = sum(pages) + 3
    k = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(nb, hkv, page, d, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(nb, generator=g)
    table = torch.zeros(len(lens), max(pages), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages):
        table[i, :n] = perm[at:at + n].to(torch.int32)
        at += n
    q = torch.randn(len(lens), hkv * group, d, generator=g).to(torch.bfloat16).cuda()
    return q, k, v, table.cuda(), torch.tensor(lens, dtype=torch.int32).cuda()


def _static(lib, out, q, k, v, table, lens, splits):
    """hkb_paged_decode_static through ctypes: head-major caches as (blocks, page, heads, d) strides."""
    from hk_dsl_b200.runtime.lib import CacheT

    n, hq, d = q.shape
    cache = lambda c: CacheT(c.data_ptr(), c.stride(0), c.stride(2), c.stride(1), c.shape[0])
    return lib.hkb_paged_decode_static(
        out.data_ptr(), out.stride(0), out.stride(1), q.data_ptr(), q.stride(0), q.stride(1), cache(k), cache(v),
        table.data_ptr(), table.stride(0), table.shape[1], lens.data_ptr(), None, n, hq, k.shape[1], d, k.shape[2],
        d ** -0.5, 0, None, None, splits, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("group", [4, 8])
def test_built_in_scratch_matches_caller_scratch_on_two_calls_in_a_row(group):
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb

    lib = hkb.load()
    splits = 8
    # the second call is smaller and has an empty request: whatever the first left in the array must not leak
    for seed, lens in ((1, [64, 300, 512, 1000, 17]), (2, [33, 0, 129])):
        q, k, v, table, lens_t = _case(lens, group=group, seed=seed)
        want = torch.empty_like(q)
        paged.paged_attention_decode(want, q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t, q.shape[-1] ** -0.5,
                                     num_splits=splits)
        got = torch.full_like(q, 7.0)
        rc = _static(lib, got, q, k, v, table, lens_t, splits)
        assert rc == 0, hkb.strerror(rc)
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs()
        # the suite's decode tolerance (max-abs 2e-2, mean-abs 2e-3); the two paths run the same kernels
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3
        assert torch.isfinite(got.float()).all()
        if 0 in lens:
            assert (got[lens.index(0)] == 0).all()


def test_one_split_passes_through_and_oversize_is_refused_before_any_launch():
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb

    lib = hkb.load()
    q, k, v, table, lens_t = _case([200, 31], seed=3)
    want = torch.empty_like(q)
    paged.paged_attention_decode(want, q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t, q.shape[-1] ** -0.5,
                                 num_splits=1)
    got = torch.empty_like(q)
    assert _static(lib, got, q, k, v, table, lens_t, 1) == 0
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    # 2 sequences x 256 splits x 8 heads x (128 + 1) floats fits; a batch whose partials exceed 8 MiB does not
    n, hq, d = 64, 32, 128
    assert lib.hkb_scratch_bytes(n, hq, d, 16) > hkb.STATIC_SCRATCH_BYTES
    big_q = torch.zeros(n, hq, d, device="cuda", dtype=torch.bfloat16)
    big_k = torch.zeros(4, 8, 16, d, device="cuda", dtype=torch.bfloat16)
    out = torch.full_like(big_q, 7.0)
    rc = _static(lib, out, big_q, big_k, big_k, torch.zeros(n, 1, dtype=torch.int32, device="cuda"),
                 torch.ones(n, dtype=torch.int32, device="cuda"), 16)
    assert rc == hkb.ERR_STATIC_SCRATCH
    assert "built-in scratch" in hkb.strerror(rc)
    torch.cuda.synchronize()
    assert (out == 7.0).all()          # nothing was launched
