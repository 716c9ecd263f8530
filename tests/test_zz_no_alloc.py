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


def _static(lib, out, q, k, v, table, lens, splits, q_start=None, kv_dtype=0, k_scale=None, v_scale=None):
    """hkb_paged_decode_static through ctypes: head-major caches as (blocks, page, heads, d) strides."""
    from hk_dsl_b200.runtime.lib import CacheT

    n, (_, hq, d) = lens.shape[0], q.shape
    cache = lambda c: CacheT(c.data_ptr(), c.stride(0), c.stride(2), c.stride(1), c.shape[0])
    return lib.hkb_paged_decode_static(
        out.data_ptr(), out.stride(0), out.stride(1), q.data_ptr(), q.stride(0), q.stride(1), cache(k), cache(v),
        table.data_ptr(), table.stride(0), table.shape[1], lens.data_ptr(),
        q_start.data_ptr() if q_start is not None else None, n, hq, k.shape[1], d, k.shape[2],
        d ** -0.5, kv_dtype, k_scale.data_ptr() if k_scale is not None else None,
        v_scale.data_ptr() if v_scale is not None else None, splits, torch.cuda.current_stream().cuda_stream)


def _oracle(q, k, v, table, lens, k_scale=None, v_scale=None, q_start=None):
    """The float64 oracle on host copies (caches as (blocks, page, heads, d) views)."""
    from oracle import paged_oracle as orc

    return orc.paged_decode_ref(q.cpu(), k.transpose(1, 2).cpu(), v.transpose(1, 2).cpu(), table.cpu(), lens.cpu(), None,
                                k_scale.cpu() if k_scale is not None else None,
                                v_scale.cpu() if v_scale is not None else None,
                                q_start.cpu() if q_start is not None else None)


@pytest.mark.parametrize("group", [4, 8])
def test_built_in_scratch_matches_caller_scratch_on_two_calls_in_a_row(group):
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb
    from oracle import paged_oracle as orc

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
        # the two entry points run the same deterministic kernels on the same inputs: the same bits.
        # (The suite's decode tolerance, max-abs 2e-2 / mean-abs 2e-3, holds a fortiori; a slot
        # left over from the previous call leaking into this one would show up here as a changed bit.)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        # and not only each other: both against the float64 oracle
        orc.check(got, _oracle(q, k, v, table, lens_t))
        orc.check_baseline(got, _oracle(q, k, v, table, lens_t))
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


def test_query_rows_by_q_start_an_fp8_cache_and_a_float16_model():
    """The arguments the first test leaves at their defaults: cu_seqlens_q with a sequence that has no
    query row (it must write nothing), an fp8-e4m3 cache with per-tensor scales, float16 throughout.
    Each against the caller-scratch entry point bit for bit and against the float64 oracle."""
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb
    from oracle import paged_oracle as orc

    lib = hkb.load()
    splits = 4
    # (1) q_start: three sequences, the middle one without a query; q has two rows
    q, k, v, table, lens_t = _case([300, 77, 45], seed=5)
    q = q[:2].contiguous()
    q_start = torch.tensor([0, 1, 1, 2], dtype=torch.int32).cuda()
    want = torch.full_like(q, 3.0)
    paged.paged_attention_decode(want, q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t, q.shape[-1] ** -0.5,
                                 num_splits=splits, query_start_loc=q_start)
    got = torch.full_like(q, 3.0)
    assert _static(lib, got, q, k, v, table, lens_t, splits, q_start=q_start) == 0
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    orc.check(got, _oracle(q, k, v, table, lens_t, q_start=q_start))

    # (2) fp8-e4m3 cache
    q, k, v, table, lens_t = _case([513, 64, 1000], seed=6)
    ks, vs = torch.tensor([0.013]).cuda(), torch.tensor([0.011]).cuda()
    k8 = orc.quantize_fp8(k.cpu(), ks.cpu()).cuda()
    v8 = orc.quantize_fp8(v.cpu(), vs.cpu()).cuda()
    want = torch.empty_like(q)
    paged.paged_attention_decode(want, q, k8.transpose(1, 2), v8.transpose(1, 2), table, lens_t, q.shape[-1] ** -0.5,
                                 "fp8", ks, vs, num_splits=splits)
    got = torch.empty_like(q)
    assert _static(lib, got, q, k8, v8, table, lens_t, splits, kv_dtype=hkb.KV_FP8_E4M3, k_scale=ks, v_scale=vs) == 0
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    orc.check(got, _oracle(q, k8, v8, table, lens_t, ks, vs))

    # (3) float16 throughout
    q, k, v, table, lens_t = _case([200, 31, 900], seed=7)
    q, k, v = q.half(), k.half(), v.half()
    want = torch.empty_like(q)
    paged.paged_attention_decode(want, q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t, q.shape[-1] ** -0.5,
                                 num_splits=splits)
    got = torch.empty_like(q)
    assert _static(lib, got, q, k, v, table, lens_t, splits, kv_dtype=hkb.KV_F16) == 0
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    orc.check(got, _oracle(q, k, v, table, lens_t))


def test_more_sequences_than_the_stream_kernel_takes_still_fit_the_array():
    """Past 2048 sequences the split decode runs its fixed-split grid; with one kv head, a group of 1 and
    head_dim 64 the partials of 2100 sequences x 2 splits fit the 8 MiB array."""
    from hk_dsl_b200.ops import paged
    from hk_dsl_b200.runtime import lib as hkb
    from oracle import paged_oracle as orc

    lib = hkb.load()
    n, splits = 2100, 2
    assert lib.hkb_scratch_bytes(n, 1, 64, splits) <= hkb.STATIC_SCRATCH_BYTES
    lens = [1 + (i * 37) % 90 for i in range(n)]
    q, k, v, table, lens_t = _case(lens, hkv=1, group=1, d=64, seed=8)
    want = torch.empty_like(q)
    paged.paged_attention_decode(want, q, k.transpose(1, 2), v.transpose(1, 2), table, lens_t, 64 ** -0.5,
                                 num_splits=splits)
    got = torch.empty_like(q)
    assert _static(lib, got, q, k, v, table, lens_t, splits) == 0
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    orc.check(got[:64], _oracle(q[:64], k, v, table[:64], lens_t[:64]))
