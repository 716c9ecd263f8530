"""The KV-cache write against the torch scatter, bit for bit, through the C ABI.

Cases follow tests/hk/gpu/test_vllm_backend_decode.py:25-55 of the reference (head-major
pages through a transposed view, every 7th slot -1, cache pre-filled with 7.0) and
examples/09_kv_scatter.py:53-65 (slot -1 dropped), widened to vLLM's NHD layout, K|V side
by side, int32 slots, and the fp8-e4m3 cache this build adds.
"""

import pytest
import torch

from oracle import paged_oracle as orc

pytestmark = pytest.mark.gpu

PAGE = 16


def _paged():
    from hk_dsl_b200.ops import paged
    return paged


def _inputs(n=300, nb=64, hkv=8, d=128, seed=1, every=7):
    g = torch.Generator(device="cuda").manual_seed(seed)
    key = torch.randn(n, hkv, d, device="cuda", dtype=torch.bfloat16, generator=g)
    value = torch.randn(key.shape, device="cuda", dtype=torch.bfloat16, generator=g)
    slots = torch.randperm(nb * PAGE, device="cuda", generator=g)[:n]
    if every:
        slots[::every] = -1
    return key, value, slots


def test_the_cache_write_lands_head_major_and_skips_padding():
    key, value, slots = _inputs()
    nb, hkv, d = 64, 8, 128
    want = torch.full((2, nb, hkv, PAGE, d), 7.0, dtype=torch.bfloat16)
    orc.reshape_and_cache_ref(key.cpu(), value.cpu(), want[0].transpose(1, 2), want[1].transpose(1, 2),
                              slots.cpu())
    got = torch.full((2, nb, hkv, PAGE, d), 7.0, device="cuda", dtype=torch.bfloat16)
    one = torch.ones((), device="cuda", dtype=torch.float32)
    _paged().reshape_and_cache(key, value, got[0].transpose(1, 2), got[1].transpose(1, 2), slots, "auto", one, one)
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("slot_dtype", [torch.int64, torch.int32])
@pytest.mark.parametrize("hkv,d,n", [(8, 128, 300), (2, 64, 17), (1, 128, 1), (4, 128, 1000)])
def test_nhd_layout_bit_exact(slot_dtype, hkv, d, n):
    nb = 80
    key, value, slots = _inputs(n=n, nb=nb, hkv=hkv, d=d, seed=n)
    want_k = torch.full((nb, PAGE, hkv, d), 7.0, dtype=torch.bfloat16)
    want_v = torch.full_like(want_k, -3.0)
    orc.reshape_and_cache_ref(key.cpu(), value.cpu(), want_k, want_v, slots.cpu())
    got_k, got_v = torch.full_like(want_k, 7.0).cuda(), torch.full_like(want_v, -3.0).cuda()
    _paged().reshape_and_cache(key, value, got_k, got_v, slots.to(slot_dtype), "auto")
    assert torch.equal(got_k.cpu().view(torch.int16), want_k.view(torch.int16))
    assert torch.equal(got_v.cpu().view(torch.int16), want_v.view(torch.int16))


def test_k_and_v_side_by_side_in_one_tensor():
    """vLLM's [B, H, N, 2C] cache: K and V are strided slices of the last axis."""
    nb, hkv, d = 40, 4, 128
    key, value, slots = _inputs(n=200, nb=nb, hkv=hkv, d=d, seed=3)
    both = torch.full((nb, hkv, PAGE, 2 * d), 7.0, device="cuda", dtype=torch.bfloat16)
    want = both.cpu().clone()
    orc.reshape_and_cache_ref(key.cpu(), value.cpu(), want[..., :d].transpose(1, 2), want[..., d:].transpose(1, 2),
                              slots.cpu())
    _paged().reshape_and_cache(key, value, both[..., :d].transpose(1, 2), both[..., d:].transpose(1, 2), slots)
    assert torch.equal(both.cpu().view(torch.int16), want.view(torch.int16))


def test_strided_key_rows_of_a_fused_qkv():
    nb, hkv, d, n = 32, 2, 128, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = torch.randn(n, (8 + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16, generator=g)
    key = qkv[:, 8 * d:(8 + hkv) * d].view(n, hkv, d)
    value = qkv[:, (8 + hkv) * d:].view(n, hkv, d)
    slots = torch.randperm(nb * PAGE, device="cuda", generator=g)[:n]
    want_k = torch.zeros(nb, PAGE, hkv, d, dtype=torch.bfloat16)
    want_v = torch.zeros_like(want_k)
    orc.reshape_and_cache_ref(key.cpu(), value.cpu(), want_k, want_v, slots.cpu())
    got_k, got_v = torch.zeros_like(want_k).cuda(), torch.zeros_like(want_v).cuda()
    _paged().reshape_and_cache(key, value, got_k, got_v, slots)
    assert torch.equal(got_k.cpu(), want_k) and torch.equal(got_v.cpu(), want_v)


def test_slots_past_the_pool_are_dropped_not_written():
    nb, hkv, d = 8, 2, 128
    key, value, slots = _inputs(n=32, nb=nb, hkv=hkv, d=d, seed=9, every=0)
    slots[3] = nb * PAGE          # one past the pool
    slots[5] = nb * PAGE + 1000
    guard = torch.full((nb + 2, PAGE, hkv, d), 7.0, device="cuda", dtype=torch.bfloat16)
    kc = guard[1:-1]
    vc = torch.zeros(nb, PAGE, hkv, d, device="cuda", dtype=torch.bfloat16)
    _paged().reshape_and_cache(key, value, kc, vc, slots)
    assert (guard[0] == 7.0).all() and (guard[-1] == 7.0).all()
    live = slots.cpu() < nb * PAGE
    want = torch.full((nb, PAGE, hkv, d), 7.0, dtype=torch.bfloat16)
    s = slots.cpu()[live]
    want[s // PAGE, s % PAGE] = key.cpu()[live]
    assert torch.equal(kc.cpu(), want)


@pytest.mark.parametrize("layout", ["hnd", "nhd"])
def test_fp8_cache_write_bit_exact(layout):
    """RNE(float(x) / scale) saturated at +-448, compared as bytes."""
    nb, hkv, d, n = 64, 8, 128, 500
    key, value, slots = _inputs(n=n, nb=nb, hkv=hkv, d=d, seed=11)
    key = key * 3.0                     # some values saturate
    key[0, 0, 0] = 1e4
    key[1, 0, 0] = -1e4
    key[2, 0, :8] = torch.tensor([0.0, -0.0, 1e-3, -1e-3, 2 ** -9, 2 ** -10, 0.0175, 447.0],
                                 dtype=torch.bfloat16)
    ks = torch.tensor([0.021], device="cuda")
    vs = torch.tensor([0.0133], device="cuda")
    shape = (nb, hkv, PAGE, d) if layout == "hnd" else (nb, PAGE, hkv, d)
    want_k = torch.full(shape, 0x55, dtype=torch.uint8)
    want_v = torch.full(shape, 0x55, dtype=torch.uint8)
    got_k, got_v = want_k.clone().cuda(), want_v.clone().cuda()
    view = (lambda t: t.transpose(1, 2)) if layout == "hnd" else (lambda t: t)
    orc.reshape_and_cache_ref(key.cpu(), value.cpu(), view(want_k), view(want_v), slots.cpu(), "fp8",
                              ks.cpu(), vs.cpu())
    _paged().reshape_and_cache(key, value, view(got_k), view(got_v), slots, "fp8", ks, vs)
    assert torch.equal(got_k.cpu(), want_k)
    assert torch.equal(got_v.cpu(), want_v)
    # the float8 dtype is taken as well as raw bytes
    got2 = torch.full(shape, 0x55, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    got2v = got2.clone()
    _paged().reshape_and_cache(key, value, view(got2), view(got2v), slots, "fp8_e4m3", ks, vs)
    assert torch.equal(got2.view(torch.uint8).cpu(), want_k)


def test_refusals_before_any_launch():
    paged = _paged()
    key, value, slots = _inputs(n=8, nb=4, hkv=2, d=128)
    kc = torch.zeros(4, PAGE, 2, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        paged.reshape_and_cache(key, value, kc[..., :64], kc, slots)
    with pytest.raises(TypeError):
        paged.reshape_and_cache(key, value, kc, kc.clone(), slots.float())
    with pytest.raises(TypeError):
        paged.reshape_and_cache(key, value, kc, kc.clone(), slots, "fp8")           # bf16 cache, fp8 asked
    with pytest.raises(NotImplementedError):
        paged.reshape_and_cache(key, value, kc, kc.clone(), slots, "fp8_e5m2")
    with pytest.raises(RuntimeError):
        paged.reshape_and_cache(key.cpu(), value.cpu(), kc.cpu(), kc.cpu(), slots.cpu())   # no CPU path


@pytest.mark.parametrize("kv", ["auto", "fp8"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_against_vllms_own_cache_write_bit_for_bit(kv, dtype):
    """The arithmetic of the cache write lives in vLLM, not in hk-dsl (its backend calls
    `vllm._custom_ops.reshape_and_cache_flash`, python/hk/integration/vllm_backend.py:594-599): where a
    vLLM is installed beside this build, the two ops must leave the same bytes -- 16-bit caches and,
    which nothing in the reference pins, the fp8-e4m3 cache with per-tensor scales."""
    pytest.importorskip("vllm")
    try:
        from vllm import _custom_ops as vops
        vops.reshape_and_cache_flash  # noqa: B018
        import vllm._C  # noqa: F401  (the compiled ops)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM's compiled cache ops are not usable here: {type(e).__name__}")
    if kv == "fp8" and dtype != torch.bfloat16:
        pytest.skip("an fp8 cache goes with bfloat16 activations in this build")
    paged = _paged()
    key, value, slots = _inputs(n=513, nb=80, seed=11)
    key, value = (key * 3).to(dtype), (value * 3).to(dtype)
    nb, hkv, d = 80, 8, 128
    cache_dtype = torch.uint8 if kv == "fp8" else dtype
    ks, vs = torch.tensor([0.0173], device="cuda"), torch.tensor([0.0221], device="cuda")
    ours = torch.zeros(2, nb, PAGE, hkv, d, device="cuda", dtype=cache_dtype)
    theirs = torch.zeros_like(ours)
    paged.reshape_and_cache(key, value, ours[0], ours[1], slots, kv, ks, vs)
    vops.reshape_and_cache_flash(key, value, theirs[0], theirs[1], slots, kv, ks, vs)
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.uint8), theirs.view(torch.uint8))
    assert int((ours.view(torch.uint8) != 0).sum()) > 0
