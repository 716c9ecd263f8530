"""The split planner (python/hk/ops/paged.py:877-914, tests/hk/ir/test_paged_decode_plan.py of
the reference: powers of two, few distinct plans, HK_SPLITS override) and the C-ABI library:
it loads, exports every symbol include/hkb.h declares, and refuses bad arguments without a GPU."""

import ctypes
import os
import re

import pytest

from hk_dsl_b200.ops import paged
from hk_dsl_b200.runtime import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported():
    text = open(os.path.join(ROOT, "include", "hkb.h")).read()
    declared = set(re.findall(r"\b(hkb_[a-z0-9_]+)\s*\(", text))
    declared -= {"hkb_status"}
    assert declared == set(lib.SIGNATURES), (declared ^ set(lib.SIGNATURES))
    loaded = lib.load()
    for name in declared:
        assert getattr(loaded, name) is not None
    assert loaded.hkb_version() == 122


def test_status_text_and_refusals_need_no_gpu():
    l = lib.load()
    assert lib.strerror(0) == "ok" and "unknown" in lib.strerror(-77)
    for code in (-1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -100):
        assert lib.strerror(code) and "unknown" not in lib.strerror(code)
    c = lib.CacheT(16, 2048, 128, 32768, 4)
    # argument checks come before any CUDA call: head_dim 96, block_size 20, group 3/2, NULL pointers
    assert l.hkb_paged_decode(16, 1, 1, 16, 1, 1, c, c, 16, 8, 8, 16, None, 1, 4, 2, 96, 16, 0.1, 0, None, None, 1, None, None, None) == -2
    assert l.hkb_paged_decode(16, 1, 1, 16, 1, 1, c, c, 16, 8, 8, 16, None, 1, 4, 2, 128, 20, 0.1, 0, None, None, 1, None, None, None) == -3
    assert l.hkb_paged_decode(16, 1, 1, 16, 1, 1, c, c, 16, 8, 8, 16, None, 1, 3, 2, 128, 16, 0.1, 0, None, None, 1, None, None, None) == -4
    assert l.hkb_paged_decode(None, 1, 1, 16, 1, 1, c, c, 16, 8, 8, 16, None, 1, 4, 2, 128, 16, 0.1, 0, None, None, 1, None, None, None) == -1
    assert l.hkb_paged_decode(16, 1, 1, 16, 1, 1, c, c, 16, 8, 8, 16, None, 1, 4, 2, 128, 16, 0.1, 1, None, None, 1, None, None, None) == -10
    assert l.hkb_paged_decode(16, 1, 1, 16, 1, 1, c, c, 16, 8, 8, 16, None, 1, 4, 2, 128, 16, 0.1, 0, None, None, 4, None, None, None) == -8
    assert l.hkb_paged_decode(16, 1, 1, 16, 1, 1, c, c, 16, 8, 8, 16, None, 0, 4, 2, 128, 16, 0.1, 0, None, None, 1, None, None, None) == 0
    assert l.hkb_reshape_and_cache(16, 16, 256, 128, 256, 128, c, c, 16, 1, 0, 2, 128, 16, 0, None, None, None) == 0
    assert l.hkb_reshape_and_cache(16, 16, 256, 128, 256, 128, c, c, None, 1, 4, 2, 128, 16, 0, None, None, None) == -1
    assert l.hkb_reshape_and_cache(16, 16, 256, 128, 256, 128, c, c, 16, 1, 4, 2, 128, 16, 7, None, None, None) == -5
    assert l.hkb_merge(16, 128, 128, 0, None, None, 4, 4, 16, 1, 1, 2, 1, 4, 128, None, None, None) == -1
    with pytest.raises(lib.HkbError, match="head_dim"):
        lib.check("hkb_paged_decode", -2)


def test_decode_step_refuses_everything_before_its_first_launch():
    """hkb_decode_step runs up to three launches; whatever any of them would refuse -- the merge's
    alignment and stride rules included -- comes back before the first one, so a negative status
    always means that nothing ran. No GPU is needed: every case below is refused on the host."""
    l = lib.load()
    c = lib.CacheT(16, 2048, 128, 32768, 4)

    def step(out=16, out_st=(512, 128), key=16, kst=(256, 128), splits=4, po=16, pl=16, arrivals=None, nseq=1,
             fn=l.hkb_decode_step):
        return fn(out, out_st[0], out_st[1], 16, 512, 128, key, key, kst[0], kst[1], kst[0], kst[1], 16 if key else None,
                  1, c, c, 16, 8, 8, 16, None, nseq, 4, 2, 128, 16, 0.1, 0, None, None, splits, po, pl, arrivals, None)

    assert step(nseq=0) == 0
    assert step(out=18) == -7                      # the merge stores 8-byte pairs: out must be 8-byte aligned
    assert step(out_st=(510, 128)) == -6           # and its strides multiples of 4 elements
    assert step(out_st=(512, 126)) == -6
    assert step(po=None) == -8                     # splits without scratch
    assert step(kst=(257, 128)) == -6              # new rows are read as 16-byte chunks
    assert step(key=20) == -7
    # the record-writing form: a record needs the merge, hence at least two splits
    rec = l.hkb_decode_step_record
    args = (16, 16, 16, 512, 128, None, None, 0, 0, 0, 0, None, 0, c, c, 16, 8, 8, 16, None, 1, 4, 2, 128, 16, 0.1, 0,
            None, None)
    assert rec(*args, 1, 16, 16, None) == -8
    assert rec(*args[:20], 0, *args[21:], 4, 16, 16, None) == 0        # no sequences: nothing to do
    assert rec(None, 16, *args[2:], 4, 16, 16, None) == -1


def test_probe_refuses_bad_arguments_without_a_gpu():
    l = lib.load()
    assert l.hkb_hbm_read_probe(None, 1 << 20, 2, 4, 16, None) == -1
    assert l.hkb_hbm_read_probe(16, 1 << 20, 0, 4, 16, None) == -9
    assert l.hkb_hbm_read_probe(24, 1 << 20, 2, 4, 16, None) == -7


def test_scratch_sizes():
    l = lib.load()
    off = l.hkb_scratch_lse_offset(64, 32, 128, 4)
    assert off == 64 * 4 * 32 * 128 * 4 and off % 256 == 0
    assert l.hkb_scratch_bytes(64, 32, 128, 4) >= off + 64 * 4 * 32 * 4
    assert l.hkb_scratch_bytes(0, 32, 128, 4) == 0


def test_plans_are_powers_of_two_and_few(monkeypatch):
    monkeypatch.delenv("HK_SPLITS", raising=False)
    plans = [paged.plan_splits_for(n, 8, 2560, 148) for n in range(1, 257)]
    assert all(p & (p - 1) == 0 and 1 <= p <= paged.MAX_SPLITS for p in plans)
    assert len(set(plans)) <= 9
    assert plans == sorted(plans, reverse=True)                 # fewer requests, more splits
    assert paged.plan_splits_for(512, 8, 2560, 148) == 4
    assert paged.plan_splits_for(64, 8, 2560, 148) == 32 and paged.plan_splits_for(2, 8, 8192, 148) == 256
    # never (many) more slots than 2-tile pieces of the longest sequence allowed
    assert paged.plan_splits_for(1, 1, 16, 148) <= 16
    assert paged.plan_splits_for(1, 1, 1, 148) == 2


def test_c_planner_equals_python_planner():
    l = lib.load()
    for n in (1, 2, 3, 4, 8, 16, 24, 32, 64, 100, 128, 256):
        for hkv in (1, 2, 4, 8):
            for tiles in (1, 7, 64, 512, 8192):
                assert l.hkb_plan_splits(n, hkv, tiles, 148) == paged.plan_splits_for(n, hkv, tiles, 148), (n, hkv, tiles)


def test_hk_splits_override(monkeypatch):
    for v in ("off", "0", "1"):
        monkeypatch.setenv("HK_SPLITS", v)
        assert paged.plan_splits(1, 8, 2560) == 1
    monkeypatch.setenv("HK_SPLITS", "8")
    assert paged.plan_splits(64, 8, 2560) == 8
    monkeypatch.setenv("HK_SPLITS", "12")
    assert paged.plan_splits(64, 8, 2560) == 8                   # a power of two
    monkeypatch.setenv("HK_SPLITS", "64")
    assert paged.plan_splits(64, 8, 4) == 4                      # never more than the pages
    monkeypatch.setenv("HK_SPLITS", "auto")
    assert paged.plan_splits(64, 8, 2560) == paged.plan_splits_for(64, 8, 2560, paged.sm_count())


def test_worker_choice_and_step_sizes_are_host_facts():
    """Which worker walks a GQA group, and the arrival-counter size of the one-launch step: host-only
    entry points, callable without a GPU. Defaults (no HKB_MMA_MIN_GROUP in the environment):
    bf16 caches go to the tensor-core worker from a group of 4, fp8 caches always."""
    h = lib.load()
    if not os.environ.get("HKB_MMA_MIN_GROUP"):
        assert [h.hkb_walk_uses_mma(g, lib.KV_BF16) for g in (1, 2, 3, 4, 6, 8, 16)] == [0, 0, 0, 1, 1, 1, 1]
        assert [h.hkb_walk_uses_mma(g, lib.KV_FP8_E4M3) for g in (1, 2, 4, 8)] == [1, 1, 1, 1]
    assert h.hkb_arrivals_bytes(64, 8) == 64 * 8 * 2 * 17 * 4
    assert h.hkb_arrivals_bytes(0, 8) == 0 and h.hkb_arrivals_bytes(4, 0) == 0
