"""The decode's launch contract refuses wrong shapes and dtypes before anything is launched,
with messages that name the tensor (python/hk/ops/paged.py:746-802 and
tests/hk/ir/test_paged_contract.py of the reference). CPU tensors: only metadata is read."""

import pytest
import torch

from hk_dsl_b200.ops import paged


def _ok(reqs=3, hkv=2, g=4, d=128, page=16, blocks=10, pages=5, splits=1):
    q = torch.zeros(reqs, hkv, g, d, dtype=torch.bfloat16)
    k = torch.zeros(blocks, hkv, page, d, dtype=torch.bfloat16)
    return dict(q=q, k_cache=k, v_cache=k.clone(), block_table=torch.zeros(reqs, pages, dtype=torch.int32),
                seq_lens=torch.zeros(reqs, dtype=torch.int32), out=torch.zeros_like(q))


def test_a_good_call_passes():
    paged.check_decode(**_ok())
    a = _ok()
    a["block_table"] = torch.zeros(8, 5, dtype=torch.int32)     # more rows than requests is fine
    a["seq_lens"] = torch.zeros(8, dtype=torch.int32)
    paged.check_decode(**a)
    paged.check_decode(**_ok(page=48))
    a = _ok()
    a["k_cache"] = a["k_cache"].to(torch.float8_e4m3fn)
    a["v_cache"] = a["v_cache"].to(torch.float8_e4m3fn)
    paged.check_decode(**a)


@pytest.mark.parametrize("name,bad,word", [
    ("q", lambda a: a["q"][0], "q is"),
    ("q", lambda a: torch.zeros(3, 2, 17, 128, dtype=torch.bfloat16), "1 to 16 query rows"),
    ("q", lambda a: a["q"].float(), "bfloat16"),
    ("q", lambda a: torch.zeros(3, 2, 4, 96, dtype=torch.bfloat16), "head_dim"),
    ("out", lambda a: a["out"][:, :, :2], "out is"),
    ("k_cache", lambda a: torch.zeros(10, 3, 16, 128, dtype=torch.bfloat16), "k_cache is"),
    ("k_cache", lambda a: torch.zeros(10, 2, 20, 128, dtype=torch.bfloat16), "multiple of 16"),
    ("v_cache", lambda a: torch.zeros(9, 2, 16, 128, dtype=torch.bfloat16), "v_cache is"),
    ("v_cache", lambda a: a["v_cache"].half(), "v_cache is"),
    ("block_table", lambda a: a["block_table"].long(), "int32"),
    ("block_table", lambda a: a["block_table"][:2], "requests >= 3"),
    ("seq_lens", lambda a: a["seq_lens"].long(), "int32"),
    ("seq_lens", lambda a: a["seq_lens"][:1], "requests >= 3"),
])
def test_refusals_name_the_tensor(name, bad, word):
    a = _ok()
    a[name] = bad(a)
    with pytest.raises(ValueError, match=word):
        paged.check_decode(**a)


def test_tile_rows_and_scratch():
    a = _ok()
    with pytest.raises(ValueError, match="16-row tile"):
        paged.check_decode(**a, rows="tile")
    with pytest.raises(ValueError, match="need scratch"):
        paged.check_decode(**a, splits=4)
    good = paged.fused_scratch(3 * 4, 2, 128, "cpu", group=4)
    paged.check_decode(**a, splits=4, scratch=good)
    small = paged.fused_scratch(3 * 2, 2, 128, "cpu", group=4)
    with pytest.raises(ValueError, match="scratch o_part"):
        paged.check_decode(**a, splits=4, scratch=small)
    with pytest.raises(ValueError, match="scratch lse_part"):
        paged.check_decode(**a, splits=4, scratch=(good[0], good[1][:, :, :2]))


def test_no_cpu_path():
    a = _ok()
    with pytest.raises(RuntimeError, match="no CPU path"):
        paged.decode(a["q"], a["k_cache"], a["v_cache"], a["block_table"], a["seq_lens"], a["out"], None, 1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        paged.reshape_and_cache(torch.zeros(2, 2, 128, dtype=torch.bfloat16), torch.zeros(2, 2, 128, dtype=torch.bfloat16),
                                torch.zeros(4, 16, 2, 128, dtype=torch.bfloat16), torch.zeros(4, 16, 2, 128, dtype=torch.bfloat16),
                                torch.zeros(2, dtype=torch.int64))


def test_the_joined_step_and_the_prefill_have_no_cpu_path_either():
    q = torch.zeros(2, 8, 128, dtype=torch.bfloat16)
    kv = torch.zeros(2, 2, 128, dtype=torch.bfloat16)
    cache = torch.zeros(4, 16, 2, 128, dtype=torch.bfloat16)
    table = torch.zeros(2, 2, dtype=torch.int32)
    lens = torch.ones(2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        paged.decode_step(torch.empty_like(q), q, kv, kv, cache, cache, torch.zeros(2, dtype=torch.int64), table, lens, 0.1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        paged.paged_prefill(torch.empty_like(q), q, cache, cache, table, lens, torch.tensor([0, 1, 2], dtype=torch.int32),
                            torch.zeros(2, 2, dtype=torch.int32), 0.1)


def test_strides_are_checked_on_every_call_not_once_a_shape():
    """The shape memo holds shapes and dtypes, not strides: a view of an already-passed shape whose
    heads are not evenly strided (here: transposed rows) must still be refused, on every call."""
    a = _ok()
    paged._PASSED.clear()
    q = a["q"]
    key = (q.shape, q.dtype, a["k_cache"].shape, a["k_cache"].dtype, a["v_cache"].shape, a["block_table"].shape,
           a["block_table"].dtype, a["seq_lens"].shape, a["seq_lens"].dtype, a["out"].shape, a["out"].dtype, 1, None, None)
    paged._PASSED.add(key)                       # as if a well-formed call of this shape had passed before
    reqs, hkv, g, d = q.shape
    bad = torch.zeros(reqs, hkv, d, g, dtype=q.dtype).transpose(2, 3)        # same shape, head_dim not contiguous
    assert bad.shape == q.shape
    with pytest.raises(ValueError, match="evenly strided"):
        paged.decode(bad, a["k_cache"], a["v_cache"], a["block_table"], a["seq_lens"], a["out"], None, 1)
    uneven = torch.zeros(reqs, hkv, g + 1, d, dtype=q.dtype)[:, :, :g]       # kv-head stride != group x row stride
    with pytest.raises(ValueError, match="evenly strided"):
        paged.decode(a["q"], a["k_cache"], a["v_cache"], a["block_table"], a["seq_lens"], uneven, None, 1)
    paged.even_heads(a["q"], "q")


def test_backend_check_counts_pages_of_the_caches_own_block_size():
    """A table column is one page of the cache in hand: 32, 64 or a hybrid model's 544 tokens, not
    always 16."""
    from hk_dsl_b200.integration.vllm_backend import HKAttentionImplCore

    core = HKAttentionImplCore.__new__(HKAttentionImplCore)
    for block_size, max_len in ((16, 4096), (32, 4096), (64, 4096), (544, 8192)):
        cols = -(-max_len // block_size)
        table = torch.zeros(2, cols, dtype=torch.int32)
        lens = torch.tensor([max_len - 3, 17], dtype=torch.int32)       # a sequence near max_model_len
        core._checked = False
        core._check(table, lens, block_size)
        assert core._checked
        with pytest.raises(ValueError, match=f"pages of {block_size} tokens"):
            core._check(table[:, : cols - 1], torch.tensor([max_len, 1], dtype=torch.int32), block_size)
    with pytest.raises(TypeError, match="int32"):
        core._check(torch.zeros(2, 4, dtype=torch.int64), torch.ones(2, dtype=torch.int32), 16)
