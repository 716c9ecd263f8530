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
