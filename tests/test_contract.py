"""The engine contract of the two vLLM routes (introspection only; no GPU): facts gathered from
the installed vLLM hold; a lost name breaks exactly the route that binds to it; a route with a
broken contract or a raising apply is left off with one warning line and the other is applied
(the reference's rule since it went per route, python/hk/integration/contract.py:10-16, 864-906)."""

import pytest

from hk_dsl_b200.integration import contract

vllm = pytest.importorskip("vllm")


def test_the_installed_engine_holds_both_contracts():
    assert contract.check_each(["vllm_prefill", "vllm_backend"]) == {}
    f = contract.gather_vllm_backend()
    assert "CUSTOM" in f["backend_slots"] and f["impl_forward"][:7] == list(contract.FORWARD_NEEDS)


def test_a_lost_name_breaks_the_route_that_reads_it():
    f = contract.gather_vllm_prefill()
    f["unified_attention"] = [n for n in f["unified_attention"] if n != "seqused_k"]
    assert contract.judge_vllm_prefill(f) == ["unified_attention lost ['seqused_k']"]
    b = contract.gather_vllm_backend()
    b["backend_slots"] = ["FLASH_ATTN"]
    b["impl_forward"] = ["layer", "q", "k", "v", "kv_cache", "attn_metadata", "output"]
    got = contract.judge_vllm_backend(b)
    assert len(got) == 2 and "has no CUSTOM" in got[0] and "now takes" in got[1]


def test_routes_are_judged_and_applied_one_by_one(monkeypatch, capsys):
    monkeypatch.setitem(contract.JUDGE, "vllm_prefill", lambda f: ["unified_attention lost ['q']"])
    calls = []
    appliers = {"vllm_backend": lambda: (calls.append("backend") or "backend registered", lambda: None),
                "vllm_prefill": lambda: (calls.append("prefill") or "prefill applied", lambda: None)}
    reports, applied, off = contract.apply_routes(["vllm_backend", "vllm_prefill"], appliers)
    assert calls == ["backend"] and reports == ["backend registered"] and list(applied) == ["vllm_backend"]
    assert off == {"vllm_prefill": ["unified_attention lost ['q']"]}
    err = capsys.readouterr().err
    assert "route vllm_prefill OFF -- engine contract FAILED" in err and "HK_VLLM_PREFILL=0" in err
    assert "The other route is unaffected" in err


def test_an_apply_that_raises_is_reported_and_the_other_goes_on(monkeypatch, capsys):
    def boom():
        raise RuntimeError("no such slot")

    reports, applied, off = contract.apply_routes(
        ["vllm_backend", "vllm_prefill"], {"vllm_backend": boom, "vllm_prefill": lambda: ("prefill applied", lambda: None)})
    assert reports == ["prefill applied"] and list(applied) == ["vllm_prefill"]
    assert off == {"vllm_backend": ["raised RuntimeError: no such slot"]}
    assert "route vllm_backend OFF -- the route failed to apply" in capsys.readouterr().err


def test_a_moved_module_is_a_broken_contract(monkeypatch):
    def gone():
        raise ImportError("No module named 'vllm.v1.attention.ops.triton_unified_attention'")

    monkeypatch.setitem(contract.GATHER, "vllm_prefill", gone)
    got = contract.check_each(["vllm_prefill", "vllm_backend", "not_a_route"])
    assert list(got) == ["vllm_prefill"] and got["vllm_prefill"][0].startswith("ImportError")
