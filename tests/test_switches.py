"""Route switches: the reference's precedence (HK_DISABLE > engine switch > route switch >
default by arch), checked rule by rule and differentially against decisions recorded from
the reference's own switches.py (tests/golden/switches_golden.json)."""

import json
import os

import pytest

from hk_dsl_b200.integration import switches

GOLD = os.path.join(os.path.dirname(__file__), "golden", "switches_golden.json")


def test_every_decision_matches_the_reference():
    gold = json.load(open(GOLD))
    ref_arch = gold["validated_arch"]
    for r in gold["rows"]:
        gpu = switches.SM100 if r["validated_gpu"] else None
        d = switches.decide(r["route"], r["env"], gpu=gpu)
        assert d.on == r["on"], (r, d)
        assert d.value == r["value"], (r, d)
        want = r["why"].replace(ref_arch, switches.SM100)
        if want.startswith("default off on"):           # the tail lists each build's own validated archs
            assert d.why.startswith(want.split("(")[0].strip()), (r, d)
        else:
            assert d.why == want, (r, d)


def test_precedence():
    on = {"HK_VLLM_PREFILL": "1", "HK_VLLM_BACKEND": "1"}
    assert not switches.decide("vllm_prefill", dict(on, HK_DISABLE="1")).on
    assert switches.decide("vllm_prefill", dict(on, HK_DISABLE="0")).on
    assert not switches.decide("vllm_backend", dict(on, HK_PATCH_VLLM="off")).on
    assert switches.decide("vllm_backend", dict(on, HK_PATCH_VLLM="1")).on
    assert not switches.decide("vllm_prefill", {"HK_VLLM_PREFILL": "no"}, gpu=switches.SM100).on
    assert switches.decide("vllm_prefill", {}, gpu=switches.SM100).on
    assert not switches.decide("vllm_prefill", {}, gpu=None).on
    assert not switches.decide("vllm_prefill", {}, gpu="sm_90").on
    assert not switches.decide("vllm_backend", {}, gpu=switches.SM100).on      # off until asked for
    assert switches.decide("vllm_backend", {"HK_VLLM_BACKEND": "FLASH_ATTN"}).value == "FLASH_ATTN"
    assert switches.decide("vllm_backend", {"HK_VLLM_BACKEND": " on "}).value == ""
    assert switches.decide("vllm_prefill", {"HK_VLLM_PREFILL": ""}, gpu=None).why.startswith("default off")


def test_disabled_and_tables():
    assert switches.disabled({"HK_DISABLE": "1"}) and switches.disabled({"HK_DISABLE": "anything"})
    assert not switches.disabled({"HK_DISABLE": "false"}) and not switches.disabled({})
    assert set(switches.on("vllm", {"HK_VLLM_BACKEND": "1", "HK_VLLM_PREFILL": "1"})) == {"vllm_backend", "vllm_prefill"}
    assert switches.on("vllm", {"HK_DISABLE": "1", "HK_VLLM_BACKEND": "1"}) == {}
    t = switches.table({"HK_DISABLE": "1"})
    assert "vllm_backend" in t and "HK_DISABLE=1" in t and t.count("off") >= 2


def test_status_cli(capsys):
    from hk_dsl_b200.integration.__main__ import main

    assert main(["--status"]) == 0
    out = capsys.readouterr().out
    assert "vllm_prefill" in out and "hkb library" in out
    assert main(["--bogus"]) == 2


def test_plugin_never_raises_and_says_what_it_did(capsys, monkeypatch):
    from hk_dsl_b200.integration import _vllm_plugin

    monkeypatch.setenv("HK_DISABLE", "1")
    _vllm_plugin.register()
    assert "off (HK_DISABLE=1)" in capsys.readouterr().out
    monkeypatch.delenv("HK_DISABLE")
    monkeypatch.setenv("HK_PATCH_VLLM", "0")
    _vllm_plugin.register()
    assert "no route on" in capsys.readouterr().out
    # a route whose apply raises is off with a warning; the plugin still returns
    monkeypatch.delenv("HK_PATCH_VLLM")
    monkeypatch.setenv("HK_VLLM_BACKEND", "1")
    monkeypatch.setenv("HK_VLLM_PREFILL", "0")
    monkeypatch.setitem(_vllm_plugin.APPLY, "vllm_backend", lambda: (_ for _ in ()).throw(RuntimeError("boom")))
    _vllm_plugin.register()
    got = capsys.readouterr()
    assert "WARNING" in got.err and "boom" in got.err and "route vllm_backend OFF" in got.err     # the warning line: stderr
    assert "no route applied" in got.out
