"""The patch / op contract (python/hk/integration/engine.py:45-230 of the reference;
its GPU half is tests/hk/gpu/test_engine.py:35-75): counters, declared graph contracts,
refusal under capture -- the host logic, with capture faked."""

import pytest

from hk_dsl_b200.integration import engine


def test_counters_split_eager_and_captured(monkeypatch):
    p = engine.Patch("t_counts", ("decode", "fallback"))
    p.count("decode")
    p.count("fallback")
    monkeypatch.setattr(engine, "capturing", lambda: True)
    p.count("decode")
    assert p.stats == {"decode": 1, "fallback": 1} and p.captured == {"decode": 1, "fallback": 0}
    assert "captured: decode 1" in p.summary()
    p.reset()
    assert sum(p.stats.values()) == 0 and sum(p.captured.values()) == 0
    assert engine.PATCHES["t_counts"] is p


def test_contract_declarations():
    with pytest.raises(ValueError):
        engine.Patch("t_bad", ("a",), graph="sometimes")
    with pytest.raises(ValueError):
        engine.Patch("t_never_no_reason", ("a",), graph="never")
    engine.Patch("t_never", ("a",), graph="never", why="plans on host metadata")


def test_a_never_patch_refuses_capture_naming_its_reason(monkeypatch):
    p = engine.Patch("t_never2", ("a",), graph="never", why="reads lengths on the host")
    calls = []
    f = p.guard(lambda x: calls.append(x) or x + 1)
    assert f(1) == 2                                   # free outside capture
    monkeypatch.setattr(engine, "capturing", lambda: True)
    with pytest.raises(engine.GraphCaptureError, match="reads lengths on the host"):
        f(1)
    assert calls == [1]


def test_capturing_is_false_without_a_gpu():
    import torch

    if not torch.cuda.is_available():
        assert engine.capturing() is False
