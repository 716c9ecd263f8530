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


def test_an_op_registers_and_runs_through_the_dispatcher_on_cpu():
    """`Op.define` on the CPU dispatch key: the guarded implementation is what torch.ops calls,
    the fake is registered, a second define is a no-op."""
    import torch

    seen = []

    def impl(x, out):
        seen.append(tuple(x.shape))
        out.copy_(x + 1)

    op = engine.Op("hk_test_ns::bump", "bump(Tensor x, Tensor(a!) out) -> ()", lambda x, out: None, ("launch",))
    assert not op.defined
    assert op.define(impl, dispatch="CPU") is op and op.defined
    assert op.define(impl, dispatch="CPU") is op
    x, out = torch.zeros(3), torch.empty(3)
    op(x, out)                                              # a CPU tensor: through the dispatcher
    assert out.tolist() == [1.0, 1.0, 1.0] and seen == [(3,)]
    torch.ops.hk_test_ns.bump(x, out)
    assert seen == [(3,), (3,)]
    assert (op.ns, op.op_name) == ("hk_test_ns", "bump")


def test_guard_keeps_the_wrapped_functions_name():
    p = engine.Patch("t_named", ("a",))

    def wrapper_body(x):
        """doc"""
        return x

    g = p.guard(wrapper_body)
    assert g.__name__ == "wrapper_body" and g.__doc__ == "doc" and g.__wrapped__ is wrapper_body and g(3) == 3


def test_the_plugin_entry_point_is_declared_and_resolves():
    """pyproject.toml declares the `vllm.general_plugins` entry point vLLM's workers load
    (the reference: pyproject.toml:54-55); the target it names exists and is callable."""
    import importlib
    import os
    import tomllib

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "pyproject.toml"), "rb") as f:
        meta = tomllib.load(f)
    eps = meta["project"]["entry-points"]["vllm.general_plugins"]
    assert list(eps) == ["hk_attention"]
    module, _, attr = eps["hk_attention"].partition(":")
    fn = getattr(importlib.import_module(module), attr)
    assert callable(fn) and fn.__name__ == "register"
    for pkg in meta["tool"]["setuptools"]["packages"]:
        importlib.import_module(pkg)
