"""What every engine patch of this build has in common: counted paths, the CUDA-graph
contract, and the opaque torch custom op.

The shape is hk-dsl's (python/hk/integration/engine.py:45-230): a `Patch` counts which way
calls went (eager and captured calls apart, because a graph replay runs no Python) and
declares `graph="safe"` or `graph="never"`; under capture a "never" patch raises
`GraphCaptureError` with its reason, and a "safe" patch runs with torch's sync-debug mode
set to error, so a host sync inside a wrapper (`.item()`, `.tolist()`, a blocking copy)
raises at the line that does it, naming the patch. `Op` is a patch that is also
`torch.ops.<ns>.<name>` with a fake implementation, called directly in eager code.
"""

from __future__ import annotations

import contextlib
import functools
import os
from typing import Callable, Dict, List, Sequence

GRAPH_CONTRACTS = ("safe", "never")

#: every patch constructed, by name, for the status report
PATCHES: Dict[str, "Patch"] = {}

#: HK_HOST_FASTPATH=0 routes every call through the dispatcher (python/hk/runtime/hostpath.py:24-27)
FASTPATH = os.environ.get("HK_HOST_FASTPATH", "1").strip().lower() not in ("0", "off", "no", "false")


class GraphCaptureError(RuntimeError):
    """A patch did, under CUDA-graph capture, something a replay cannot repeat."""


_CAPTURING: List[Callable[[], bool]] = []


def capturing() -> bool:
    """Whether the current stream is capturing a CUDA graph. No sync; False without a GPU."""
    if _CAPTURING:
        return _CAPTURING[0]()
    try:
        import torch  # noqa: PLC0415
    except ImportError:
        return False
    if not torch.cuda.is_available():
        return False                      # asked again next time: a GPU may yet appear
    _CAPTURING.append(torch.cuda.is_current_stream_capturing)
    return _CAPTURING[0]()


@contextlib.contextmanager
def no_host_sync(what: str):
    """Raise `GraphCaptureError` naming `what` at any host sync torch makes inside."""
    import warnings  # noqa: PLC0415

    import torch  # noqa: PLC0415

    prev = torch.cuda.get_sync_debug_mode()
    with warnings.catch_warnings():
        warnings.filterwarnings("ignore", message="Synchronization debug mode")
        torch.cuda.set_sync_debug_mode("error")
    try:
        yield
    except RuntimeError as ex:
        msg = str(ex)
        if isinstance(ex, GraphCaptureError) or not ("synchroniz" in msg or "stream is capturing" in msg):
            raise
        raise GraphCaptureError(
            f"{what} synchronized with the host while a CUDA graph was being captured. A replay runs no "
            f"Python, so whatever the wrapper read back is frozen at the capture batch's value. Keep the "
            f"decision on host values the engine already has, or declare the patch graph='never'. "
            f"({msg.splitlines()[0]})") from ex
    finally:
        torch.cuda.set_sync_debug_mode(prev)


class Patch:
    """One place an engine runs this build's kernels: its paths, counted, and its CUDA-graph
    contract, enforced by `guard`."""

    def __init__(self, name: str, paths: Sequence[str], *, graph: str = "safe", why: str = ""):
        if graph not in GRAPH_CONTRACTS:
            raise ValueError(f"graph contract {graph!r} is not one of {GRAPH_CONTRACTS}")
        if graph != "safe" and not why:
            raise ValueError(f"{name}: a patch that cannot be captured says why")
        self.name = name
        self.paths = tuple(paths)
        self.graph = graph
        self.why = why
        self.stats: Dict[str, int] = {p: 0 for p in self.paths}
        self.captured: Dict[str, int] = {p: 0 for p in self.paths}
        PATCHES[name] = self

    def count(self, path: str) -> None:
        (self.captured if capturing() else self.stats)[path] += 1

    def reset(self) -> None:
        for d in (self.stats, self.captured):
            for p in d:
                d[p] = 0

    def check_capture(self) -> None:
        if self.graph == "never" and capturing():
            raise GraphCaptureError(f"{self.name} is declared graph='never' and is being captured: {self.why}")

    def guard(self, fn: Callable) -> Callable:
        """`fn` under this patch's contract. Free outside capture."""

        @functools.wraps(fn)
        def guarded(*args, **kwargs):
            if not capturing():
                return fn(*args, **kwargs)
            self.check_capture()
            with no_host_sync(self.name):
                return fn(*args, **kwargs)

        return guarded

    def summary(self) -> str:
        def fmt(d):
            return ", ".join(f"{p} {n}" for p, n in d.items())

        cap = sum(self.captured.values())
        return f"{self.name}: {fmt(self.stats)}" + (f"; captured: {fmt(self.captured)}" if cap else "")


class Op(Patch):
    """A patch that is an opaque torch custom op, `torch.ops.<ns>.<name>`. `schema` is the
    torch.library schema without the namespace; `fake` is what torch.compile traces."""

    def __init__(self, qualname: str, schema: str, fake: Callable, paths: Sequence[str], **kw):
        super().__init__(qualname, paths, **kw)
        self.ns, self.op_name = qualname.split("::")
        self.schema = schema
        self.fake = fake
        self._lib = None
        self._op = None
        self._direct = None

    @property
    def defined(self) -> bool:
        return self._lib is not None

    def define(self, impl: Callable, dispatch: str = "CUDA") -> "Op":
        """Register `impl`, guarded, and the fake. Idempotent."""
        if self._lib is not None:
            return self
        import torch  # noqa: PLC0415

        lib = torch.library.Library(self.ns, "FRAGMENT")
        lib.define(self.schema)
        guarded = self.guard(impl)
        lib.impl(self.op_name, guarded, dispatch)
        torch.library.register_fake(self.name, self.fake, lib=lib)
        self._lib = lib
        self._op = getattr(getattr(torch.ops, self.ns), self.op_name)
        if dispatch == "CUDA":
            self._direct = (guarded, torch.Tensor, torch.compiler.is_compiling)
        return self

    def __call__(self, *args, **kwargs):
        """The op -- or, in eager code on CUDA tensors, the guarded implementation called
        without the dispatcher (the dispatcher costs microseconds a call and buys nothing
        where nothing is tracing)."""
        if FASTPATH and self._direct is not None and args:
            guarded, tensor, compiling = self._direct
            x = args[0]
            if type(x) is tensor and x.is_cuda and not compiling():
                return guarded(*args, **kwargs)
        op = self._op
        if op is None:
            import torch  # noqa: PLC0415

            op = getattr(getattr(torch.ops, self.ns), self.op_name)
        return op(*args, **kwargs)
