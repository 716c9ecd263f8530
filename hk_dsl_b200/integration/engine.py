"""What every engine patch of this build has in common: counted paths, the CUDA-graph
contract, and the opaque torch custom op.

The public surface is hk-dsl's (python/hk/integration/engine.py:45-230) because its users
and tests speak it: `Patch(name, paths, graph=, why=)` with `count / reset / check_capture /
guard / summary` and the `stats` / `captured` tallies, `Op(qualname, schema, fake, paths)`
with `define` and a direct call, `capturing()`, `no_host_sync(what)`, `GraphCaptureError`.
The rules behind it:

* a path is counted where it ran: eagerly, or while a CUDA graph was being captured (a
  replay runs no Python, so captured calls are a different statistic);
* a patch declares whether it may be captured. `graph="never"` needs a reason and refuses
  capture with it; `graph="safe"` is held to its word: while capturing, the wrapped call
  runs with torch's sync-debug mode on "error", so a host read-back (`.item()`, `.tolist()`,
  a blocking copy) fails at the line that does it, with the patch's name in the message;
* an `Op` is a patch that is also `torch.ops.<ns>.<name>` with a fake implementation for
  tracing. Eager calls on CUDA tensors skip the dispatcher (it costs microseconds and buys
  nothing when nothing traces); HK_HOST_FASTPATH=0 sends every call through it
  (python/hk/runtime/hostpath.py:24-27).
"""

from __future__ import annotations

import os
from typing import Callable, Dict, Optional, Sequence

GRAPH_CONTRACTS = ("safe", "never")

#: every patch constructed, by name, for the status report
PATCHES: Dict[str, "Patch"] = {}

FASTPATH = os.environ.get("HK_HOST_FASTPATH", "1").strip().lower() not in ("0", "off", "no", "false")


class GraphCaptureError(RuntimeError):
    """A patch did, under CUDA-graph capture, something a replay cannot repeat."""


class _CaptureProbe:
    """Asks torch whether the current stream is capturing, binding torch's function on first use
    with a GPU present (without one the answer is False and the question is asked again later)."""

    def __init__(self):
        self._ask: Optional[Callable[[], bool]] = None

    def __call__(self) -> bool:
        ask = self._ask
        if ask is None:
            try:
                import torch  # noqa: PLC0415
            except ImportError:
                return False
            if not torch.cuda.is_available():
                return False
            ask = self._ask = torch.cuda.is_current_stream_capturing
        return bool(ask())


_probe = _CaptureProbe()


def capturing() -> bool:
    """Whether the current stream is capturing a CUDA graph. No sync; False without a GPU."""
    return _probe()


class no_host_sync:  # noqa: N801  (used as `with no_host_sync("name"):`, like the reference's context manager)
    """Inside the block any host synchronisation torch performs raises `GraphCaptureError`
    that names `what`. The previous sync-debug mode is restored on the way out."""

    _SIGNS = ("synchroniz", "stream is capturing")

    def __init__(self, what: str):
        self.what = what
        self._before = None

    def __enter__(self):
        import warnings  # noqa: PLC0415

        import torch  # noqa: PLC0415

        self._before = torch.cuda.get_sync_debug_mode()
        with warnings.catch_warnings():
            warnings.filterwarnings("ignore", message="Synchronization debug mode")
            torch.cuda.set_sync_debug_mode("error")
        return self

    def __exit__(self, kind, err, tb):
        import torch  # noqa: PLC0415

        torch.cuda.set_sync_debug_mode(self._before)
        if err is None or isinstance(err, GraphCaptureError) or not isinstance(err, RuntimeError):
            return False
        text = str(err)
        if not any(sign in text for sign in self._SIGNS):
            return False
        first = text.splitlines()[0] if text else ""
        raise GraphCaptureError(
            f"{self.what} read something back from the device during CUDA-graph capture. Replays execute the "
            f"recorded launches only -- no Python runs -- so a value fetched here would stay what it was for "
            f"the captured batch. Decide from values the host already holds, or declare the patch "
            f"graph='never' with the reason. [{first}]") from err


class _Guarded:
    """A callable under a patch's graph contract: untouched outside capture; under capture a
    "never" patch refuses and a "safe" one runs with host syncs turned into errors."""

    def __init__(self, patch: "Patch", fn: Callable):
        self.patch, self.fn = patch, fn
        for attr in ("__name__", "__qualname__", "__doc__", "__module__"):
            if hasattr(fn, attr):
                setattr(self, attr, getattr(fn, attr))
        self.__wrapped__ = fn

    def __call__(self, *args, **kwargs):
        if capturing():
            self.patch.check_capture()
            with no_host_sync(self.patch.name):
                return self.fn(*args, **kwargs)
        return self.fn(*args, **kwargs)


class Patch:
    """One place an engine runs this build's kernels: its paths, counted, and its CUDA-graph
    contract, enforced by `guard`."""

    def __init__(self, name: str, paths: Sequence[str], *, graph: str = "safe", why: str = ""):
        if graph not in GRAPH_CONTRACTS:
            raise ValueError(f"graph contract {graph!r} is not one of {GRAPH_CONTRACTS}")
        if graph == "never" and not why:
            raise ValueError(f"{name}: a patch that cannot be captured says why")
        self.name, self.paths, self.graph, self.why = name, tuple(paths), graph, why
        # tallies by "was a graph being captured": False -> eager calls, True -> captured calls
        self._tally = {flag: dict.fromkeys(self.paths, 0) for flag in (False, True)}
        PATCHES[name] = self

    @property
    def stats(self) -> Dict[str, int]:
        return self._tally[False]

    @property
    def captured(self) -> Dict[str, int]:
        return self._tally[True]

    def count(self, path: str) -> None:
        self._tally[bool(capturing())][path] += 1

    def reset(self) -> None:
        for tally in self._tally.values():
            tally.update(dict.fromkeys(tally, 0))

    def check_capture(self) -> None:
        if self.graph == "never" and capturing():
            raise GraphCaptureError(f"{self.name} is declared graph='never' and is being captured: {self.why}")

    def guard(self, fn: Callable) -> Callable:
        """`fn` under this patch's contract. Free outside capture."""
        return _Guarded(self, fn)

    def summary(self) -> str:
        parts = [", ".join(f"{path} {hits}" for path, hits in self.stats.items())]
        if any(self.captured.values()):
            parts.append("captured: " + ", ".join(f"{path} {hits}" for path, hits in self.captured.items()))
        return f"{self.name}: " + "; ".join(parts)


class Op(Patch):
    """A patch that is an opaque torch custom op, `torch.ops.<ns>.<name>`. `schema` is the
    torch.library schema without the namespace; `fake` is what torch.compile traces."""

    def __init__(self, qualname: str, schema: str, fake: Callable, paths: Sequence[str], **kw):
        super().__init__(qualname, paths, **kw)
        self.ns, _, self.op_name = qualname.partition("::")
        self.schema, self.fake = schema, fake
        self._lib = None           # the torch.library fragment that keeps the registration alive
        self._impl = None          # the guarded implementation, for direct eager calls
        self._cuda_only = False
        self._torch = None         # the torch module, bound at define() so a call does not import

    @property
    def defined(self) -> bool:
        return self._lib is not None

    def _dispatcher_entry(self):
        import torch  # noqa: PLC0415

        return getattr(getattr(torch.ops, self.ns), self.op_name)

    def define(self, impl: Callable, dispatch: str = "CUDA") -> "Op":
        """Register `impl`, guarded, and the fake. Idempotent."""
        if self.defined:
            return self
        import torch  # noqa: PLC0415

        fragment = torch.library.Library(self.ns, "FRAGMENT")
        fragment.define(self.schema)
        self._impl = self.guard(impl)
        fragment.impl(self.op_name, self._impl, dispatch)
        torch.library.register_fake(self.name, self.fake, lib=fragment)
        self._cuda_only = dispatch == "CUDA"
        self._torch = torch
        self._lib = fragment
        return self

    def _eager_cuda(self, args) -> bool:
        """Plain CUDA tensor first, nothing tracing: the dispatcher would only cost time."""
        if not (FASTPATH and self._cuda_only and args):
            return False
        torch = self._torch
        first = args[0]
        return type(first) is torch.Tensor and first.is_cuda and not torch.compiler.is_compiling()

    def __call__(self, *args, **kwargs):
        if self._impl is not None and self._eager_cuda(args):
            return self._impl(*args, **kwargs)
        return self._dispatcher_entry()(*args, **kwargs)
