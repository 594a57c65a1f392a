"""Phase tracing: NVTX ranges and device-side phase times, off unless asked for.

    TERRACE_TRACE=nvtx     every ``phase(name)`` block becomes an NVTX range (for a timeline tool)
    TERRACE_TRACE=events   every block is bracketed by CUDA events on the current stream and
                           accumulated per name; ``report()`` synchronises once and returns the
                           totals, ``report(group)`` the max over ranks
    TERRACE_TRACE=1        both

Disabled (the default) ``phase`` returns one shared no-op context manager: no allocation, no
device call.  On a CPU the ``events`` mode falls back to ``perf_counter``.

The events are recorded on the stream the work runs on and read only in ``report()``, so tracing
adds no host synchronisation to a step; what it measures is the *span* of each phase on its
stream.  With the serial schedule of the fused layer that is the phase's exposed time; with
the overlap schedule the dispatch span shrinks to its launches and the waiting shows up inside
the "experts" and "combine" spans, which is how the exposed share is read off.  The reference has no tracing; its protocol for attributing exposed time per stream is
prose (``docs/09-phase-model.md:49-85``), and its timing idiom is barrier / synchronize /
perf_counter with a max over ranks (``bench/a2a_form_probe.py:47-77``).
"""
from __future__ import annotations

import os
import time
from collections import OrderedDict

_MODE = None            # None = not read yet; frozenset of {"nvtx", "events"}
_SPANS = OrderedDict()  # name -> list of (start, stop) events or float seconds
_MAX_PENDING = 4096     # events kept per name before the oldest are folded into the total
_TOTALS = OrderedDict() # name -> [milliseconds, count] already folded


def _mode():
    global _MODE
    if _MODE is None:
        v = os.environ.get("TERRACE_TRACE", "0").strip().lower()
        if v in ("", "0", "off", "false"):
            _MODE = frozenset()
        elif v in ("1", "on", "true", "all"):
            _MODE = frozenset(("nvtx", "events"))
        else:
            parts = [p.strip() for p in v.replace("+", ",").split(",") if p.strip()]
            bad = [p for p in parts if p not in ("nvtx", "events")]
            if bad:
                _MODE = frozenset()
                raise ValueError("TERRACE_TRACE=%r: expected 0, 1, nvtx, events or nvtx,events" % v)
            _MODE = frozenset(parts)
    return _MODE


def reset(mode: str | None = None) -> None:
    """Forget everything recorded; with ``mode`` also override the environment switch."""
    global _MODE
    _SPANS.clear()
    _TOTALS.clear()
    if mode is None:
        _MODE = None
    else:
        os.environ["TERRACE_TRACE"] = mode
        _MODE = None


def enabled() -> bool:
    return bool(_mode())


class _Noop:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NOOP = _Noop()


class _Phase:
    __slots__ = ("name", "cuda", "start", "nvtx")

    def __init__(self, name: str, cuda: bool):
        self.name, self.cuda, self.start, self.nvtx = name, cuda, None, False

    def __enter__(self):
        mode = _mode()
        if self.cuda:
            import torch
            if "nvtx" in mode:
                torch.cuda.nvtx.range_push(self.name)
                self.nvtx = True
            if "events" in mode:
                self.start = torch.cuda.Event(enable_timing=True)
                self.start.record()
        elif "events" in mode:
            self.start = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.start is not None:
            if self.cuda:
                import torch
                stop = torch.cuda.Event(enable_timing=True)
                stop.record()
            else:
                stop = time.perf_counter()
            pending = _SPANS.setdefault(self.name, [])
            pending.append((self.start, stop))
            if len(pending) > _MAX_PENDING:
                _fold(self.name, pending[: _MAX_PENDING // 2])
                del pending[: _MAX_PENDING // 2]
        if self.nvtx:
            import torch
            torch.cuda.nvtx.range_pop()
        return False


def phase(name: str, cuda: bool | None = None):
    """Context manager around one phase.  ``cuda=None`` decides by ``torch.cuda.is_available()``
    the first time tracing is on."""
    if not _mode():
        return _NOOP
    if cuda is None:
        import torch
        cuda = torch.cuda.is_available()
    return _Phase(name, cuda)


def _fold(name: str, spans) -> None:
    ms = 0.0
    for a, b in spans:
        ms += a.elapsed_time(b) if hasattr(a, "elapsed_time") else (b - a) * 1e3
    tot = _TOTALS.setdefault(name, [0.0, 0])
    tot[0] += ms
    tot[1] += len(spans)


def report(group=None, reset_after: bool = True) -> dict:
    """``{name: {"ms": total, "calls": n, "ms_per_call": ...}}``; with a process group (or
    ``group=True`` for the default one) the totals are the max over ranks.  Synchronises the
    device once."""
    has_events = any(hasattr(a, "elapsed_time") for spans in _SPANS.values() for a, _ in spans[:1])
    if has_events:
        import torch
        torch.cuda.synchronize()
    for name, spans in list(_SPANS.items()):
        _fold(name, spans)
        spans.clear()
    out = OrderedDict((n, {"ms": t[0], "calls": t[1]}) for n, t in _TOTALS.items())
    if group is not None and out:
        import torch
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            pg = None if group is True else group
            dev = "cuda" if dist.get_backend(pg) == "nccl" else "cpu"
            t = torch.tensor([v["ms"] for v in out.values()], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=pg)
            for v, ms in zip(out.values(), t.tolist()):
                v["ms"] = ms
    for v in out.values():
        v["ms_per_call"] = v["ms"] / max(v["calls"], 1)
    if reset_after:
        _SPANS.clear()
        _TOTALS.clear()
    return out


def format_report(rep: dict) -> str:
    total = sum(v["ms"] for v in rep.values()) or 1.0
    lines = ["%-28s %10s %8s %12s %7s" % ("phase", "ms", "calls", "ms / call", "share")]
    for name, v in rep.items():
        lines.append("%-28s %10.3f %8d %12.4f %6.1f%%" % (name, v["ms"], v["calls"],
                                                          v["ms_per_call"],
                                                          100.0 * v["ms"] / total))
    return "\n".join(lines)
