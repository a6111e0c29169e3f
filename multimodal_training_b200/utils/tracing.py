"""Step tracing: NVTX ranges, device-timed phases without host syncs, and a Chrome trace file.

The reference only has ``training.profile_time``: a ``torch.cuda.synchronize()`` plus ``time.perf_counter()``
around each actor's forward and backward (python/ray/vision.py:439-441,470-474; python/ray/text.py:709-711),
which serialises the step it measures.  Here:

* :func:`trace_range` opens an NVTX range (visible in Nsight Systems / Compute timelines) when tracing is on;
* :class:`PhaseTimer` brackets phases with CUDA events on the launching stream and resolves them after the step,
  so the numbers are device time and the step keeps running asynchronously;
* :meth:`PhaseTimer.chrome_trace` writes the phases of the recorded steps as a ``chrome://tracing`` JSON file.

Tracing is off by default; ``training.trace: true`` (or ``MMT_TRACE=1``) turns it on.
"""
from __future__ import annotations

import contextlib
import json
import os
import time

import torch

_ENABLED = os.environ.get("MMT_TRACE", "0") not in ("", "0", "false")


def enable(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(on)


def enabled() -> bool:
    return _ENABLED


@contextlib.contextmanager
def trace_range(name: str):
    """NVTX range around a block of launches (no-op unless tracing is on and CUDA is in use).

    A start/end range, not push/pop: push/pop ranges belong to the calling thread, and the kernels of a backward
    pass are launched by autograd's worker thread, so a profiler filtering on a push/pop range would miss them."""
    if _ENABLED and torch.cuda.is_available():
        handle = torch.cuda.nvtx.range_start(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_end(handle)
    else:
        yield


class PhaseTimer:
    """Device-timed phases of training steps.

    ``with timer.phase("text.forward"): ...`` records a pair of CUDA events (host clock on CPU); ``end_step()``
    closes a step; ``summary()`` synchronises once and returns the mean milliseconds per phase.
    """

    def __init__(self, use_cuda: bool | None = None):
        self.cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.steps: list[list[tuple]] = []
        self._cur: list[tuple] = []

    @contextlib.contextmanager
    def phase(self, name: str):
        host0 = time.perf_counter()
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        with trace_range(name):
            yield
        if self.cuda:
            e1.record()
            self._cur.append((name, host0, e0, e1))
        else:
            self._cur.append((name, host0, None, time.perf_counter() - host0))

    def end_step(self) -> None:
        self.steps.append(self._cur)
        self._cur = []

    def _resolved(self):
        if self.cuda:
            torch.cuda.synchronize()
        for i, step in enumerate(self.steps):
            for name, host0, e0, e1 in step:
                ms = e0.elapsed_time(e1) if self.cuda else e1 * 1e3
                yield i, name, host0, ms

    def summary(self) -> dict[str, float]:
        tot: dict[str, list[float]] = {}
        for _, name, _, ms in self._resolved():
            tot.setdefault(name, []).append(ms)
        return {k: sum(v) / len(v) for k, v in tot.items()}

    def chrome_trace(self, path: str, rank: int = 0) -> str:
        events = []
        for i, name, host0, ms in self._resolved():
            events.append({"name": name, "ph": "X", "pid": rank, "tid": 0, "ts": host0 * 1e6, "dur": ms * 1e3,
                           "args": {"step": i}})
        with open(path, "w") as f:
            json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
        return path
