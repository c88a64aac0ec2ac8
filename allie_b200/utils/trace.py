"""Phase tracing for the training loop.

The reference only prints wall-clock deltas per ``log_interval`` (``src/modeling/trainer.py:240,
291-298``).  Here every phase of a step (data, forward/backward, gradient synchronisation and
optimizer) is bracketed by an NVTX range, which any CUDA timeline tool picks up, and - when tracing
is switched on - by a pair of CUDA events on the launching stream, so per-phase device times can be
read without a profiler attached.  Tracing never synchronises the host inside a step: the events are
resolved when ``summary()`` is called.

    tracer = PhaseTracer(enabled=True)
    with tracer.phase("forward_backward"):
        ...
    tracer.summary()   # {"forward_backward": {"count": 8, "ms": 664.1}, ...}; also resets

``ALLIE_TRACE=1`` in the environment enables the event timers of the trainer's tracer.
"""
from __future__ import annotations

import contextlib
import os
from collections import defaultdict

import torch


class PhaseTracer:
    def __init__(self, enabled: bool | None = None, device: torch.device | str | None = None):
        if enabled is None:
            enabled = os.environ.get("ALLIE_TRACE", "0") == "1"
        self.enabled = bool(enabled)
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._pending: dict[str, list] = defaultdict(list)     # phase -> [(start_event, end_event)]
        self._host_ms: dict[str, float] = defaultdict(float)   # CPU fallback (no CUDA)
        self._count: dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def phase(self, name: str):
        """NVTX range always (it costs a few hundred nanoseconds with no tool attached); device
        timers only when enabled."""
        if self.cuda:
            torch.cuda.nvtx.range_push(name)
        start = end = t0 = None
        if self.enabled:
            if self.cuda:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
            else:
                import time

                t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.enabled:
                self._count[name] += 1
                if self.cuda:
                    end.record()
                    self._pending[name].append((start, end))
                else:
                    import time

                    self._host_ms[name] += (time.perf_counter() - t0) * 1e3
            if self.cuda:
                torch.cuda.nvtx.range_pop()

    def summary(self, reset: bool = True) -> dict[str, dict[str, float]]:
        """Per-phase call count and total milliseconds since the last summary (device time where
        CUDA is in use).  Waits for the recorded events, so call it at logging points only."""
        out: dict[str, dict[str, float]] = {}
        for name, n in self._count.items():
            ms = self._host_ms.get(name, 0.0)
            for s, e in self._pending.get(name, []):
                e.synchronize()
                ms += s.elapsed_time(e)
            out[name] = {"count": n, "ms": ms}
        if reset:
            self._pending.clear(); self._host_ms.clear(); self._count.clear()
        return out
