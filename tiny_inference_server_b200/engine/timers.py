"""Where the time of a step goes, behind ``EngineConfig.profile``.

Upstream's ``Probe`` (evals.py:42-83) wraps the scheduler's methods and the model's launch paths,
synchronises the device around each and adds up milliseconds per phase (admit, prefill, decode,
sample, ...).  Here the phases of ``Engine.step`` are timed without stopping the device: host
phases with the host's clock (what the host spends on admission, planning and layout, on issuing
the launches, on waiting for the tokens, on bookkeeping), device phases with pairs of CUDA events
on the launching stream whose times are read only when a summary is asked for.  Off, every call
is a no-op.
"""
from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Dict, List, Tuple


class PhaseTimers:
    #: device event pairs kept at most (a summary empties the list)
    MAX_EVENTS = 8192

    def __init__(self, enabled: bool = False, cuda: bool = True):
        self.enabled = enabled
        self.cuda = cuda
        self.host_ms: Dict[str, float] = {}
        self.host_calls: Dict[str, int] = {}
        self.device_ms: Dict[str, float] = {}
        self.device_calls: Dict[str, int] = {}
        self._events: List[Tuple[str, object, object]] = []
        self.steps = 0

    def begin_step(self) -> None:
        if self.enabled:
            self.steps += 1

    @contextmanager
    def host(self, phase: str):
        if not self.enabled:
            yield
            return
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.host_ms[phase] = self.host_ms.get(phase, 0.0) + (time.perf_counter() - t0) * 1e3
            self.host_calls[phase] = self.host_calls.get(phase, 0) + 1

    @contextmanager
    def device(self, phase: str):
        if not (self.enabled and self.cuda):
            yield
            return
        import torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self._events.append((phase, a, b))
            if len(self._events) > self.MAX_EVENTS:
                self._drain()

    def _drain(self) -> None:
        for phase, a, b in self._events:
            b.synchronize()
            self.device_ms[phase] = self.device_ms.get(phase, 0.0) + a.elapsed_time(b)
            self.device_calls[phase] = self.device_calls.get(phase, 0) + 1
        self._events = []

    def summary(self) -> dict:
        """{"steps": n, "host_ms": {phase: total}, "device_ms": {phase: total}, "calls": {...}}.
        Waits for the device events still outstanding."""
        self._drain()
        return {"steps": self.steps,
                "host_ms": {k: round(v, 3) for k, v in self.host_ms.items()},
                "device_ms": {k: round(v, 3) for k, v in self.device_ms.items()},
                "calls": dict(self.host_calls, **{f"device:{k}": v for k, v in self.device_calls.items()})}

    def reset(self) -> None:
        self._drain()
        self.host_ms.clear()
        self.host_calls.clear()
        self.device_ms.clear()
        self.device_calls.clear()
        self.steps = 0
