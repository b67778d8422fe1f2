"""Lightweight tracing: NVTX ranges when CUDA is present plus wall-clock accounting.

``trace_range(name)`` is a context manager.  Accumulated host time and call counts per
range are available through ``summary()``, which the examples and ``bench.py`` print to
show where quorum, reconfiguration, heal and allreduce time goes.
"""

from __future__ import annotations

import threading
import time
from contextlib import contextmanager
from typing import Dict, Generator, Tuple

import torch

_lock = threading.Lock()
_totals: Dict[str, Tuple[int, float]] = {}
_nvtx = torch.cuda.is_available()


@contextmanager
def trace_range(name: str) -> Generator[None, None, None]:
    t0 = time.perf_counter()
    pushed = False
    if _nvtx:
        try:
            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:  # noqa: BLE001 - tracing must never break training
            pushed = False
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()
        dt = time.perf_counter() - t0
        with _lock:
            n, total = _totals.get(name, (0, 0.0))
            _totals[name] = (n + 1, total + dt)


def summary() -> Dict[str, Dict[str, float]]:
    with _lock:
        return {k: {"calls": n, "total_s": t, "mean_ms": 1e3 * t / max(n, 1)} for k, (n, t) in _totals.items()}


def reset() -> None:
    with _lock:
        _totals.clear()


class CudaTimer:
    """CUDA-event timer on the current stream: ``with CudaTimer() as t: ...; t.ms``."""

    def __init__(self) -> None:
        self._start = torch.cuda.Event(enable_timing=True)
        self._end = torch.cuda.Event(enable_timing=True)
        self.ms = 0.0

    def __enter__(self) -> "CudaTimer":
        self._start.record()
        return self

    def __exit__(self, *exc: object) -> None:
        self._end.record()
        self._end.synchronize()
        self.ms = self._start.elapsed_time(self._end)
