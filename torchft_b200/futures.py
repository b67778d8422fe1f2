"""Deadlines for ``torch.futures.Future``.

``future_timeout(fut, timeout)`` returns a future that mirrors ``fut`` but fails with
``TimeoutError`` if ``fut`` has not completed in time; ``future_wait`` blocks with a
deadline.  One daemon thread owns a heap of deadlines (started lazily, shared by the
whole process); completing the source future early simply wins the race.

Same contract as the reference's ``torchft/futures.py:12-165`` (message text
``"future did not complete within ..."`` included), built on a heap + condition
variable instead of an asyncio loop.
"""

from __future__ import annotations

import heapq
import itertools
import threading
import time
from datetime import timedelta
from typing import Callable, List, Optional, Tuple, TypeVar
from unittest.mock import Mock

from torch.futures import Future

T = TypeVar("T")


class _DeadlineThread:
    def __init__(self) -> None:
        self._cv = threading.Condition()
        self._heap: List[Tuple[float, int, Callable[[], None]]] = []
        self._cancelled: set = set()
        self._counter = itertools.count()
        self._thread: Optional[threading.Thread] = None

    def _ensure_started(self) -> None:
        if self._thread is None or not self._thread.is_alive():
            self._thread = threading.Thread(target=self._run, name="tft_deadlines", daemon=True)
            self._thread.start()

    def schedule(self, delay_s: float, fn: Callable[[], None]) -> int:
        with self._cv:
            self._ensure_started()
            handle = next(self._counter)
            heapq.heappush(self._heap, (time.monotonic() + max(delay_s, 0.0), handle, fn))
            self._cv.notify()
            return handle

    def cancel(self, handle: int) -> None:
        with self._cv:
            self._cancelled.add(handle)
            self._cv.notify()

    def _run(self) -> None:
        while True:
            with self._cv:
                while True:
                    # drop cancelled entries sitting at the top
                    while self._heap and self._heap[0][1] in self._cancelled:
                        self._cancelled.discard(heapq.heappop(self._heap)[1])
                    if not self._heap:
                        self._cancelled.clear()
                        self._cv.wait()
                        continue
                    now = time.monotonic()
                    if self._heap[0][0] <= now:
                        _, _, fn = heapq.heappop(self._heap)
                        break
                    self._cv.wait(self._heap[0][0] - now)
            try:
                fn()
            except Exception:  # a callback must never kill the timer thread
                pass


_DEADLINES = _DeadlineThread()


def future_timeout(fut: "Future[T]", timeout: timedelta) -> "Future[T]":
    """Returns a future completing like ``fut`` or failing with ``TimeoutError`` after ``timeout``."""
    if isinstance(fut, Mock):
        return fut
    out: Future = Future()
    lock = threading.Lock()
    done = [False]

    def finish(setter: Callable[[], None]) -> None:
        with lock:
            if done[0]:
                return
            done[0] = True
        setter()

    def on_deadline() -> None:
        finish(lambda: out.set_exception(TimeoutError(f"future did not complete within {timeout}")))

    handle = _DEADLINES.schedule(timeout.total_seconds(), on_deadline)

    def on_done(f: "Future[T]") -> None:
        _DEADLINES.cancel(handle)
        try:
            value = f.value()
        except Exception as e:  # noqa: BLE001 - forwarded to the caller
            err = e
            finish(lambda: out.set_exception(err))
        else:
            finish(lambda: out.set_result(value))

    fut.add_done_callback(on_done)
    return out


def future_wait(fut: "Future[T]", timeout: timedelta) -> T:
    """Blocks until ``fut`` completes or raises ``TimeoutError`` after ``timeout``."""
    if isinstance(fut, Mock):
        return fut.wait()
    event = threading.Event()
    fut.add_done_callback(lambda _f: event.set())
    if not event.wait(timeout.total_seconds()):
        raise TimeoutError(f"future did not complete within {timeout}")
    return fut.wait()
