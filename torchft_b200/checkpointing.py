"""Live-recovery checkpoint transports.

A transport moves the state dict of a healthy replica to a recovering one while
training continues.  ``CheckpointTransport`` is the interface the ``Manager`` drives;
``CheckpointServer`` is the portable HTTP implementation: the source serves
``GET /checkpoint/<step>`` as a ``torch.save`` stream of
``{"user": ..., "torchft": {"step", "batches_committed"}}`` and the receiver loads it
with ``torch.load``.  Serving is gated: requests block until ``send_checkpoint`` opened
the gate for a step and fail once ``disallow_checkpoint`` closed it again, so the
weights cannot be read while the optimizer mutates them.

Interface, URL scheme, status codes and message texts follow the reference's
``torchft/checkpointing.py:34-270``; the gate here is a reader count under a condition
variable (several peers can be served at once, closing waits for all of them) where the
reference holds one lock.  The NVLink peer-to-peer transport for GPUs of one NVSwitch
domain lives in ``torchft_b200.parallel.nvlink_heal``.
"""

from __future__ import annotations

import io
import logging
import socket
import threading
import time
import urllib.request
from abc import ABC, abstractmethod
from contextlib import contextmanager
from datetime import timedelta
from http.server import BaseHTTPRequestHandler
from typing import Dict, Generator, Generic, Iterator, List, Optional, Tuple, Type, TypeVar

import torch

from torchft_b200.http import advertised_host, make_http_server

logger: logging.Logger = logging.getLogger(__name__)

T = TypeVar("T")

_URL_PREFIX = "/checkpoint/"


def _cuda_devices(state: object) -> List[torch.device]:
    """The CUDA devices that hold tensors of ``state``."""
    from torch.utils._pytree import tree_leaves

    found: Dict[torch.device, None] = {}
    for leaf in tree_leaves(state):
        if isinstance(leaf, torch.Tensor) and leaf.device.type == "cuda":
            found.setdefault(leaf.device, None)
    return list(found)


def _record_ready(state: object) -> Dict[torch.device, "torch.cuda.Event"]:
    """One event per CUDA device of ``state``, recorded on the caller's current stream there.

    Everything queued so far on that stream that writes the state -- the previous optimizer step, a
    recovery copy -- precedes the event, so a copy that waits for it reads final values.  The
    ``Manager`` calls this from its quorum thread, whose current stream is the device's default
    stream: training that runs on the default stream (or that joins its side streams back into it
    before the step ends, as ``HSDPEngine.state_dict`` does) is covered.
    """
    ready: Dict[torch.device, "torch.cuda.Event"] = {}
    for device in _cuda_devices(state):
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(device))
        ready[device] = event
    return ready


def _compact(state: object, ready: Optional[Dict[torch.device, "torch.cuda.Event"]] = None) -> object:
    """Tensors of a state dict as stand-alone CPU tensors.

    ``ready`` maps a CUDA device to an event that the copies from that device wait for (see
    ``_record_ready``); without it the copies are ordered after nothing.

    ``torch.save`` writes the whole storage behind every tensor and refuses storages that are
    viewed under two dtypes.  State that lives as views of one large arena (a symmetric heap, a
    flat parameter buffer) would therefore be saved with the entire arena, or not at all; a
    copy to host memory gives every tensor a storage of exactly its own size.
    """
    from torch.utils._pytree import tree_map

    side: Dict[torch.device, "torch.cuda.Stream"] = {}

    def one(x: object) -> object:
        if not isinstance(x, torch.Tensor):
            return x
        t = x.detach()
        if t.device.type == "cuda":
            # A stream of its own: the serving thread must not queue behind (or implicitly
            # synchronise with) whatever the training thread has running on this device.
            stream = side.get(t.device)
            if stream is None:
                stream = side[t.device] = torch.cuda.Stream(device=t.device)
                if ready is not None and t.device in ready:
                    stream.wait_event(ready[t.device])
            with torch.cuda.device(t.device), torch.cuda.stream(stream):
                return t.to("cpu")
        if t.device.type != "cpu":
            return t.to("cpu")
        if t.untyped_storage().nbytes() != t.numel() * t.element_size():
            return t.clone()
        return t

    return tree_map(one, state)


class CheckpointTransport(Generic[T], ABC):
    @abstractmethod
    def metadata(self) -> str:
        """Opaque string a recovering peer needs to reach this transport (sent through the quorum)."""

    @abstractmethod
    def send_checkpoint(self, dst_ranks: List[int], step: int, state_dict: T, timeout: timedelta) -> None:
        """Makes ``state_dict`` of ``step`` available to the replica ranks ``dst_ranks``."""

    def disallow_checkpoint(self) -> None:
        """Called after the step, before ``state_dict`` may change again."""

    @abstractmethod
    def recv_checkpoint(self, src_rank: int, metadata: str, step: int, timeout: timedelta) -> T:
        """Fetches the state dict of ``step`` from the peer described by ``metadata``."""

    def shutdown(self, wait: bool = True) -> None:
        """Releases sockets and threads."""


@contextmanager
def _timed_acquire(lock: threading.Lock, timeout: timedelta) -> Generator[None, None, None]:
    if not lock.acquire(timeout=timeout.total_seconds()):
        raise TimeoutError(f"timed out acquiring lock after {timeout}")
    try:
        yield
    finally:
        lock.release()


class _Served(tuple):
    """``(state dict, events that mark it final)`` as kept behind the gate."""


class _Gate(Generic[T]):
    """What may be served right now: nothing (closed), or one state dict of one step (open).

    Readers enter with ``reading()``; they wait while the gate is closed and are counted while
    they stream.  ``close()`` returns only when the last reader has left, which is what lets the
    caller change the weights afterwards.
    """

    def __init__(self) -> None:
        self._cond = threading.Condition()
        self._open = False
        self._readers = 0
        self._step = -1
        self._payload: Optional[T] = None

    def open(self, step: int, payload: T) -> None:
        with self._cond:
            self._step, self._payload, self._open = step, payload, True
            self._cond.notify_all()

    def reopen(self, step: int) -> None:
        """Opens for ``step`` with the payload of the last ``open``."""
        with self._cond:
            self._step, self._open = step, True
            self._cond.notify_all()

    def close(self) -> None:
        with self._cond:
            self._open = False
            while self._readers:
                self._cond.wait()

    @contextmanager
    def reading(self, timeout: timedelta) -> Iterator[Tuple[int, Optional[T]]]:
        deadline = time.monotonic() + timeout.total_seconds()
        with self._cond:
            while not self._open:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError(f"timed out waiting for a checkpoint to be allowed after {timeout}")
                self._cond.wait(left)
            self._readers += 1
            served = (self._step, self._payload)
        try:
            yield served
        finally:
            with self._cond:
                self._readers -= 1
                self._cond.notify_all()


def _checkpoint_handler(gate: "_Gate[object]", timeout: timedelta) -> Type[BaseHTTPRequestHandler]:
    """Request handler of one ``CheckpointServer``."""
    socket_timeout = timeout.total_seconds()

    class _Handler(BaseHTTPRequestHandler):
        timeout = socket_timeout  # per-connection socket timeout

        def _head(self, status: int, content_type: str) -> None:
            self.send_response(status)
            self.send_header("Content-type", content_type)
            self.end_headers()

        def do_GET(self) -> None:  # noqa: N802 - http.server API
            try:
                with gate.reading(timeout) as (step, state):
                    if self.path != f"{_URL_PREFIX}{step}":
                        self._head(400, "text/plain")
                        self.wfile.write(f"invalid checkpoint requested, serving {step} but got {self.path}".encode())
                        return
                    self._head(200, "application/octet-stream")
                    payload, ready = state if isinstance(state, _Served) else (state, None)
                    torch.save(_compact(payload, ready), self.wfile)
            except Exception as e:  # noqa: BLE001 - reported to the client
                logger.exception(f"exception while serving checkpoint: {e}")
                try:
                    self._head(500, "text/plain")
                    self.wfile.write(str(e).encode())
                except Exception:  # noqa: BLE001 - peer already gone
                    pass

        def log_message(self, fmt: str, *args: object) -> None:
            logger.debug(fmt % args)

    return _Handler


class CheckpointServer(CheckpointTransport[T]):
    """HTTP transport; one server per rank, started on an ephemeral port with the gate closed."""

    def __init__(self, timeout: timedelta) -> None:
        self._timeout = timeout
        self._gate: _Gate[T] = _Gate()
        self._stopped = False
        self._server = make_http_server(0, _checkpoint_handler(self._gate, timeout))  # type: ignore[arg-type]
        self._thread = threading.Thread(target=self._serve, daemon=True, name="tft_checkpoint_server")
        self._thread.start()
        logger.info(f"checkpoint server listening on {self.address()}")

    # ---- CheckpointTransport
    def metadata(self) -> str:
        return self.address()

    def send_checkpoint(self, dst_ranks: List[int], step: int, state_dict: T, timeout: timedelta) -> None:
        # Nothing is pushed: the state dict is served by reference while the gate is open.  The serving
        # thread copies from a stream of its own, which by itself is ordered after nothing: the events
        # recorded here, on the caller's streams, are what puts those copies after the kernels that
        # still write the state (the reference gets that order from torch.save running on the default stream).
        self._gate.open(step, _Served((state_dict, _record_ready(state_dict))))  # type: ignore[arg-type]

    def disallow_checkpoint(self) -> None:
        self._gate.close()

    def recv_checkpoint(self, src_rank: int, metadata: str, step: int, timeout: timedelta) -> T:
        return self.load_from_address(f"{metadata}{step}", timeout)

    def shutdown(self, wait: bool = True) -> None:
        if self._stopped:
            return
        self._stopped = True
        if wait:
            self._server.shutdown()
            self._thread.join()
        else:
            threading.Thread(target=self._server.shutdown, daemon=True).start()
        self._server.server_close()

    # ---- HTTP specifics
    def allow_checkpoint(self, step: int) -> None:
        """Re-opens the gate for ``step`` with the state dict given to the last ``send_checkpoint``."""
        self._gate.reopen(step)

    def address(self) -> str:
        """``http://<host>:<port>/checkpoint/`` -- append the step to fetch."""
        host = advertised_host(socket.gethostname())
        return f"http://{host}:{self._server.socket.getsockname()[1]}{_URL_PREFIX}"

    @classmethod
    def load_from_address(cls, address: str, timeout: timedelta) -> T:
        """Streams and unpickles the checkpoint at ``address``."""
        logger.info(f"fetching checkpoint from {address}")
        with urllib.request.urlopen(address, timeout=timeout.total_seconds()) as response:
            # torch.load needs a seekable file; a buffered read of the stream keeps one copy.
            blob = io.BytesIO(response.read())
        # Non-tensor state (schedulers, counters, ...) is allowed, hence weights_only=False.
        return torch.load(blob, weights_only=False)

    def _serve(self) -> None:
        try:
            self._server.serve_forever()
        except Exception as e:  # noqa: BLE001
            logger.exception(f"checkpoint server crashed: {e}")
