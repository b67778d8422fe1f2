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
``torchft/checkpointing.py:34-270``; the NVLink peer-to-peer transport for GPUs of one
NVSwitch domain lives in ``torchft_b200.parallel.nvlink_heal``.
"""

from __future__ import annotations

import io
import logging
import socket
import threading
import urllib.request
from abc import ABC, abstractmethod
from contextlib import contextmanager
from datetime import timedelta
from http.server import BaseHTTPRequestHandler
from typing import Dict, Generator, Generic, List, Optional, TypeVar

import torch

from torchft_b200.http import advertised_host, make_http_server

logger: logging.Logger = logging.getLogger(__name__)

T = TypeVar("T")


def _compact(state: object) -> object:
    """Tensors of a state dict as stand-alone CPU tensors.

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


class CheckpointServer(CheckpointTransport[T]):
    """HTTP transport; one server per rank, started on an ephemeral port."""

    def __init__(self, timeout: timedelta) -> None:
        # The gate lock is HELD while serving is disallowed.
        self._checkpoint_lock = threading.Lock()
        self._disallowed = False
        self._step = -1
        self._timeout = timeout
        self._state_dict: Optional[T] = None
        self._stopped = False
        self.disallow_checkpoint()

        transport = self

        class RequestHandler(BaseHTTPRequestHandler):
            timeout = transport._timeout.total_seconds()  # per-connection socket timeout

            def do_GET(self) -> None:  # noqa: N802 - http.server API
                try:
                    with _timed_acquire(transport._checkpoint_lock, transport._timeout):
                        step = transport._step
                        prefix = "/checkpoint/"
                        if self.path != f"{prefix}{step}":
                            self.send_response(400)
                            self.send_header("Content-type", "text/plain")
                            self.end_headers()
                            self.wfile.write(
                                f"invalid checkpoint requested, serving {step} but got {self.path}".encode()
                            )
                            return
                        self.send_response(200)
                        self.send_header("Content-type", "application/octet-stream")
                        self.end_headers()
                        torch.save(_compact(transport._state_dict), self.wfile)
                except Exception as e:  # noqa: BLE001 - reported to the client
                    logger.exception(f"exception while serving checkpoint: {e}")
                    try:
                        self.send_response(500)
                        self.send_header("Content-type", "text/plain")
                        self.end_headers()
                        self.wfile.write(str(e).encode())
                    except Exception:  # noqa: BLE001 - peer already gone
                        pass

            def log_message(self, fmt: str, *args: object) -> None:
                logger.debug(fmt % args)

        self._server = make_http_server(0, RequestHandler)
        logger.info(f"checkpoint server listening on {self.address()}")
        self._thread = threading.Thread(target=self._serve, daemon=True, name="tft_checkpoint_server")
        self._thread.start()

    @classmethod
    def load_from_address(cls, address: str, timeout: timedelta) -> T:
        """Streams and unpickles the checkpoint at ``address``."""
        logger.info(f"fetching checkpoint from {address}")
        with urllib.request.urlopen(address, timeout=timeout.total_seconds()) as f:
            # torch.load needs a seekable file; a buffered read of the stream keeps one copy.
            data = io.BytesIO(f.read())
        # Non-tensor state (schedulers, counters, ...) is allowed, hence weights_only=False.
        return torch.load(data, weights_only=False)

    def address(self) -> str:
        """``http://<host>:<port>/checkpoint/`` -- append the step to fetch."""
        port = self._server.socket.getsockname()[1]
        return f"http://{advertised_host(socket.gethostname())}:{port}/checkpoint/"

    def _serve(self) -> None:
        try:
            self._server.serve_forever()
        except Exception as e:  # noqa: BLE001
            logger.exception(f"checkpoint server crashed: {e}")

    def disallow_checkpoint(self) -> None:
        if not self._disallowed:
            self._disallowed = True
            self._checkpoint_lock.acquire()

    def allow_checkpoint(self, step: int) -> None:
        self._step = step
        if self._disallowed:
            self._disallowed = False
            self._checkpoint_lock.release()

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

    def metadata(self) -> str:
        return self.address()

    def send_checkpoint(self, dst_ranks: List[int], step: int, state_dict: T, timeout: timedelta) -> None:
        # Nothing is pushed: the state dict is served by reference while the gate is open.
        self._state_dict = state_dict
        self.allow_checkpoint(step)

    def recv_checkpoint(self, src_rank: int, metadata: str, step: int, timeout: timedelta) -> T:
        return self.load_from_address(f"{metadata}{step}", timeout)
