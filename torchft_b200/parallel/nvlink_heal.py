"""Live-recovery checkpoint transport over NVLink peer memory.

The HTTP transport of ``torchft_b200.checkpointing`` serialises the whole state dict with
``torch.save`` on the source, ships it over TCP and deserialises it on the receiver -- every
byte crosses host memory twice (the reference does the same,
``torchft/checkpointing.py:139-203``).  Here the bulk never leaves the GPUs:

* The source describes its state dict in a small *manifest*: every CUDA tensor that lives
  in the symmetric heap becomes ``(offset, shape, dtype)``; everything else (step counters,
  scheduler state, tensors outside the heap) is pickled into the manifest itself.
* The receiver fetches the manifest over HTTP (``GET /checkpoint/<step>``, same URL scheme
  and the same gate as the HTTP transport), maps the source's heap through its CUDA IPC
  handle and pulls each tensor with a copy kernel that reads the peer's memory directly
  (``tft_p2p_pull``), straight into its own live tensors when it was given receive targets.
* While a receiver is copying, the source keeps the gate lock held for it (a *lease*), so
  ``disallow_checkpoint()`` -- called before the optimizer may mutate the weights -- waits
  for the copy to finish exactly as it waits for an HTTP stream to finish.

Both ranks must sit on GPUs of one NVLink domain.  Rank r of the recovering replica group
pulls from rank r of the source group, so sharded state moves shard to shard.
"""

from __future__ import annotations

import ctypes
import io
import logging
import pickle
import socket
import threading
import urllib.request
import uuid
from datetime import timedelta
from http.server import BaseHTTPRequestHandler
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from torchft_b200.checkpointing import CheckpointTransport, _timed_acquire
from torchft_b200.http import advertised_host, make_http_server
from torchft_b200.ops import _lib
from torchft_b200.parallel.nvlink import SymmetricHeap, _lib_p2p, _PeerMappings, _RawCudaBuffer

logger = logging.getLogger(__name__)


class _HeapRef:
    """Placeholder of a tensor that stays in the source's heap."""

    __slots__ = ("offset", "shape", "dtype")

    def __init__(self, offset: int, shape: Tuple[int, ...], dtype: torch.dtype) -> None:
        self.offset, self.shape, self.dtype = offset, tuple(shape), dtype


def _describe(obj: Any, heap: SymmetricHeap) -> Any:
    """Replaces heap tensors by ``_HeapRef``; other values stay and get pickled."""
    if isinstance(obj, torch.Tensor):
        off = heap.offset_of(obj) if obj.is_cuda else None
        if off is not None and obj.is_contiguous() and off % 16 == 0:
            return _HeapRef(off, tuple(obj.shape), obj.dtype)
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _describe(v, heap) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_describe(v, heap) for v in obj)
    return obj


class NVLinkCheckpointTransport(CheckpointTransport[Dict[str, Any]]):
    def __init__(self, heap: SymmetricHeap, timeout: timedelta, max_blocks: int = 128,
                 copy_engine_min_bytes: int = 1 << 20) -> None:
        """``copy_engine_min_bytes``: tensors of at least this size are pulled by a copy engine
        (``cudaMemcpyAsync`` out of the peer's mapped heap), smaller ones by ``pull_copy_kernel``."""
        self._heap = heap
        self._timeout = timeout
        self._max_blocks = max_blocks
        self.copy_engine_min_bytes = copy_engine_min_bytes
        self._checkpoint_lock = threading.Lock()
        self._disallowed = False
        self._step = -1
        self._state_dict: Optional[Dict[str, Any]] = None
        self._leases: Dict[str, threading.Event] = {}
        self._ready_event: Optional[torch.cuda.Event] = None
        self._leases_lock = threading.Lock()
        self._targets_fn: Optional[Callable[[], Dict[str, Any]]] = None
        self._stream = torch.cuda.Stream(device=heap.device)
        self._stopped = False
        self.bytes_pulled = 0
        self.disallow_checkpoint()

        transport = self

        class Handler(BaseHTTPRequestHandler):
            timeout = transport._timeout.total_seconds()

            def _reply(self, code: int, body: bytes, ctype: str = "application/octet-stream") -> None:
                self.send_response(code)
                self.send_header("Content-type", ctype)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                self.wfile.flush()

            def do_GET(self) -> None:  # noqa: N802
                try:
                    if self.path.startswith("/done/"):
                        with transport._leases_lock:
                            ev = transport._leases.get(self.path[len("/done/"):])
                        if ev is not None:
                            ev.set()
                        self._reply(200, b"ok", "text/plain")
                        return
                    with _timed_acquire(transport._checkpoint_lock, transport._timeout):
                        step = transport._step
                        if self.path != f"/checkpoint/{step}":
                            self._reply(400, f"invalid checkpoint requested, serving {step} but got {self.path}".encode(), "text/plain")
                            return
                        lease = str(uuid.uuid4())
                        done = threading.Event()
                        with transport._leases_lock:
                            transport._leases[lease] = done
                        manifest = {
                            "lease": lease,
                            "handle": transport._heap.handle,
                            "heap_bytes": transport._heap.nbytes,
                            "state": _describe(transport._state_dict, transport._heap),
                        }
                        # Everything the copy will read was queued before the gate opened; wait for
                        # exactly that work.  (A full device synchronisation could wait on a
                        # collective that itself waits for the receiver: a cycle.)
                        if transport._ready_event is not None:
                            transport._ready_event.synchronize()
                        self._reply(200, pickle.dumps(manifest))
                        # hold the gate until the receiver reports that its copy finished
                        if not done.wait(transport._timeout.total_seconds()):
                            logger.warning("receiver never confirmed the end of its copy; releasing the gate")
                        with transport._leases_lock:
                            transport._leases.pop(lease, None)
                except Exception as e:  # noqa: BLE001 - reported to the client
                    logger.exception(f"exception while serving checkpoint: {e}")
                    try:
                        self._reply(500, str(e).encode(), "text/plain")
                    except Exception:  # noqa: BLE001
                        pass

            def log_message(self, fmt: str, *args: object) -> None:
                logger.debug(fmt % args)

        self._server = make_http_server(0, Handler)
        self._thread = threading.Thread(target=self._server.serve_forever, daemon=True, name="tft_nvlink_heal")
        self._thread.start()

    # ------------------------------------------------------------------ configuration
    def set_receive_targets(self, fn: Callable[[], Dict[str, Any]]) -> None:
        """``fn()`` returns this rank's own state dict (same structure as the one it would send).

        With targets, tensors are pulled directly into the live destination tensors and no
        second copy of the state ever exists on the receiver.
        """
        self._targets_fn = fn

    def bind_manager(self, manager: Any) -> None:
        self.set_receive_targets(manager._manager_state_dict)

    def address(self) -> str:
        port = self._server.socket.getsockname()[1]
        return f"http://{advertised_host(socket.gethostname())}:{port}/checkpoint/"

    # ------------------------------------------------------------------ CheckpointTransport
    def metadata(self) -> str:
        return self.address()

    def disallow_checkpoint(self) -> None:
        if not self._disallowed:
            self._disallowed = True
            self._checkpoint_lock.acquire()

    def allow_checkpoint(self, step: int) -> None:
        self._step = step
        if self._disallowed:
            self._disallowed = False
            self._checkpoint_lock.release()

    def send_checkpoint(self, dst_ranks: List[int], step: int, state_dict: Dict[str, Any], timeout: timedelta) -> None:
        self._state_dict = state_dict
        with torch.cuda.device(self._heap.device):
            self._ready_event = torch.cuda.Event()
            self._ready_event.record(torch.cuda.current_stream())
        self.allow_checkpoint(step)

    def _peer_ptr(self, handle: bytes) -> int:
        """Maps the sender's heap for one transfer; ``recv_checkpoint`` unmaps it again, so that a
        sender that later leaves does not keep its memory pinned through this process."""
        if handle == self._heap.handle:
            return self._heap.ptr  # loop-back (tests): a process cannot open its own handle
        return _PeerMappings.acquire(handle, self._heap.device)

    def _pull(self, dst: torch.Tensor, src_ptr: int, nbytes: int) -> None:
        lib = _lib_p2p()
        if not hasattr(lib.tft_p2p_pull, "_tft_ready"):
            lib.tft_p2p_pull.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
            lib.tft_p2p_pull.restype = ctypes.c_int
            lib.tft_p2p_pull._tft_ready = True  # type: ignore[attr-defined]
        if nbytes >= self.copy_engine_min_bytes:
            # big tensors go through a copy engine: link rate, no SM involved
            if not hasattr(lib.tft_p2p_pull_ce, "_tft_ready"):
                lib.tft_p2p_pull_ce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
                lib.tft_p2p_pull_ce.restype = ctypes.c_int
                lib.tft_p2p_pull_ce._tft_ready = True  # type: ignore[attr-defined]
            _lib.check(lib.tft_p2p_pull_ce(dst.data_ptr(), src_ptr, nbytes, self._stream.cuda_stream), "tft_p2p_pull_ce")
            self.bytes_pulled += nbytes
            return
        main = nbytes // 16 * 16
        if main and dst.data_ptr() % 16 == 0 and src_ptr % 16 == 0:
            _lib.check(lib.tft_p2p_pull(dst.data_ptr(), src_ptr, main, self._max_blocks, self._stream.cuda_stream), "tft_p2p_pull")
            _lib.count_launch()
        else:
            main = 0
        if main < nbytes:  # ragged tail or unaligned tensor: plain device copy of the rest
            src = torch.as_tensor(_RawCudaBuffer(src_ptr + main, nbytes - main), device=dst.device)
            dst.view(-1).view(torch.uint8)[main:].copy_(src, non_blocking=True)
        self.bytes_pulled += nbytes

    def _materialise(self, desc: Any, target: Any, base: int) -> Any:
        if isinstance(desc, _HeapRef):
            numel = 1
            for s in desc.shape:
                numel *= s
            nbytes = numel * torch.empty((), dtype=desc.dtype).element_size()
            if (isinstance(target, torch.Tensor) and target.is_cuda and target.is_contiguous()
                    and tuple(target.shape) == desc.shape and target.dtype == desc.dtype):
                dst = target
            else:
                dst = torch.empty(desc.shape, dtype=desc.dtype, device=self._heap.device)
            self._pull(dst, base + desc.offset, nbytes)
            return dst
        if isinstance(desc, dict):
            return {k: self._materialise(v, target.get(k) if isinstance(target, dict) else None, base) for k, v in desc.items()}
        if isinstance(desc, (list, tuple)):
            tl = target if isinstance(target, (list, tuple)) and len(target) == len(desc) else [None] * len(desc)
            return type(desc)(self._materialise(v, t, base) for v, t in zip(desc, tl))
        return desc

    def recv_checkpoint(self, src_rank: int, metadata: str, step: int, timeout: timedelta) -> Dict[str, Any]:
        with urllib.request.urlopen(f"{metadata}{step}", timeout=timeout.total_seconds()) as f:
            manifest = pickle.loads(f.read())
        mapped = False
        try:
            base = self._peer_ptr(manifest["handle"])
            mapped = manifest["handle"] != self._heap.handle
            targets = self._targets_fn() if self._targets_fn is not None else None
            with torch.cuda.device(self._heap.device), torch.cuda.stream(self._stream):
                state = self._materialise(manifest["state"], targets, base)
            self._stream.synchronize()
        finally:
            if mapped:
                self._stream.synchronize()  # also on the error path: nothing queued may outlive the mapping
                _PeerMappings.release(manifest["handle"], self._heap.device)
            done_url = metadata.rsplit("/checkpoint/", 1)[0] + f"/done/{manifest['lease']}"
            try:
                urllib.request.urlopen(done_url, timeout=timeout.total_seconds()).read()
            except Exception as e:  # noqa: BLE001 - the source releases the gate after its own timeout
                logger.warning(f"could not confirm the end of the copy to the source: {e}")
        return state

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
