"""NVLink peer-memory communication: symmetric heap, communicators, process group.

``SymmetricHeap``       one cudaMalloc'ed region per process, exported with CUDA IPC.  Tensors
                        carved from it sit at the same offset on every rank, so a kernel
                        can address any peer's copy.
``NVLinkCommunicator``  a set of peers that mapped each other's heaps, plus a signalling
                        channel in the heap header.  ``configure`` re-targets it at a new
                        membership (handles travel through the quorum's store prefix); its
                        collectives are single kernels from ``csrc/kernels/p2p_comm.cu``
                        whose waits are bounded, so a dead peer yields an error status
                        instead of a hang.
``ProcessGroupNVLink``  the torchft ``ProcessGroup`` contract on top of it (backend name
                        ``torchft-nvlink``), with the fused ``allreduce_scaled`` that
                        ``Manager.allreduce`` uses.
``NVLinkShardComm``     reduce-scatter / all-gather for the shard dimension of HSDP.

All ranks must live on GPUs of one NVLink/NVSwitch domain (one node).  The reference has
no counterpart: it delegates to NCCL (``torchft/process_group.py:320-336``).
"""

from __future__ import annotations

import ctypes
import logging
import threading
import time
import zlib
from datetime import timedelta
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch.distributed import Store
from torch.distributed.distributed_c10d import ReduceOp, Work
from torch.futures import Future

from torchft_b200.ops import _lib
from torchft_b200.process_group import ProcessGroup, create_store_client

logger = logging.getLogger(__name__)

MAX_RANKS = 8
_PROTOS_DONE = False


def _lib_p2p() -> ctypes.CDLL:
    global _PROTOS_DONE
    lib = _lib.lib()
    if not _PROTOS_DONE:
        P, I, L, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_uint
        head = [P, I, I, U, U, I, P, P]  # heaps, rank, world, epoch, seq, timeout_ms, abort, status
        lib.tft_p2p_header_bytes.restype = L
        lib.tft_p2p_header_bytes.argtypes = []
        for name, args in {
            "tft_p2p_heap_alloc": [L, P, P],
            "tft_p2p_heap_free": [P],
            "tft_p2p_peer_open": [P, P],
            "tft_p2p_peer_close": [P],
            "tft_p2p_abort_word_alloc": [P, P],
            "tft_p2p_reset_channel": [P, I, P],
            "tft_p2p_allreduce": head + [L, L, I, F, I, I, P],
            "tft_p2p_reduce_scatter": head + [L, L, I, F, I, P],
            "tft_p2p_all_gather": head + [L, L, I, P],
            "tft_p2p_all_gather_ce": head + [L, L, I, P],
            "tft_p2p_reduce_scatter_ce": head + [L, L, I, F, P, I, I, P],
            "tft_p2p_allreduce_ce": head + [L, L, I, F, P, I, P],
            "tft_p2p_allreduce_oneshot": head + [L, L, I, F, I, P],
            "tft_p2p_broadcast": head + [L, L, I, I, P],
            "tft_p2p_barrier": head + [P],
            "tft_ag_gemm_bf16": head + [P, L, P, I, I, I, I, I, P, I, P],
            "tft_gemm_rs_bf16": head + [P, P, P, I, I, I, I, I, I, L, L, I, P],
            "tft_diloco_outer": head + [L, L, P, P, P, P, L, I, F, F, F, I, I, I, P, I, P],
        }.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = I
        _PROTOS_DONE = True
    return lib


class _RawCudaBuffer:
    """Exposes raw device memory to ``torch.as_tensor`` without copying."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class _PeerMappings:
    """Process-wide table of peer heaps mapped into this process: one CUDA-IPC mapping per handle,
    reference counted.  A peer's heap stays allocated on ITS GPU for as long as any process keeps it
    mapped, also after the peer has exited, so a mapping is closed as soon as its last user (a
    communicator whose membership no longer has the peer, a finished heal transfer) lets go of it:
    the replacement of a departed replica needs that memory for its own heap."""

    _lock = threading.Lock()
    _table: Dict[bytes, List[int]] = {}  # handle -> [pointer, references]

    @classmethod
    def acquire(cls, handle: bytes, device: torch.device) -> int:
        with cls._lock:
            entry = cls._table.get(handle)
            if entry is None:
                out = ctypes.c_void_p()
                with torch.cuda.device(device):
                    _lib.check(_lib_p2p().tft_p2p_peer_open(handle, ctypes.byref(out)), "tft_p2p_peer_open")
                entry = cls._table[handle] = [int(out.value), 0]
            entry[1] += 1
            return entry[0]

    @classmethod
    def release(cls, handle: bytes, device: torch.device) -> None:
        """The caller guarantees that nothing it queued on the device still uses the mapping."""
        with cls._lock:
            entry = cls._table.get(handle)
            if entry is None:
                return
            entry[1] -= 1
            if entry[1] > 0:
                return
            del cls._table[handle]
            with torch.cuda.device(device):
                _lib_p2p().tft_p2p_peer_close(ctypes.c_void_p(entry[0]))

    @classmethod
    def open_count(cls) -> int:
        with cls._lock:
            return len(cls._table)


class SymmetricHeap:
    """Device memory that peers can map.  Bump allocator; nothing is ever freed individually."""

    _instances: Dict[int, "SymmetricHeap"] = {}

    def __init__(self, nbytes: int, device: Optional[torch.device] = None) -> None:
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        lib = _lib_p2p()
        self.header_bytes = int(lib.tft_p2p_header_bytes())
        self.nbytes = (int(nbytes) + self.header_bytes + 255) // 256 * 256
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            _lib.check(lib.tft_p2p_heap_alloc(self.nbytes, ctypes.byref(ptr), handle), "tft_p2p_heap_alloc")
        self.ptr = int(ptr.value)
        self.handle = bytes(handle)
        self._bytes = torch.as_tensor(_RawCudaBuffer(self.ptr, self.nbytes), device=self.device)
        self._cursor = self.header_bytes
        self._pool = None
        self._pool_allocator = None
        self._channels = 0
        self._lock = threading.Lock()

    @classmethod
    def get(cls, nbytes: int = 1 << 30, device: Optional[torch.device] = None) -> "SymmetricHeap":
        """Process-wide heap of the current device (created on first use with ``nbytes``)."""
        idx = torch.cuda.current_device() if device is None else (device.index or 0)
        heap = cls._instances.get(idx)
        if heap is None:
            heap = cls(nbytes, torch.device("cuda", idx))
            cls._instances[idx] = heap
        return heap

    def new_channel(self) -> int:
        with self._lock:
            ch = self._channels
            if ch >= 16:
                raise RuntimeError("all 16 signalling channels of the heap are in use")
            self._channels += 1
            return ch

    def free_bytes(self) -> int:
        return self.nbytes - self._cursor

    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A zero-initialised 1-D tensor inside the heap (256-byte aligned)."""
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        with self._lock:
            start = (self._cursor + 255) // 256 * 256
            if start + nbytes > self.nbytes:
                raise RuntimeError(
                    f"symmetric heap exhausted: need {nbytes} bytes, {self.nbytes - start} left of {self.nbytes}"
                )
            self._cursor = start + nbytes
        return self._bytes[start : start + nbytes].view(dtype)

    def mem_pool(self, nbytes: int) -> "torch.cuda.MemPool":
        """A ``torch.cuda.MemPool`` whose memory is a slice of ``nbytes`` of this heap.

        Tensors allocated under ``torch.cuda.use_mem_pool(pool)`` -- by anyone, including libraries that
        allocate for themselves -- then lie inside the heap.  Meant for set-up time: wrap a model in
        ``DistributedDataParallel`` under it and its gradient buckets are heap tensors, which
        ``ProcessGroupNVLink`` reduces in place instead of staging them.  Every rank must make the same
        allocations in the same order (the collectives address peers by offset).  One pool per heap.
        """
        if self._pool is None:
            from torchft_b200.utils import build

            lib = _lib_p2p()
            region = self.alloc(nbytes + 512, torch.uint8)
            start = (region.data_ptr() + 511) // 512 * 512
            lib.tft_pool_bind.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64]
            lib.tft_pool_bind.restype = ctypes.c_int
            _lib.check(lib.tft_pool_bind(self.device.index or 0, start, nbytes), "tft_pool_bind")
            allocator = torch.cuda.memory.CUDAPluggableAllocator(str(build.kernels_lib_path()), "tft_pool_malloc", "tft_pool_free")
            self._pool_allocator = allocator  # must outlive the pool
            self._pool = torch.cuda.MemPool(allocator.allocator())
        return self._pool

    def allocating(self, nbytes: int):
        """Context manager: CUDA allocations of this thread on this device come from the heap (see ``mem_pool``)."""
        return torch.cuda.use_mem_pool(self.mem_pool(nbytes), device=self.device)

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        """Byte offset of ``t`` inside the heap, or None if it lives elsewhere."""
        p = t.data_ptr()
        if self.ptr <= p and p + t.numel() * t.element_size() <= self.ptr + self.nbytes:
            return p - self.ptr
        return None


class _Watcher:
    """Completes futures once their CUDA event fired, turning a device status into an exception."""

    def __init__(self) -> None:
        self._cv = threading.Condition()
        self._items: List[Tuple[torch.cuda.Event, Future, object, torch.Tensor, str]] = []
        self._thread: Optional[threading.Thread] = None

    def submit(self, event: torch.cuda.Event, fut: Future, result: object, status_host: torch.Tensor, what: str) -> None:
        with self._cv:
            if self._thread is None or not self._thread.is_alive():
                self._thread = threading.Thread(target=self._run, daemon=True, name="tft_nvlink_watcher")
                self._thread.start()
            self._items.append((event, fut, result, status_host, what))
            self._cv.notify()

    def _run(self) -> None:
        while True:
            with self._cv:
                while not self._items:
                    self._cv.wait()
                event, fut, result, status_host, what = self._items.pop(0)
            try:
                event.synchronize()
                code = int(status_host.item())
                if code != 0:
                    fut.set_exception(TimeoutError(f"{what}: device-side wait gave up (status {code}); a peer is gone or slow"))
                else:
                    fut.set_result(result)
            except Exception as e:  # noqa: BLE001 - forwarded through the future
                if not fut.done():
                    fut.set_exception(e)


_WATCHER = _Watcher()


class _StreamWork(dist._Work):
    """Work that ran on a side stream.

    ``wait`` blocks the calling thread until the kernel has finished (at most ``timeout``), raises
    ``TimeoutError`` if a device-side wait inside it gave up, and orders the caller's current stream
    after it.  Blocking is what lets a caller that only ever calls ``wait()`` (FSDP2 through
    ``ManagedProcessGroup``) learn of a failed collective; ``get_future`` reports the same outcome
    without blocking.
    """

    def __init__(self, event: torch.cuda.Event, fut: Future) -> None:
        super().__init__()
        self._event = event
        self._fut = fut

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        if timeout is not None:
            deadline = time.monotonic() + timeout.total_seconds()
            while not self._fut.done():
                if time.monotonic() > deadline:
                    raise TimeoutError(f"NVLink collective did not finish within {timeout}")
                time.sleep(0.0005)
        self._fut.wait()  # raises what the watcher recorded (device status, CUDA error)
        torch.cuda.current_stream().wait_event(self._event)
        return True

    def get_future(self) -> Future:
        return self._fut


class NVLinkCommunicator:
    def __init__(self, heap: SymmetricHeap, timeout: timedelta = timedelta(seconds=10), max_blocks: int = 64,
                 copy_engine_min_bytes: Optional[int] = None, oneshot_max_bytes: int = 0) -> None:
        """
        Args:
            oneshot_max_bytes: allreduce buffers up to this size (at most 128 KiB) use the one-block
                one-shot kernel instead of the two-shot one (0: never).  Every member must use the same value.
            timeout: budget of every device-side wait (a peer that does not show up within it
                makes the collective fail with a status instead of hanging)
            max_blocks: thread blocks per collective kernel (SMs lent to communication)
            copy_engine_min_bytes: allreduce buffers of at least this size move by the copy engines
                (see ``allreduce_``); ``None`` keeps every size on the fused kernel
        """
        self.copy_engine_min_bytes = copy_engine_min_bytes
        self.oneshot_max_bytes = min(int(oneshot_max_bytes), 128 << 10)
        self.heap = heap
        self.device = heap.device
        self.channel = heap.new_channel()
        self.timeout_ms = max(int(timeout.total_seconds() * 1000), 1)
        self.max_blocks = max_blocks
        self.rank = 0
        self.world = 1
        self.epoch = 0
        self.seq = 0
        self._peers: Dict[bytes, int] = {}  # handle -> mapped pointer, for the peers of the current membership
        self._heaps = (ctypes.c_void_p * MAX_RANKS)()
        self._heaps[0] = heap.ptr
        lib = _lib_p2p()
        host, dev = ctypes.c_void_p(), ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.tft_p2p_abort_word_alloc(ctypes.byref(host), ctypes.byref(dev)), "tft_p2p_abort_word_alloc")
        self._abort_host = ctypes.cast(host, ctypes.POINTER(ctypes.c_int))
        self._abort_dev = dev
        self._status_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.stream = torch.cuda.Stream(device=self.device)
        self._bound: Optional[Tuple[Store, str]] = None
        self._generation = 0
        self._status_pinned: Optional[torch.Tensor] = None
        self._rs_ce_stage: Optional[torch.Tensor] = None  # local staging of the copy-engine reduce-scatter
        self._rs_stage: Optional[torch.Tensor] = None  # staging area of the wgrad GEMM fused with reduce-scatter
        self._rs_flags: Optional[torch.Tensor] = None
        self._block_ready: Optional[torch.Tensor] = None  # per-block counters of the fused all-gather GEMM
        self._phase_flag: Optional[torch.Tensor] = None  # phase word of the fused DiLoCo outer step

    # ------------------------------------------------------------------ membership
    @staticmethod
    def epoch_of(epoch_key) -> int:
        """The 11-bit membership tag (1..2047) that every flag of a membership carries.

        An integer (the quorum id, a generation counter) maps to ``n mod 2047 + 1``, so consecutive
        memberships always differ and two equal tags are 2047 reconfigurations apart.  A string that
        ends in ``.../<integer>`` or ``.../<integer>/<rank>`` (the store prefix the ``Manager`` hands
        to ``configure``: ``host:port/torchft/<quorum_id>/<rank>``) is read as that integer; any other
        string is hashed, which keeps distinct names apart only with probability 2046/2047.
        """
        if isinstance(epoch_key, int):
            return epoch_key % 2047 + 1
        parts = [p for p in str(epoch_key).split("/") if p]
        if "torchft" in parts[:-1]:
            tail = parts[parts.index("torchft") + 1]
            if tail.isdigit():
                return int(tail) % 2047 + 1
        if parts and parts[-1].isdigit():
            return int(parts[-1]) % 2047 + 1
        return (zlib.crc32(str(epoch_key).encode()) % 2047) + 1

    def configure(self, store: Store, rank: int, world: int, epoch_key) -> None:
        """Joins the membership identified by ``store`` (a prefix unique to it).

        Exchanges heap handles, maps new peers, clears this communicator's flags and
        synchronises through the store so nobody signals into a header that is about to
        be cleared.  ``epoch_key`` names the membership (see ``epoch_of``); every member must
        pass the same one.
        """
        if world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks per NVLink communicator, got {world}")
        lib = _lib_p2p()
        self.rank, self.world = rank, world
        self.epoch = self.epoch_of(epoch_key)
        self.seq = 0
        with torch.cuda.device(self.device):
            # Nothing of the old membership may still run.  The abort word is cleared only afterwards:
            # kernels that an abort() was meant to end must still see it while they drain.
            torch.cuda.synchronize(self.device)
            self._abort_host[0] = 0
            self._status_dev.zero_()
            _lib.check(lib.tft_p2p_reset_channel(self.heap.ptr, self.channel, _lib.stream_ptr()), "tft_p2p_reset_channel")
            torch.cuda.synchronize(self.device)
        if world == 1:
            self._heaps[0] = self.heap.ptr
            self._keep_peers({})
            return
        store.set(f"handle/{rank}", self.heap.handle)
        store.set(f"nbytes/{rank}", str(self.heap.nbytes))
        peers: Dict[bytes, int] = {}
        for r in range(world):
            if r == rank:
                self._heaps[r] = self.heap.ptr
                continue
            handle = bytes(store.get(f"handle/{r}"))
            ptr = self._peers.get(handle) or peers.get(handle)
            if ptr is None:
                ptr = _PeerMappings.acquire(handle, self.device)
            peers[handle] = ptr
            self._heaps[r] = ptr
        self._keep_peers(peers)
        # barrier through the store: every header is clean before the first flag is written
        store.set(f"ready/{rank}", b"1")
        for r in range(world):
            store.get(f"ready/{r}")

    def _keep_peers(self, peers: Dict[bytes, int]) -> None:
        """Lets go of the mappings of peers that left the membership (the device was synchronised at
        the top of ``configure``: none of this communicator's kernels still reads them)."""
        for handle in list(self._peers):
            if handle not in peers:
                _PeerMappings.release(handle, self.device)
        self._peers = peers

    def close(self) -> None:
        """Unmaps every peer (after the device has drained)."""
        torch.cuda.synchronize(self.device)
        self._keep_peers({})

    def abort(self) -> None:
        """Makes every wait of kernels in flight give up (host-side kill switch)."""
        self._abort_host[0] = 1

    def bind(self, store: Store, rank: int, world: int, name: str) -> None:
        """For a communicator whose members never change (the shard group of a replica group):
        configures it as generation 0 of ``name`` and remembers the store, so ``renew`` can move
        all members to the next generation after a failed step."""
        self._bound = (store, name)
        self._generation = 0
        self.configure(dist.PrefixStore(f"{name}/gen0", store), rank, world, 0)

    def renew(self) -> None:
        """Next generation of a bound communicator: fresh flags, sequence numbers, status and abort
        word.  Every member must call it the same number of times (e.g. whenever the group-wide
        commit vote fails)."""
        store, name = self._bound
        self._generation += 1
        self.configure(dist.PrefixStore(f"{name}/gen{self._generation}", store), self.rank, self.world, self._generation)

    def status_async(self) -> Tuple[torch.Tensor, torch.cuda.Event]:
        """Queues a copy of the status word to pinned host memory on the current stream.  Returns the
        host tensor and an event; after ``event.synchronize()`` a non-zero value means that a wait of
        an earlier collective on this stream gave up."""
        if self._status_pinned is None:
            self._status_pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_pinned.copy_(self._status_dev, non_blocking=True)
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(self.device))
        return self._status_pinned, event

    # ------------------------------------------------------------------ launch helpers
    def _head(self):
        self.seq += 1
        epoch_word = self.epoch | (self.channel << 16)
        return (self._heaps, self.rank, self.world, epoch_word, self.seq, self.timeout_ms, self._abort_dev,
                _lib.ptr(self._status_dev))

    def _offset(self, t: torch.Tensor) -> int:
        off = self.heap.offset_of(t)
        if off is None:
            raise ValueError("tensor does not live in the symmetric heap")
        assert t.is_contiguous()
        return off

    def status(self) -> int:
        """Synchronising read of the device status word (0 = healthy)."""
        return int(self._status_dev.item())

    def check(self, what: str = "NVLink collective") -> None:
        code = self.status()
        if code != 0:
            raise TimeoutError(f"{what}: device-side wait gave up (status {code}); a peer is gone or slow")

    # ------------------------------------------------------------------ collectives (on the current stream)
    def allreduce_(self, t: torch.Tensor, scale: float = 1.0, contribute: bool = True) -> None:
        """In place on a heap tensor: ``t <- scale * sum over contributing ranks``.

        Buffers of at least ``copy_engine_min_bytes`` (``None``: never) move by the copy engines between
        one-block barrier kernels, with a short local kernel for the sum, instead of by the fused
        peer-load kernel: slower in isolation for mid-sized buffers, but it leaves the SMs to the
        GEMMs it overlaps with.  Every member must use the same threshold.
        """
        if self.world == 1:
            if not contribute:
                t.zero_()
            elif scale != 1.0:
                t.mul_(scale)
            return
        nbytes = t.numel() * t.element_size()
        assert nbytes % 16 == 0, "buffer length must be a multiple of 16 bytes"
        dtype = 0 if t.dtype == torch.bfloat16 else 1
        assert t.dtype in (torch.bfloat16, torch.float32)
        if nbytes <= self.oneshot_max_bytes:
            code = _lib_p2p().tft_p2p_allreduce_oneshot(*self._head(), self._offset(t), nbytes, dtype, scale,
                                                        1 if contribute else 0, _lib.stream_ptr())
            _lib.check(code, "tft_p2p_allreduce_oneshot")
            _lib.count_launch()
            return
        if self.copy_engine_min_bytes is not None and nbytes >= self.copy_engine_min_bytes:
            if not contribute:
                t.zero_()  # rare (a healing replica): costs one pass over the buffer instead of a kernel variant
            per = -(-(nbytes // 16) // self.world) * 16
            need = per * (self.world - 1)
            if self._rs_ce_stage is None or self._rs_ce_stage.numel() < need:
                self._rs_ce_stage = torch.empty(need, dtype=torch.uint8, device=self.device)
            head = self._head()
            self.seq += 2
            code = _lib_p2p().tft_p2p_allreduce_ce(*head, self._offset(t), nbytes, dtype, scale, self._rs_ce_stage.data_ptr(),
                                                   148, _lib.stream_ptr())
            _lib.check(code, "tft_p2p_allreduce_ce")
            _lib.count_launch(4)
            return
        code = _lib_p2p().tft_p2p_allreduce(*self._head(), self._offset(t), nbytes, dtype, scale, 1 if contribute else 0,
                                            self.max_blocks, _lib.stream_ptr())
        _lib.check(code, "tft_p2p_allreduce")
        _lib.count_launch()

    def reduce_scatter_(self, full: torch.Tensor, scale: float = 1.0, engine: str = "sm", closing: bool = True) -> None:
        """``full`` holds ``world`` equal slices; rank r ends with ``scale * sum`` in slice r.

        ``engine="sm"``: one kernel loads the peers' copies of the slice over NVLink and adds them.
        ``engine="copy"``: the copy engines pull the peers' copies into a local staging area between
        barrier kernels and a short local kernel adds them (same summation order, same bits); the SMs
        stay with whatever computes beside it.  ``closing=False`` drops the final barrier: the caller
        then guarantees by other means that no peer overwrites its buffer while it may still be read
        (``HSDPEngine`` does: the commit vote of the step follows every rank's collectives).
        """
        if self.world == 1:
            if scale != 1.0:
                full.mul_(scale)
            return
        slice_bytes = full.numel() * full.element_size() // self.world
        assert slice_bytes % 16 == 0
        dtype = 0 if full.dtype == torch.bfloat16 else 1
        if engine == "sm":
            code = _lib_p2p().tft_p2p_reduce_scatter(*self._head(), self._offset(full), slice_bytes, dtype, scale,
                                                     self.max_blocks, _lib.stream_ptr())
            _lib.check(code, "tft_p2p_reduce_scatter")
            _lib.count_launch()
            return
        if engine != "copy":
            raise ValueError(f"unknown reduce-scatter engine {engine!r}")
        need = slice_bytes * (self.world - 1)
        if self._rs_ce_stage is None or self._rs_ce_stage.numel() < need:
            self._rs_ce_stage = torch.empty(need, dtype=torch.uint8, device=self.device)  # local: no peer touches it
        head = self._head()
        if closing:
            self.seq += 1
        code = _lib_p2p().tft_p2p_reduce_scatter_ce(*head, self._offset(full), slice_bytes, dtype, scale,
                                                    self._rs_ce_stage.data_ptr(), 1 if closing else 0, 148,
                                                    _lib.stream_ptr())
        _lib.check(code, "tft_p2p_reduce_scatter_ce")
        _lib.count_launch(3 if closing else 2)

    def all_gather_(self, full: torch.Tensor, engine: str = "sm") -> None:
        """Every rank ends with all ``world`` slices of ``full``; on entry slice r of rank r is valid.

        ``engine="sm"``: one kernel pushes this rank's slice into every peer's buffer.
        ``engine="copy"`` / ``"copy-push"``: the GPU's copy engines move the slices (pulled from, or
        pushed to, the peers) between two one-block barrier kernels, which leaves every SM to whatever
        computes at the same time.
        """
        if self.world == 1:
            return
        slice_bytes = full.numel() * full.element_size() // self.world
        assert slice_bytes % 16 == 0
        if engine == "sm":
            code = _lib_p2p().tft_p2p_all_gather(*self._head(), self._offset(full), slice_bytes, self.max_blocks,
                                                 _lib.stream_ptr())
            _lib.check(code, "tft_p2p_all_gather")
            _lib.count_launch()
            return
        if engine not in ("copy", "copy-push"):
            raise ValueError(f"unknown all-gather engine {engine!r}")
        head = self._head()
        self.seq += 1  # the closing barrier's sequence number
        code = _lib_p2p().tft_p2p_all_gather_ce(*head, self._offset(full), slice_bytes, 1 if engine == "copy" else 0,
                                                _lib.stream_ptr())
        _lib.check(code, "tft_p2p_all_gather_ce")
        _lib.count_launch(2)

    def all_gather_linear(self, x: torch.Tensor, w_full: torch.Tensor, out: Optional[torch.Tensor] = None,
                          copy_ctas: int = 16) -> torch.Tensor:
        """``x @ w_full.T`` where ``w_full [N, K]`` lives in the symmetric heap and only this rank's
        row slice of it is valid on entry: ONE kernel pulls the peers' slices over NVLink into
        ``w_full`` and runs the tcgen05 GEMM on the blocks as they arrive (own rows first).

        On return (stream order) ``w_full`` is completely gathered, so backward can use it as is.
        Use a communicator (channel) of its own for this: it runs on the compute stream.
        """
        assert x.dtype == torch.bfloat16 and w_full.dtype == torch.bfloat16 and w_full.is_contiguous()
        N, K = w_full.shape
        x2 = x.reshape(-1, K)
        assert x2.stride(1) == 1
        M = x2.shape[0]
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        if self.world == 1:
            from torchft_b200.ops.gemm import gemm

            gemm(x2, w_full, out)
            return out.view(*x.shape[:-1], N)
        if self._block_ready is None or self._block_ready.numel() < N // 256:
            self._block_ready = torch.zeros(max(N // 256, 256), dtype=torch.int32, device=x.device)
        code = _lib_p2p().tft_ag_gemm_bf16(
            *self._head(), x2.data_ptr(), self._offset(w_full), out.data_ptr(), M, N, K, x2.stride(0), out.stride(0),
            self._block_ready.data_ptr(), copy_ctas, _lib.stream_ptr())
        _lib.check(code, "tft_ag_gemm_bf16")
        _lib.count_launch()
        return out.view(*x.shape[:-1], N)

    def wgrad_reduce_scatter(self, dy: torch.Tensor, x: torch.Tensor, out_rows: torch.Tensor,
                             accumulate: bool = False) -> None:
        """``out_rows (+)= (sum over ranks of dy.T @ x)[rows of this rank]`` in ONE kernel.

        ``dy [tokens, M]`` and ``x [tokens, N]`` are this rank's local bf16 activations; the product
        ``dy.T @ x`` is the weight gradient ``[M, N]`` of a linear layer whose rows are sharded over the
        ranks of this communicator, and ``out_rows [M / world, N]`` is this rank's shard of it.  The
        tcgen05 GEMM's epilogue sends every tile to the rank that owns it and the owner adds the
        partial tiles up in fp32 (``csrc/kernels/gemm_rs.cu``), so neither the full local product nor a
        separate reduce-scatter exists.  Needs ``M % (128 * world) == 0`` and ``N % 256 == 0``
        (``can_fuse_wgrad``); runs on the current stream; use a communicator (channel) of its own.
        """
        assert dy.dtype == x.dtype == out_rows.dtype == torch.bfloat16
        assert dy.dim() == 2 and x.dim() == 2 and dy.shape[0] == x.shape[0]
        assert dy.stride(1) == 1 and x.stride(1) == 1 and out_rows.stride(1) == 1
        K, M = dy.shape
        N = x.shape[1]
        assert self.can_fuse_wgrad(M, N) and tuple(out_rows.shape) == (M // self.world, N)
        lib = _lib_p2p()
        need = M * N
        if self._rs_stage is None or self._rs_stage.numel() < need:
            # grows to the largest weight seen; allocate the largest one first to avoid waste
            self._rs_stage = self.heap.alloc(need, torch.bfloat16)
        flags = (M // 128) * (N // 256)
        if self._rs_flags is None or self._rs_flags.numel() < flags:
            self._rs_flags = self.heap.alloc(max(flags, 8192), torch.int32)
        code = lib.tft_gemm_rs_bf16(
            *self._head(), dy.data_ptr(), x.data_ptr(), out_rows.data_ptr(), M, N, K, dy.stride(0), x.stride(0),
            out_rows.stride(0), self._offset(self._rs_stage), self._offset(self._rs_flags), 1 if accumulate else 0,
            _lib.stream_ptr())
        _lib.check(code, "tft_gemm_rs_bf16")
        _lib.count_launch()

    def can_fuse_wgrad(self, rows: int, cols: int) -> bool:
        """Whether a weight ``[rows, cols]`` meets the tiling rules of ``wgrad_reduce_scatter``."""
        return self.world > 1 and rows % (128 * self.world) == 0 and cols % 256 == 0

    def reserve_wgrad_staging(self, rows: int, cols: int) -> None:
        """Allocates the staging area and flags for weights up to ``[rows, cols]`` now.  The heap is a
        bump allocator and every rank must allocate the same things in the same order, so do this once,
        on every rank, with the largest weight, before training."""
        if self._rs_stage is None or self._rs_stage.numel() < rows * cols:
            self._rs_stage = self.heap.alloc(rows * cols, torch.bfloat16)
        flags = max((rows // 128) * (cols // 256), 8192)
        if self._rs_flags is None or self._rs_flags.numel() < flags:
            self._rs_flags = self.heap.alloc(flags, torch.int32)

    def diloco_outer_(self, local: torch.Tensor, grad: torch.Tensor, global_in: torch.Tensor, mom_in: torch.Tensor,
                      global_out: torch.Tensor, mom_out: torch.Tensor, *, inv_n: float, lr: float, momentum: float,
                      nesterov: bool, first: bool, contribute: bool = True) -> None:
        """DiLoCo outer step in one kernel: averaged pseudo-gradient over the replicas into ``grad``
        (every rank), then momentum and new global weights into ``mom_out`` / ``global_out``.

        ``local`` and ``grad`` are flat heap tensors of the weight dtype; the others are flat tensors
        of this rank (``mom_*`` fp32).  Nothing that survives a failed step is modified: the caller
        swaps the ``*_out`` buffers in after the commit vote.
        """
        assert local.dtype == grad.dtype == global_in.dtype == global_out.dtype
        assert local.dtype in (torch.bfloat16, torch.float32)
        assert mom_in.dtype == mom_out.dtype == torch.float32
        n = local.numel()
        assert grad.numel() == n and global_in.numel() == n and global_out.numel() == n
        assert mom_in.numel() == n and mom_out.numel() == n
        if self._phase_flag is None:
            self._phase_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        code = _lib_p2p().tft_diloco_outer(
            *self._head(), self._offset(local), self._offset(grad), global_in.data_ptr(), mom_in.data_ptr(),
            global_out.data_ptr(), mom_out.data_ptr(), n, 1 if local.dtype == torch.bfloat16 else 0, inv_n, lr, momentum,
            1 if nesterov else 0, 1 if first else 0, 1 if contribute else 0, self._phase_flag.data_ptr(), 132,
            _lib.stream_ptr())
        _lib.check(code, "tft_diloco_outer")
        _lib.count_launch()

    def broadcast_(self, t: torch.Tensor, root: int) -> None:
        if self.world == 1:
            return
        nbytes = t.numel() * t.element_size()
        assert nbytes % 16 == 0
        code = _lib_p2p().tft_p2p_broadcast(*self._head(), self._offset(t), nbytes, root, self.max_blocks, _lib.stream_ptr())
        _lib.check(code, "tft_p2p_broadcast")
        _lib.count_launch()

    def barrier(self) -> None:
        if self.world == 1:
            return
        _lib.check(_lib_p2p().tft_p2p_barrier(*self._head(), _lib.stream_ptr()), "tft_p2p_barrier")
        _lib.count_launch()


class ProcessGroupNVLink(ProcessGroup):
    """Reconfigurable process group over NVLink peer memory (one node, up to 8 GPUs).

    Tensors that live in the symmetric heap are reduced in place; any other CUDA tensor
    goes through a staging buffer in the heap (two extra local copies).  Collectives run
    on the communicator's own stream, ordered after the caller's current stream; the
    returned work's future completes when the kernel finished and fails with
    ``TimeoutError`` if a device-side wait gave up.
    """

    def __init__(self, timeout: timedelta = timedelta(seconds=10), heap: Optional[SymmetricHeap] = None,
                 staging_bytes: int = 256 << 20, max_blocks: int = 64, copy_engine_min_bytes: Optional[int] = None) -> None:
        super().__init__(0, 1)
        self._heap = heap if heap is not None else SymmetricHeap.get(max(staging_bytes * 2, 1 << 30))
        self._comm = NVLinkCommunicator(self._heap, timeout=timeout, max_blocks=max_blocks,
                                        copy_engine_min_bytes=copy_engine_min_bytes)
        self._staging = self._heap.alloc(staging_bytes, torch.uint8)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._configured = False
        self._store: Optional[Store] = None
        self._first_pending = False

    @property
    def communicator(self) -> NVLinkCommunicator:
        return self._comm

    def configure(self, store_addr: str, rank: int, world_size: int) -> None:
        store = create_store_client(store_addr)
        self._comm.configure(store, rank, world_size, epoch_key=store_addr)
        self._configured = True
        self._store = store
        self._first_pending = world_size > 1

    def _rendezvous(self) -> None:
        """Host-side meeting before the FIRST collective of a membership.

        Right after a reconfiguration the members are far apart in time: one may spend many
        seconds fetching a checkpoint while the others are ready.  Meeting on the host first
        keeps the ready ones from occupying their GPU with a kernel that only waits (and from
        holding up copies that the checkpoint transfer needs on that GPU).  Later collectives
        run in the lockstep of training and go straight to the device.
        """
        if not self._first_pending:
            return
        comm = self._comm
        self._store.set(f"go/{comm.rank}", b"1")
        try:
            self._store.wait([f"go/{r}" for r in range(comm.world)], timedelta(milliseconds=comm.timeout_ms))
        except Exception as e:  # noqa: BLE001 - c10d raises its own error type on expiry
            raise TimeoutError(f"peers did not reach their first collective within {comm.timeout_ms} ms: {e}") from e
        self._first_pending = False

    def abort(self) -> None:
        self._comm.abort()

    def size(self) -> int:
        return self._comm.world

    def getBackendName(self) -> str:  # noqa: N802
        return "torchft-nvlink"

    # -- helpers
    def _launch(self, tensors: List[torch.Tensor], fn, what: str) -> Work:
        """Runs ``fn(buffer)`` per tensor on the communicator stream (staging when needed)."""
        if not self._configured:
            raise RuntimeError("torchft-nvlink process group used before configure()")
        self._rendezvous()
        comm = self._comm
        current = torch.cuda.current_stream(comm.device)
        comm.stream.wait_stream(current)
        with torch.cuda.stream(comm.stream):
            for t in tensors:
                assert t.is_cuda and t.is_contiguous(), "NVLink collectives need contiguous CUDA tensors"
                if comm.world > 1 and self._heap.offset_of(t) is None:
                    nbytes = t.numel() * t.element_size()
                    pad = (-nbytes) % 16
                    if nbytes + pad > self._staging.numel():
                        raise ValueError(f"tensor of {nbytes} bytes exceeds the staging buffer; allocate it in the heap")
                    stage = self._staging[: nbytes + pad]
                    flat = stage[:nbytes].view(t.dtype)
                    if pad:
                        stage[nbytes:].zero_()
                    flat.copy_(t.view(-1))
                    fn(stage.view(t.dtype))  # the zeroed tail rides along
                    t.view(-1).copy_(flat)
                else:
                    fn(t.view(-1))
                t.record_stream(comm.stream)
            self._status_host.copy_(comm._status_dev, non_blocking=True)
            event = torch.cuda.Event()
            event.record(comm.stream)
        fut: Future = Future()
        _WATCHER.submit(event, fut, tensors, self._status_host, what)
        return _StreamWork(event, fut)

    # -- c10d surface
    def allreduce(self, tensors: List[torch.Tensor], opts: object) -> Work:
        op = opts.reduceOp if hasattr(opts, "reduceOp") else opts
        # explicit comparisons: ``op in (SUM, AVG)`` asks the enum member first, and that one does not
        # recognise the ReduceOp object an AllreduceOptions carries
        if not (op == ReduceOp.SUM or op == ReduceOp.AVG):
            raise NotImplementedError(f"torchft-nvlink supports SUM and AVG, not {op}")
        scale = 1.0 / self._comm.world if op == ReduceOp.AVG else 1.0
        return self._launch(tensors, lambda b: self._comm.allreduce_(b, scale), "allreduce")

    def allreduce_scaled(self, tensor: torch.Tensor, scale: float, contribute: bool = True) -> Work:
        """Sum, scaling and the zero contribution of a non-participating rank in one kernel."""
        return self._launch([tensor], lambda b: self._comm.allreduce_(b, scale, contribute), "allreduce")

    def fused_outer_step(self, keep: List[torch.Tensor], **kwargs) -> Work:
        """``NVLinkCommunicator.diloco_outer_`` on the communicator stream, as a work object."""
        if not self._configured:
            raise RuntimeError("torchft-nvlink process group used before configure()")
        self._rendezvous()
        comm = self._comm
        comm.stream.wait_stream(torch.cuda.current_stream(comm.device))
        with torch.cuda.stream(comm.stream):
            comm.diloco_outer_(**kwargs)
            self._status_host.copy_(comm._status_dev, non_blocking=True)
            event = torch.cuda.Event()
            event.record(comm.stream)
        fut: Future = Future()
        _WATCHER.submit(event, fut, keep, self._status_host, "diloco_outer")
        return _StreamWork(event, fut)

    @property
    def heap(self) -> SymmetricHeap:
        return self._heap

    def broadcast(self, tensor_list: List[torch.Tensor], opts: object) -> Work:
        root = int(getattr(opts, "rootRank", 0))
        return self._launch(tensor_list, lambda b: self._comm.broadcast_(b, root), "broadcast")

    def allgather(self, output_tensors: List[List[torch.Tensor]], input_tensor: List[torch.Tensor], opts: object = None) -> Work:
        comm = self._comm
        if not self._configured:
            raise RuntimeError("torchft-nvlink process group used before configure()")
        self._rendezvous()
        current = torch.cuda.current_stream(comm.device)
        comm.stream.wait_stream(current)
        with torch.cuda.stream(comm.stream):
            for outs, inp in zip(output_tensors, input_tensor):
                nbytes = inp.numel() * inp.element_size()
                slot = (nbytes + 15) // 16 * 16
                if slot * comm.world > self._staging.numel():
                    raise ValueError("allgather exceeds the staging buffer")
                stage = self._staging[: slot * comm.world]
                stage[comm.rank * slot : comm.rank * slot + nbytes].view(inp.dtype).copy_(inp.reshape(-1))
                comm.all_gather_(stage)
                for r, o in enumerate(outs):
                    o.view(-1).copy_(stage[r * slot : r * slot + nbytes].view(inp.dtype))
            self._status_host.copy_(comm._status_dev, non_blocking=True)
            event = torch.cuda.Event()
            event.record(comm.stream)
        fut: Future = Future()
        _WATCHER.submit(event, fut, output_tensors, self._status_host, "allgather")
        return _StreamWork(event, fut)


class NVLinkShardComm:
    """Shard-dimension collectives of the HSDP engine over a fixed replica-group communicator."""

    def __init__(self, comm: NVLinkCommunicator, gather_engine: str = "sm", reduce_engine: str = "sm") -> None:
        """``gather_engine`` / ``reduce_engine``: who moves the data of the all-gather and of the
        reduce-scatter, ``"sm"`` kernels or the ``"copy"`` engines (see ``NVLinkCommunicator.all_gather_``
        and ``reduce_scatter_``)."""
        self.comm = comm
        self.gather_engine = gather_engine
        self.reduce_engine = reduce_engine

    @property
    def rank(self) -> int:
        return self.comm.rank

    @property
    def world(self) -> int:
        return self.comm.world

    def reduce_scatter_(self, full: torch.Tensor, shard_numel: int) -> None:
        # no closing barrier: the engine votes on the step only after every rank's collectives are done,
        # and gradients are not written again before that vote
        self.comm.reduce_scatter_(full, 1.0, self.reduce_engine, closing=False)

    def all_gather_(self, full: torch.Tensor, shard_numel: int) -> None:
        self.comm.all_gather_(full, self.gather_engine)

    def status_async(self):
        return self.comm.status_async()

    def renew(self) -> None:
        """After a step that did not commit: all members move to fresh flags (needs ``comm.bind``)."""
        if self.comm._bound is not None:
            self.comm.renew()
        else:
            # Not bound to a store: the members cannot meet again, but the sticky status must not fail
            # every later step.  Flags of the lost step can then still be pending on a peer; use bind().
            self.comm._status_dev.zero_()
