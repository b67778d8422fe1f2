"""Reconfigurable process groups.

A fault-tolerant job changes membership while it runs, so every process group here can
be re-pointed at a new set of peers with ``configure(store_addr, rank, world_size)``;
the ``Manager`` calls it whenever the quorum id changes, with a store prefix that is
unique per quorum.

Backends:

* ``ProcessGroupGloo`` / ``ProcessGroupNCCL`` -- stock c10d backends re-created on every
  ``configure`` (NCCL communicators are aborted first).
* ``ProcessGroupBabyGloo`` / ``ProcessGroupBabyNCCL`` -- the same, hosted in a child
  process that is killed on reconfigure, so a wedged collective can always be cleared.
* ``ProcessGroupDummy`` -- world size 1, completes everything immediately.
* ``torchft_b200.parallel.nvlink.ProcessGroupNVLink`` -- the B200-native backend: in-kernel
  peer loads/stores over NVLink with bounded waits, fused reduce + scale + cast.
* Wrappers: ``ErrorSwallowingProcessGroupWrapper`` and ``ManagedProcessGroup`` (reports
  errors to a ``Manager``; its ``size()`` is the number of participating replicas).

API surface and backend names follow the reference's ``torchft/process_group.py``.
"""

from __future__ import annotations

import logging
import multiprocessing.connection
import queue
import threading
from contextlib import nullcontext
from datetime import timedelta
from typing import TYPE_CHECKING, Any, Callable, Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch.distributed import PrefixStore, ProcessGroup as BaseProcessGroup, Store, TCPStore
from torch.distributed.distributed_c10d import (
    AllgatherOptions,
    AllreduceOptions,
    BroadcastOptions,
    ReduceOp,
    Work,
)
from torch.futures import Future

if TYPE_CHECKING:
    from torchft_b200.manager import Manager

logger: logging.Logger = logging.getLogger(__name__)


def _take_reply(replies: "mp.Queue", budget: Union[float, timedelta]) -> object:
    """Next message of a child process, within ``budget``.

    A child reports a failure by sending the exception object itself; it is re-raised in the parent,
    so the caller sees the child's error where it waited for the answer.  No message in time is a
    ``TimeoutError`` (the usual sign of a wedged collective in the child).
    """
    seconds = budget.total_seconds() if isinstance(budget, timedelta) else float(budget)
    try:
        message = replies.get(timeout=seconds)
    except queue.Empty:
        raise TimeoutError(f"no reply from the worker process within {seconds:g} s") from None
    if isinstance(message, BaseException):
        raise message
    return message


def create_store_client(store_addr: str) -> Store:
    """``host:port/prefix`` -> ``PrefixStore(prefix, TCPStore client)``."""
    host, _, rest = store_addr.partition(":")
    port, _, prefix = rest.partition("/")
    store = TCPStore(host_name=host, port=int(port), is_master=False, wait_for_workers=False)
    return PrefixStore(prefix, store)


class ProcessGroup(BaseProcessGroup):
    """Base class: a c10d process group that can be reconfigured at run time."""

    def __init__(self, *args: object, **kwargs: object) -> None:
        super().__init__(*args, **kwargs)  # type: ignore[arg-type]
        self._group_name: Optional[str] = None

    def configure(self, store_addr: str, rank: int, world_size: int) -> None:
        """Re-targets the group.  ``store_addr`` (``host:port/prefix``) is unique per quorum.

        Outstanding work of the previous configuration is abandoned; errors of older
        work objects must not be trusted after this returns.
        """
        raise NotImplementedError("not implemented")

    # -- collectives (lists of tensors, as in c10d)
    def allreduce(self, tensors: List[torch.Tensor], opts: Union[AllreduceOptions, ReduceOp]) -> Work:
        raise NotImplementedError("not implemented")

    def allgather(self, output_tensors: List[List[torch.Tensor]], input_tensor: List[torch.Tensor], opts: AllgatherOptions) -> Work:
        raise NotImplementedError("not implemented")

    def broadcast(self, tensor_list: List[torch.Tensor], opts: BroadcastOptions) -> Work:
        raise NotImplementedError("not implemented")

    def broadcast_one(self, tensor: torch.Tensor, root: int) -> Work:
        opts = BroadcastOptions()
        opts.rootRank = root
        return self.broadcast([tensor], opts)

    def allreduce_scaled(self, tensor: torch.Tensor, scale: float, contribute: bool = True) -> Work:
        """``tensor <- scale * sum_over_ranks(tensor)``; a rank with ``contribute=False`` adds zeros.

        Generic two-step form (zero fill, SUM allreduce, in-place multiply when the work
        completes).  Backends with a fused kernel override this.
        """
        if not contribute:
            tensor.zero_()
        work = self.allreduce([tensor], ReduceOp.SUM)
        if scale == 1.0:
            return work
        return _ScaledWork(work, tensor, scale)

    def size(self) -> int:
        raise NotImplementedError("not implemented")

    def getBackendName(self) -> str:  # noqa: N802 - c10d API
        raise NotImplementedError("not implemented")

    # -- registration with c10d so DeviceMesh / functional collectives can resolve the group
    def _register(self, name: str) -> str:
        group_name = f"{self.getBackendName()}:{name}"

        def create_pg(prefix_store: PrefixStore, rank: int, world_size: int, timeout: float) -> "ProcessGroup":
            return self

        devices = ["cuda", "cpu"] if torch.cuda.is_available() else ["cpu"]
        dist.Backend.register_backend(group_name, create_pg, devices=devices)
        return group_name

    def register(self, name: str) -> BaseProcessGroup:
        """Registers this group with c10d under a unique ``name`` (call once).

        A resizable world does not fit c10d's registry, so the registered group has
        world size 1 (just this rank) and its backend factory hands back ``self``.
        """
        group_name = self._register(name)
        return dist.new_group(
            ranks=[dist.get_rank()],
            backend=group_name,
            group_desc=group_name,
            timeout=timedelta(seconds=60.0),
        )

    @property
    def group_name(self) -> str:
        if self._group_name is None:
            raise ValueError("ProcessGroup name not set")
        return self._group_name

    def _set_group_name(self, name: str) -> None:
        self._group_name = name

    def unregister(self) -> None:
        dist.destroy_process_group(self)

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}()"


class _ScaledWork(dist._Work):
    """Multiplies the reduced tensor by ``scale`` once the inner work completes."""

    def __init__(self, work: Work, tensor: torch.Tensor, scale: float) -> None:
        super().__init__()
        self._work = work
        self._tensor = tensor
        self._scale = scale
        self._applied = False
        self._lock = threading.Lock()

    def _apply(self) -> None:
        with self._lock:
            if not self._applied:
                self._applied = True
                self._tensor.mul_(self._scale)

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        if timeout is not None:
            self._work.wait(timeout)
        else:
            self._work.wait()
        self._apply()
        return True

    def get_future(self) -> Future:
        def scale(fut: Future) -> object:
            value = fut.value()
            self._apply()
            return value

        return self._work.get_future().then(scale)


class ProcessGroupWrapper(ProcessGroup):
    """Holds a c10d process group and rebuilds it on every ``configure``."""

    PG_CLASS: Optional[type] = None

    def __init__(self, pg: Optional[BaseProcessGroup] = None) -> None:
        super().__init__(0, 1)
        self._pg: Optional[BaseProcessGroup] = pg

    def configure(self, store_addr: str, rank: int, world_size: int) -> None:
        pg = self._pg
        if isinstance(pg, ProcessGroup):
            pg.configure(store_addr, rank, world_size)
            return
        if pg is not None and hasattr(pg, "abort"):
            try:
                pg.abort()  # type: ignore[attr-defined]
            except Exception as e:  # noqa: BLE001 - the old group is being discarded anyway
                logger.warning(f"abort of previous process group failed: {e}")
        self._pg = None
        store = create_store_client(store_addr)
        self._pg = self._create_pg(store, rank, world_size)

    def abort(self) -> None:
        pg = self._pg
        if pg is not None and hasattr(pg, "abort"):
            pg.abort()  # type: ignore[attr-defined]

    def _create_pg(self, store: Store, rank: int, world_size: int) -> BaseProcessGroup:
        raise NotImplementedError("not implemented")

    def _require(self) -> BaseProcessGroup:
        if self._pg is None:
            raise RuntimeError(f"{self.getBackendName()} process group used before configure()")
        return self._pg

    def allreduce(self, tensors: List[torch.Tensor], opts: object) -> Work:
        return self._require().allreduce(tensors, opts)

    def allgather(self, output_tensors: List[List[torch.Tensor]], input_tensor: List[torch.Tensor], opts: object = None) -> Work:
        if opts is None:
            opts = AllgatherOptions()
        return self._require().allgather(output_tensors, input_tensor, opts)

    def broadcast(self, tensor_list: List[torch.Tensor], opts: object) -> Work:
        return self._require().broadcast(tensor_list, opts)

    def size(self) -> int:
        return self._require().size()

    @property
    def parent(self) -> Optional[BaseProcessGroup]:
        return self._pg

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(pg={self._pg})"


class ProcessGroupGloo(ProcessGroupWrapper):
    """Reconfigurable Gloo (CPU/TCP) group."""

    def __init__(self, timeout: timedelta = timedelta(seconds=60.0)) -> None:
        super().__init__()
        self._timeout = timeout

    def _create_pg(self, store: Store, rank: int, world_size: int) -> BaseProcessGroup:
        return dist.ProcessGroupGloo(store, rank, world_size, self._timeout)

    def getBackendName(self) -> str:  # noqa: N802
        return "torchft-gloo"


class ProcessGroupNCCL(ProcessGroupWrapper):
    """Reconfigurable in-process NCCL group.

    The previous communicator is aborted on ``configure``.  A collective stuck in the
    NCCL kernel can still block the stream; where that matters use
    ``ProcessGroupBabyNCCL`` or the NVLink backend whose kernels bound their own waits.
    """

    def __init__(self, timeout: timedelta = timedelta(seconds=60.0)) -> None:
        super().__init__()
        self._timeout = timeout

    def _create_pg(self, store: Store, rank: int, world_size: int) -> BaseProcessGroup:
        opts = dist.ProcessGroupNCCL.Options()
        opts._timeout = self._timeout
        pg = dist.ProcessGroupNCCL(store, rank, world_size, opts)
        return pg

    def getBackendName(self) -> str:  # noqa: N802
        return "torchft-nccl"


class _DummyWork(dist._Work):
    """A work item that was complete before it was handed out; counts how it is awaited."""

    def __init__(self, result: object, owner: Optional["ProcessGroupDummy"] = None) -> None:
        super().__init__()
        self._owner = owner
        self._done: Future = Future()
        self._done.set_result(result)

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        if self._owner is not None:
            self._owner.wait_count += 1
        return True

    def get_future(self) -> Future:
        if self._owner is not None:
            self._owner.get_future_count += 1
        return self._done


class ProcessGroupDummy(ProcessGroup):
    """A group of exactly one rank in which every collective is the identity and already complete.

    It stands in where a library insists on communicating although there is nobody to talk to yet:
    torch's ``DistributedDataParallel`` broadcasts the parameters in its constructor, which
    ``torchft_b200.ddp`` runs under this group before the real, reconfigurable group takes over.
    The counters (``configure_count``, ``wait_count``, ``get_future_count``, ``issued``) let tests
    see what the library did with it.  Reference: ``torchft/process_group.py`` (ProcessGroupDummy).
    """

    def __init__(self, rank: int, world: int) -> None:
        if (rank, world) != (0, 1):
            raise ValueError(f"a dummy group has one rank, got rank {rank} of {world}")
        super().__init__(rank, world)
        self.configure_count = 0
        self.wait_count = 0
        self.get_future_count = 0
        self.issued = 0

    def _complete(self, result: object) -> Work:
        self.issued += 1
        return _DummyWork(result, self)

    def configure(self, store_addr: str, rank: int, world_size: int) -> None:
        self.configure_count += 1

    def allreduce(self, tensors: List[torch.Tensor], opts: object) -> Work:
        return self._complete(tensors)  # a sum over one rank

    def broadcast(self, tensor_list: List[torch.Tensor], opts: object) -> Work:
        return self._complete(tensor_list)  # the root is the only rank

    def allgather(self, output_tensors: List[List[torch.Tensor]], input_tensor: List[torch.Tensor], opts: object = None) -> Work:
        for slot, mine in zip(output_tensors[0], input_tensor):
            slot.copy_(mine)
        return self._complete(output_tensors)

    def size(self) -> int:
        return 1

    def getBackendName(self) -> str:  # noqa: N802
        return "torchft-dummy"


class _ErrorSwallowingWork(dist._Work):
    def __init__(self, pg: "ErrorSwallowingProcessGroupWrapper", work: Work, default_result: object) -> None:
        super().__init__()
        self._pg = pg
        self._work = work
        self._default_result = default_result

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        try:
            if timeout is not None:
                self._work.wait(timeout)
            else:
                self._work.wait()
        except Exception as e:  # noqa: BLE001 - swallowed by design
            self._pg.report_error(e)
        return True

    def get_future(self) -> Future:
        fut = self._work.get_future()

        def callback(f: Future) -> object:
            try:
                return f.value()
            except Exception as e:  # noqa: BLE001 - swallowed by design
                self._pg.report_error(e)
                return self._default_result

        return fut.then(callback)


class ErrorSwallowingProcessGroupWrapper(ProcessGroupWrapper):
    """After the first failure every allreduce is a no-op until the next ``configure``."""

    def __init__(self, pg: ProcessGroup) -> None:
        super().__init__(pg)
        self._error: Optional[Exception] = None

    def configure(self, store_addr: str, rank: int, world_size: int) -> None:
        self._error = None
        super().configure(store_addr, rank, world_size)

    def report_error(self, e: Exception) -> None:
        """Records ``e``; later operations are skipped."""
        self._error = e

    def error(self) -> Optional[Exception]:
        return self._error

    def allreduce(self, tensors: List[torch.Tensor], opts: object) -> Work:
        if self._error is not None:
            return _DummyWork(tensors)
        try:
            return _ErrorSwallowingWork(self, super().allreduce(tensors, opts), tensors)
        except Exception as e:  # noqa: BLE001 - swallowed by design
            self.report_error(e)
            return _DummyWork(tensors)


class _ManagedWork(dist._Work):
    def __init__(self, manager: "Manager", work: Work, default_result: object) -> None:
        super().__init__()
        self._manager = manager
        self._work = work
        self._default_result = default_result

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        try:
            if self._work is not None:
                if timeout is not None:
                    self._work.wait(timeout)
                else:
                    self._work.wait()
        except Exception as e:  # noqa: BLE001 - reported, the step is discarded
            self._manager.report_error(e)
        return True

    def get_future(self) -> Future:
        return self._manager.wrap_future(self._work.get_future(), self._default_result)


class ManagedProcessGroup(ProcessGroupWrapper):
    """A process-group view of a ``Manager`` (used as the replicate dimension of HSDP).

    Operations wait for the quorum, become no-ops once the step has errored, and report
    failures to the manager instead of raising.  ``size()`` is the number of
    participating replicas, so callers that derive an averaging factor from the group
    size divide by the right number.  No scaling is applied here.
    """

    def __init__(self, manager: "Manager") -> None:
        super().__init__(manager._pg)
        self._manager = manager

    def allreduce(self, tensors: List[torch.Tensor], opts: object) -> Work:
        # Blocks until the quorum (and any reconfiguration) of this step is done.
        self._manager.wait_quorum()
        if self._manager.errored() is not None:
            return _DummyWork(tensors)
        try:
            op = opts.reduceOp if hasattr(opts, "reduceOp") else opts
            # (``op in (SUM, AVG)`` would compare the enum member first, which does not know ReduceOp objects)
            if len(tensors) == 1 and (op == ReduceOp.SUM or op == ReduceOp.AVG):
                # A replica that is still healing (or a spare) is a member of the group but its data
                # must not count, and an average is over the participants, not over the members:
                # both are what allreduce_scaled expresses (the reference hands ``opts`` to the
                # backend unchanged, so NCCL's AVG divides by the member count there).
                scale = 1.0 / max(self._manager.num_participants(), 1) if op == ReduceOp.AVG else 1.0
                work = self._manager._pg.allreduce_scaled(
                    tensors[0], scale, contribute=self._manager.is_participating())
            else:
                work = super().allreduce(tensors, opts)
        except Exception as e:  # noqa: BLE001 - reported, the step is discarded
            self._manager.report_error(e)
            return _DummyWork(tensors)
        return _ManagedWork(self._manager, work, tensors)

    def size(self) -> int:
        return self._manager.num_participants()

    def getBackendName(self) -> str:  # noqa: N802
        return self._manager._pg.getBackendName()


# =============================================================================
# Process groups hosted in a child process
# =============================================================================


class _PickleSafeOptions:
    """c10d option structs do not pickle; they cross the process boundary as dicts."""

    _TYPES = {"AllreduceOptions": AllreduceOptions, "AllgatherOptions": AllgatherOptions, "BroadcastOptions": BroadcastOptions}

    @classmethod
    def safe_args(cls, args: object) -> object:
        if isinstance(args, tuple):
            return tuple(cls.safe_args(a) for a in args)
        if isinstance(args, list):
            return [cls.safe_args(a) for a in args]
        if isinstance(args, ReduceOp):
            return {"__c10d__": "ReduceOp", "op": int(args.op) if hasattr(args, "op") else int(args)}  # type: ignore[arg-type]
        if isinstance(args, AllreduceOptions):
            return {"__c10d__": "AllreduceOptions", "reduceOp": cls.safe_args(args.reduceOp), "timeout": args.timeout}
        if isinstance(args, AllgatherOptions):
            return {"__c10d__": "AllgatherOptions", "timeout": args.timeout}
        if isinstance(args, BroadcastOptions):
            return {"__c10d__": "BroadcastOptions", "rootRank": args.rootRank, "rootTensor": args.rootTensor, "timeout": args.timeout}
        return args

    @classmethod
    def unsafe_args(cls, args: object) -> object:
        if isinstance(args, tuple):
            return tuple(cls.unsafe_args(a) for a in args)
        if isinstance(args, list):
            return [cls.unsafe_args(a) for a in args]
        if isinstance(args, dict) and "__c10d__" in args:
            kind = args["__c10d__"]
            if kind == "ReduceOp":
                return ReduceOp(ReduceOp.RedOpType(args["op"]))
            opts = cls._TYPES[kind]()
            for k, v in args.items():
                if k == "__c10d__":
                    continue
                setattr(opts, k, cls.unsafe_args(v))
            return opts
        return args


class _BabyWork(dist._Work):
    """Parent-side handle of a work item that lives in the child process."""

    def __init__(self, pg: "ProcessGroupBaby", op_id: int, stream: Optional["torch.cuda.Stream"]) -> None:
        super().__init__()
        self._pg = pg
        self._op_id = op_id
        self._stream = stream

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        return self._pg._wait(self._op_id, self._stream, timeout)

    def synchronize(self) -> None:
        self.wait()

    def get_future(self) -> Future:
        return self._pg._get_future(self._op_id)

    def __del__(self) -> None:
        try:
            self._pg._del(self._op_id)
        except Exception:  # noqa: BLE001 - interpreter shutdown / dead child
            pass


def _baby_worker(
    backend_factory: Callable[[Store, int, int, float], BaseProcessGroup],
    store_addr: str,
    rank: int,
    world_size: int,
    timeout_s: float,
    cmd_q: "mp.Queue",
    reply_q: "mp.Queue",
    event_q: "mp.Queue",
) -> None:
    """Child-process loop: owns the real process group and executes forwarded calls.

    Requests are tuples whose first element names the action; every request gets
    exactly one reply on ``reply_q`` (actions ``func``, ``wait``, ``num_active_work``)
    except ``del`` and ``future``; future completions are pushed to ``event_q``.
    """
    try:
        store = create_store_client(store_addr)
        pg = backend_factory(store, rank, world_size, timeout_s)
        reply_q.put(("ready", None))
        work: Dict[int, Work] = {}
        streams: Dict[Tuple[int, int], "torch.cuda.Stream"] = {}
        next_op = 0
        while True:
            req = cmd_q.get()
            action = req[0]
            if action == "stop":
                return
            if action == "func":
                _, name, args, kwargs, stream_key, event = req
                args = _PickleSafeOptions.unsafe_args(args)
                kwargs = {k: _PickleSafeOptions.unsafe_args(v) for k, v in kwargs.items()}
                fn = getattr(pg, name)
                if stream_key is not None:
                    # Mirror the caller's stream: one child stream per (device, parent stream).
                    if stream_key not in streams:
                        streams[stream_key] = torch.cuda.Stream(device=stream_key[0])
                    stream = streams[stream_key]
                    ctx: Any = torch.cuda.stream(stream)
                    if event is not None:
                        event.wait(stream)
                else:
                    ctx = nullcontext()
                with ctx:
                    work[next_op] = fn(*args, **kwargs)
                reply_q.put(("op", next_op))
                next_op += 1
            elif action == "wait":
                _, op_id, wait_timeout, stream_key = req
                w = work[op_id]
                if wait_timeout is not None:
                    w.wait(timedelta(seconds=wait_timeout))
                else:
                    w.wait()
                event = None
                if stream_key is not None and stream_key in streams:
                    event = torch.cuda.Event(interprocess=True)
                    event.record(streams[stream_key])
                reply_q.put(("waited", (op_id, event)))
            elif action == "del":
                work.pop(req[1], None)
            elif action == "future":
                _, op_id = req

                def done(fut: Future, op_id: int = op_id) -> None:
                    try:
                        fut.value()
                        event_q.put((op_id, True, None))
                    except Exception as e:  # noqa: BLE001 - forwarded to the parent
                        event_q.put((op_id, False, RuntimeError(f"{type(e).__name__}: {e}")))

                work[op_id].get_future().add_done_callback(done)
            elif action == "num_active_work":
                reply_q.put(("count", len(work)))
            else:
                raise ValueError(f"unknown action {action}")
    except Exception as e:  # noqa: BLE001 - the parent re-raises it
        logger.exception(f"process group worker failed: {e}")
        reply_q.put(RuntimeError(f"process group worker failed: {type(e).__name__}: {e}"))
        event_q.put(None)


class ProcessGroupBaby(ProcessGroup):
    """Runs the real process group in a spawned child so it can always be killed.

    ``configure`` terminates the previous child (and with it any stuck collective) and
    starts a new one.  CPU tensors are moved to shared memory; CUDA tensors travel as
    CUDA IPC handles and the two processes order their streams with interprocess
    events, so no host synchronisation is added.  Each child holds its own CUDA
    context (roughly 1 GB of device memory for NCCL).
    """

    def __init__(self, timeout: Union[float, timedelta] = 60.0) -> None:
        super().__init__(0, 1)
        self._world_size = -1
        self._p: Optional[mp.Process] = None
        self._cmd_q: Optional["mp.Queue"] = None
        self._reply_q: Optional["mp.Queue"] = None
        self._event_q: Optional["mp.Queue"] = None
        self._event_thread: Optional[threading.Thread] = None
        self._futures: Dict[int, Future] = {}
        self._futures_lock = threading.Lock()
        self._call_lock = threading.Lock()
        if isinstance(timeout, timedelta):
            timeout = timeout.total_seconds()
        self._timeout: float = timeout

    @classmethod
    def _create_pg(cls, store: Store, rank: int, world_size: int, timeout_s: float) -> BaseProcessGroup:
        raise NotImplementedError("not implemented")

    def _shutdown_child(self) -> None:
        if self._p is not None:
            self._p.kill()
            self._p.join(timeout=10)
            self._p = None
        if self._event_q is not None:
            try:
                self._event_q.put(None)  # wakes the event thread
            except Exception:  # noqa: BLE001
                pass
        if self._event_thread is not None:
            self._event_thread.join(timeout=5)
            self._event_thread = None
        for q in (self._cmd_q, self._reply_q, self._event_q):
            if q is not None:
                q.close()
        self._cmd_q = self._reply_q = self._event_q = None
        with self._futures_lock:
            pending, self._futures = self._futures, {}
        for fut in pending.values():
            if not fut.done():
                fut.set_exception(RuntimeError("process group was reconfigured or shut down"))

    def shutdown(self) -> None:
        self._shutdown_child()

    def configure(self, store_addr: str, rank: int, world_size: int) -> None:
        self._world_size = world_size
        self._shutdown_child()
        ctx = mp.get_context("spawn")
        self._cmd_q = ctx.Queue()
        self._reply_q = ctx.Queue()
        self._event_q = ctx.Queue()
        self._p = ctx.Process(
            target=_baby_worker,
            args=(type(self)._create_pg, store_addr, rank, world_size, self._timeout, self._cmd_q, self._reply_q, self._event_q),
            daemon=True,
        )
        self._p.start()
        self._event_thread = threading.Thread(
            target=self._event_loop, args=(self._event_q,), daemon=True, name="tft_baby_futures"
        )
        self._event_thread.start()
        # surfaces start-up failures (store unreachable, rendezvous timeout, ...)
        kind, _ = _take_reply(self._reply_q, self._timeout)  # type: ignore[misc]
        assert kind == "ready"

    def _event_loop(self, event_q: "mp.Queue") -> None:
        while True:
            try:
                item = event_q.get()
            except (EOFError, OSError, ValueError):
                return
            if item is None:
                return
            op_id, ok, err = item
            with self._futures_lock:
                fut = self._futures.pop(op_id, None)
            if fut is None:
                continue
            if ok:
                fut.set_result(None)
            else:
                fut.set_exception(err)

    def _assert_alive(self) -> None:
        p = self._p
        if p is None:
            raise RuntimeError("process group used before configure()")
        if not p.is_alive():
            raise RuntimeError(f"child process {p.pid} is dead {p.exitcode}")

    def _request(self, req: tuple, expect_reply: bool = True, timeout: Optional[float] = None) -> object:
        with self._call_lock:
            self._assert_alive()
            assert self._cmd_q is not None and self._reply_q is not None
            self._cmd_q.put(req)
            if not expect_reply:
                return None
            kind, value = _take_reply(self._reply_q, timeout if timeout is not None else self._timeout)  # type: ignore[misc]
            return value

    def _run_func(self, name: str, *args: object, **kwargs: object) -> Work:
        tensors = [t for a in args for t in (a if isinstance(a, (list, tuple)) else [a]) if isinstance(t, torch.Tensor)]
        nested = [t for a in args if isinstance(a, (list, tuple)) for l in a if isinstance(l, (list, tuple)) for t in l if isinstance(t, torch.Tensor)]
        tensors += nested
        is_cuda = any(t.is_cuda for t in tensors)
        stream = None
        stream_key = None
        event = None
        if is_cuda:
            device = next(t.device for t in tensors if t.is_cuda)
            stream = torch.cuda.current_stream(device)
            stream_key = (device.index if device.index is not None else torch.cuda.current_device(), stream.stream_id)
            event = torch.cuda.Event(interprocess=True)
            event.record(stream)
        else:
            for t in tensors:
                if not t.is_shared():
                    t.share_memory_()
        op_id = self._request(
            ("func", name, _PickleSafeOptions.safe_args(args), {k: _PickleSafeOptions.safe_args(v) for k, v in kwargs.items()}, stream_key, event)
        )
        assert isinstance(op_id, int)
        self._stream_keys = getattr(self, "_stream_keys", {})
        self._stream_keys[op_id] = stream_key
        return _BabyWork(self, op_id, stream)

    def _wait(self, op_id: int, stream: Optional["torch.cuda.Stream"], timeout: Optional[timedelta]) -> bool:
        stream_key = getattr(self, "_stream_keys", {}).get(op_id)
        t = timeout.total_seconds() if timeout is not None else None
        result = self._request(("wait", op_id, t, stream_key), timeout=t)
        assert isinstance(result, tuple)
        _, event = result
        if event is not None and stream is not None:
            event.wait(stream)
        return True

    def _get_future(self, op_id: int) -> Future:
        fut: Future = Future()
        with self._futures_lock:
            self._futures[op_id] = fut
        self._request(("future", op_id), expect_reply=False)
        return fut

    def _del(self, op_id: int) -> None:
        getattr(self, "_stream_keys", {}).pop(op_id, None)
        if self._p is not None and self._p.is_alive() and self._cmd_q is not None:
            self._cmd_q.put(("del", op_id))

    def allreduce(self, tensors: List[torch.Tensor], opts: Union[dist.AllreduceOptions, dist.ReduceOp]) -> Work:
        return self._run_func("allreduce", tensors, opts)

    def allgather(self, output_tensors: List[List[torch.Tensor]], input_tensor: List[torch.Tensor], opts: object = None) -> Work:
        if opts is None:
            opts = AllgatherOptions()
        return self._run_func("allgather", output_tensors, input_tensor, opts)

    def broadcast(self, tensor_list: List[torch.Tensor], opts: object) -> Work:
        return self._run_func("broadcast", tensor_list, opts)

    def size(self) -> int:
        return self._world_size

    def num_active_work(self) -> int:
        value = self._request(("num_active_work",))
        assert isinstance(value, int)
        return value


def _make_gloo(store: Store, rank: int, world_size: int, timeout_s: float) -> BaseProcessGroup:
    return dist.ProcessGroupGloo(store, rank, world_size, timedelta(seconds=timeout_s))


def _make_nccl(store: Store, rank: int, world_size: int, timeout_s: float) -> BaseProcessGroup:
    opts = dist.ProcessGroupNCCL.Options()
    opts._timeout = timedelta(seconds=timeout_s)
    return dist.ProcessGroupNCCL(store, rank, world_size, opts)


class ProcessGroupBabyGloo(ProcessGroupBaby):
    """Gloo in a child process (mostly useful to test the child-process machinery on CPU)."""

    _create_pg = staticmethod(_make_gloo)  # type: ignore[assignment]

    def getBackendName(self) -> str:  # noqa: N802
        return "torchft-baby-gloo"


class ProcessGroupBabyNCCL(ProcessGroupBaby):
    """NCCL in a child process: a hung communicator is cleared by killing the child.

    Tensors passed in must stay alive until the work completed, and the group uses
    about 1 GB of extra device memory for the child's CUDA context.
    """

    _create_pg = staticmethod(_make_nccl)  # type: ignore[assignment]

    def getBackendName(self) -> str:  # noqa: N802
        return "torchft-baby-nccl"


# Device-mesh glue lives in its own module; re-exported here because that is where
# users of the reference look for it (torchft/process_group.py:1057-1331).
from torchft_b200.device_mesh import (  # noqa: E402
    ManagedDeviceMesh,
    extend_device_mesh,
    ft_init_device_mesh,
)

__all__ = [
    "ProcessGroup",
    "ProcessGroupWrapper",
    "ProcessGroupGloo",
    "ProcessGroupNCCL",
    "ProcessGroupDummy",
    "ProcessGroupBaby",
    "ProcessGroupBabyGloo",
    "ProcessGroupBabyNCCL",
    "ErrorSwallowingProcessGroupWrapper",
    "ManagedProcessGroup",
    "ManagedDeviceMesh",
    "extend_device_mesh",
    "ft_init_device_mesh",
    "create_store_client",
]
