"""Per-rank fault-tolerance state machine.

One ``Manager`` lives in every rank of every replica group.  Per training step the
user (normally through ``torchft_b200.optim.Optimizer``) calls::

    manager.start_quorum()        # before forward; may run in the background
    ... forward / backward ...    # gradients flow through manager.allreduce(...)
    if manager.should_commit():   # group-wide vote
        optimizer.step()

``start_quorum`` asks the replica group's manager server (C++, hosted by local rank 0)
for a quorum; if membership changed the process group is re-pointed at the new peers,
and if this replica is behind it pulls a live checkpoint from a healthy peer while the
others keep training.  ``allreduce`` averages a tensor over the participating replicas
and never raises: an error marks the step as failed, turns the remaining allreduces of
the step into no-ops and makes ``should_commit`` return False everywhere in the group.

Behaviour and public API follow the reference's ``torchft/manager.py:73-680``.  The
averaging itself is delegated to ``ProcessGroup.allreduce_scaled`` so a backend with a
fused kernel (NVLink) does sum, 1/n scaling and the zero contribution of a healing
replica in one pass instead of three.
"""

from __future__ import annotations

import concurrent.futures
import logging
import os
import socket
import uuid
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta
from enum import Enum
from typing import TYPE_CHECKING, Callable, Dict, List, Optional, TypeVar, cast

import torch
from torch.distributed import TCPStore

from torchft_b200._control import Manager as _ManagerServer, ManagerClient
from torchft_b200.checkpointing import CheckpointServer, CheckpointTransport
from torchft_b200.futures import future_timeout
from torchft_b200.utils.tracing import trace_range

if TYPE_CHECKING:
    from torchft_b200.process_group import ProcessGroup

MANAGER_ADDR_KEY: str = "manager_addr"
MANAGER_PORT_ENV: str = "TORCHFT_MANAGER_PORT"
REPLICA_ID_KEY: str = "replica_id"

T = TypeVar("T")


class WorldSizeMode(Enum):
    """How the number of participating replicas is chosen.

    DYNAMIC: every replica of the quorum participates; gradients are divided by that count.
    FIXED_WITH_SPARES: at most ``min_replica_size`` replicas participate; the others are
    hot spares that contribute zeros but receive the averaged result.
    """

    DYNAMIC = 0
    FIXED_WITH_SPARES = 1


class Manager:
    """Fault-tolerance manager of one rank.  See the module docstring."""

    def __init__(
        self,
        pg: "ProcessGroup",
        load_state_dict: Optional[Callable[[T], None]],
        state_dict: Optional[Callable[[], T]],
        min_replica_size: int,
        use_async_quorum: bool = True,
        timeout: timedelta = timedelta(seconds=60),
        quorum_timeout: timedelta = timedelta(seconds=60),
        connect_timeout: timedelta = timedelta(seconds=60),
        rank: Optional[int] = None,
        world_size: Optional[int] = None,
        world_size_mode: WorldSizeMode = WorldSizeMode.DYNAMIC,
        store_addr: Optional[str] = None,
        store_port: Optional[int] = None,
        lighthouse_addr: Optional[str] = None,
        replica_id: Optional[str] = None,
        port: Optional[int] = None,
        hostname: str = socket.gethostname(),
        heartbeat_interval: timedelta = timedelta(milliseconds=100),
        checkpoint_transport: Optional[CheckpointTransport[Dict[str, T]]] = None,
    ) -> None:
        """
        Args:
            pg: reconfigurable process group spanning the replica groups
            load_state_dict / state_dict: user callbacks used for live recovery
            min_replica_size: fewer participants than this and no step commits
            use_async_quorum: run the quorum concurrently with the forward pass; a
                recovering replica then contributes zero gradients for its first step
            timeout: collectives, should_commit and checkpoint operations
            quorum_timeout: the quorum request (must exceed the time between two
                quorums, for example ``sync_every`` inner steps with LocalSGD)
            connect_timeout: establishing control-plane connections
            rank / world_size: local rank and size INSIDE the replica group
                (default: ``RANK`` / ``WORLD_SIZE``)
            store_addr / store_port: TCPStore of the replica group
                (default: ``MASTER_ADDR`` / ``MASTER_PORT``)
            lighthouse_addr: rank 0 only (default ``TORCHFT_LIGHTHOUSE``)
            replica_id: rank 0 only; a uuid is appended so a restarted group is new
            port: rank 0 only, manager server port (default ``TORCHFT_MANAGER_PORT`` or 0)
            hostname: rank 0 only, the name advertised to the lighthouse
            checkpoint_transport: how recovering replicas fetch state (default HTTP)
        """
        self._load_state_dict = load_state_dict
        self._user_state_dict = state_dict
        self._pending_state_dict: Optional[Dict[str, object]] = None
        self._use_async_quorum = use_async_quorum
        self._timeout = timeout
        self._quorum_timeout = quorum_timeout
        self._connect_timeout = connect_timeout
        self._world_size_mode = world_size_mode
        self._min_replica_size = min_replica_size

        store_addr = store_addr or os.environ["MASTER_ADDR"]
        store_port = store_port or int(os.environ["MASTER_PORT"])
        self._rank: int = rank if rank is not None else int(os.environ["RANK"])
        rank = self._rank
        world_size = world_size or int(os.environ["WORLD_SIZE"])

        if checkpoint_transport is None:
            checkpoint_transport = CheckpointServer[Dict[str, T]](timeout=timeout)
        self._checkpoint_transport: CheckpointTransport[Dict[str, T]] = checkpoint_transport

        self._executor = ThreadPoolExecutor(max_workers=1, thread_name_prefix="async_quorum")
        self._quorum_future: Optional[concurrent.futures.Future] = None

        self._store = TCPStore(host_name=store_addr, port=store_port, is_master=False, wait_for_workers=False)
        self._pg = pg
        self._manager: Optional[_ManagerServer] = None

        if rank == 0:
            if port is None:
                port = int(os.environ.get(MANAGER_PORT_ENV, 0))
            lighthouse_addr = lighthouse_addr or os.environ["TORCHFT_LIGHTHOUSE"]
            replica_id = (replica_id or "") + str(uuid.uuid4())
            self._manager = _ManagerServer(
                replica_id=replica_id,
                lighthouse_addr=lighthouse_addr,
                hostname=hostname,
                bind=f"[::]:{port}",
                store_addr=f"{store_addr}:{store_port}",
                world_size=world_size,
                heartbeat_interval=heartbeat_interval,
                connect_timeout=connect_timeout,
            )
            self._store.set(MANAGER_ADDR_KEY, self._manager.address())
            self._store.set(REPLICA_ID_KEY, replica_id)

        addr = self._store.get(MANAGER_ADDR_KEY).decode("utf-8")
        self._client = ManagerClient(addr, connect_timeout=connect_timeout)
        replica_id = self._store.get(REPLICA_ID_KEY).decode("utf-8")
        self._replica_id = replica_id
        self._logger = _ManagerLogger(manager=self, replica_id=replica_id or "", rank=rank)

        self._step = 0
        self._quorum_id = -1
        self._errored: Optional[Exception] = None
        self._healing = False
        self._pending_work: List[torch.futures.Future[object]] = []
        self._batches_committed = 0

        self._participating_rank: Optional[int] = None
        self._participating_world_size: int = 0
        self._replica_rank: int = 0
        self._replica_world_size: int = 0

        # Transports that can receive in place (NVLink) ask the manager for the live state.
        bind = getattr(self._checkpoint_transport, "bind_manager", None)
        if callable(bind):
            bind(self)

    # ------------------------------------------------------------------ state dict plumbing
    def set_state_dict_fns(self, load_state_dict: Callable[[T], None], state_dict: Callable[[], T]) -> None:
        self._load_state_dict = load_state_dict
        self._user_state_dict = state_dict

    def shutdown(self, wait: bool = True) -> None:
        """Stops the checkpoint transport, the manager server (rank 0) and the quorum thread."""
        self._checkpoint_transport.shutdown(wait=wait)
        if self._manager is not None:
            self._manager.shutdown()
        self._executor.shutdown(wait=wait)

    # ------------------------------------------------------------------ collectives
    def allreduce(self, tensor: torch.Tensor) -> "torch.futures.Future[torch.Tensor]":
        """Averages ``tensor`` in place over the participating replicas.

        Returns a future that completes with the tensor.  Errors are recorded, not
        raised: after the first one the remaining calls of this step return
        immediately and the tensor contents must be considered garbage until the next
        successful step.
        """
        if self.errored():
            return _completed(tensor)
        self.wait_quorum()
        # wait_quorum may surface a reconfiguration error
        if self.errored():
            return _completed(tensor)
        try:
            with trace_range("tft.allreduce"):
                n = self.num_participants()
                # A healing or spare replica is in the group but adds zeros.
                work = self._pg.allreduce_scaled(tensor, 1.0 / max(n, 1), contribute=self.is_participating())
                fut = work.get_future()

            def done(f: "torch.futures.Future[object]") -> torch.Tensor:
                f.value()
                return tensor

            return self.wrap_future(fut.then(done), tensor)
        except Exception as e:  # noqa: BLE001 - recorded, the step is discarded
            self._logger.exception(f"got exception in all reduce -- skipping remaining: {e}")
            self.report_error(e)
            return _completed(tensor)

    def run_collective(self, launch, result: T) -> "torch.futures.Future[T]":
        """Runs a fused collective with the bookkeeping of ``allreduce``.

        ``launch(pg, num_participants, contribute)`` starts the operation on the process group and
        returns its work object.  Waits for the quorum first, does nothing once the step has
        failed, and turns failures into ``report_error`` + ``result``.
        """
        if self.errored():
            return _completed(result)
        self.wait_quorum()
        if self.errored():
            return _completed(result)
        try:
            with trace_range("tft.collective"):
                work = launch(self._pg, max(self.num_participants(), 1), self.is_participating())
                fut = work.get_future()

            def done(f: "torch.futures.Future[object]") -> T:
                f.value()
                return result

            return self.wrap_future(fut.then(done), result)
        except Exception as e:  # noqa: BLE001 - recorded, the step is discarded
            self._logger.exception(f"got exception in collective -- skipping remaining: {e}")
            self.report_error(e)
            return _completed(result)

    def report_error(self, e: Exception) -> None:
        """Marks the current step as failed; it will not commit and the group reconfigures."""
        self._errored = e

    def errored(self) -> Optional[Exception]:
        return self._errored

    def wrap_future(
        self, fut: "torch.futures.Future[T]", default: T, timeout: Optional[timedelta] = None
    ) -> "torch.futures.Future[T]":
        """Adds a deadline to ``fut`` and converts failures into ``report_error`` + ``default``."""
        fut = future_timeout(fut, timeout or self._timeout)

        def callback(f: "torch.futures.Future[T]") -> T:
            try:
                return f.value()
            except Exception as e:  # noqa: BLE001 - recorded, the step is discarded
                self._logger.exception(f"got exception in future -- skipping remaining: {e}")
                self.report_error(e)
                return default

        fut = fut.then(callback)
        self._pending_work.append(cast("torch.futures.Future[object]", fut))
        return fut

    # ------------------------------------------------------------------ quorum
    def start_quorum(
        self, allow_heal: bool = True, shrink_only: bool = False, timeout: Optional[timedelta] = None
    ) -> None:
        """Begins a new step: computes the quorum (in the background in async mode).

        ``allow_heal`` must be the same on every replica.  In sync mode a recovering
        replica has its state loaded before this returns and takes part in the step;
        in async mode loading is deferred to ``should_commit`` on the calling thread.
        """
        if self._quorum_future is not None:
            self._quorum_future.result()
        # A failed step can leave the communicator out of step with its peers (one side gave up
        # on a collective the other side never started).  Ask for a fresh quorum id: every member
        # then reconfigures even though the membership is unchanged.
        force_reconfigure = self._errored is not None
        self._errored = None
        self._healing = False
        self._quorum_future = self._executor.submit(
            self._async_quorum,
            allow_heal=allow_heal,
            shrink_only=shrink_only,
            quorum_timeout=timeout or self._quorum_timeout,
            force_reconfigure=force_reconfigure,
        )
        if not self._use_async_quorum:
            self.wait_quorum()
            if self._healing:
                # The step can be joined right away because the state is loaded here.
                self._apply_pending_state_dict()
                self._healing = False

    def wait_quorum(self) -> None:
        """Blocks until the quorum, reconfiguration and checkpoint fetch of this step finished."""
        assert self._quorum_future is not None, "must call start_quorum before wait_quorum"
        self._quorum_future.result()

    def _async_quorum(
        self, allow_heal: bool, shrink_only: bool, quorum_timeout: timedelta, force_reconfigure: bool = False
    ) -> None:
        with trace_range("tft.quorum"):
            kwargs = {"force_reconfigure": True} if force_reconfigure else {}
            quorum = self._client.quorum(
                rank=self._rank,
                step=self._step,
                checkpoint_metadata=self._checkpoint_transport.metadata(),
                shrink_only=shrink_only,
                timeout=quorum_timeout,
                **kwargs,
            )
        max_step = quorum.max_step
        self._replica_rank = quorum.replica_rank
        self._replica_world_size = quorum.replica_world_size

        # Async quorum or no healing: only the replicas at max_step contribute.
        # Sync healing: everyone is up to date by the time gradients are exchanged.
        if self._use_async_quorum or not allow_heal:
            self._participating_rank, self._participating_world_size = quorum.max_rank, quorum.max_world_size
        else:
            self._participating_rank, self._participating_world_size = quorum.replica_rank, quorum.replica_world_size

        if self._world_size_mode == WorldSizeMode.FIXED_WITH_SPARES:
            self._participating_world_size = min(self._participating_world_size, self._min_replica_size)
            if self._participating_rank is not None and self._participating_rank >= self._min_replica_size:
                self._participating_rank = None

        if quorum.quorum_id != self._quorum_id:
            prefixed = f"{quorum.store_address}/torchft/{quorum.quorum_id}/{self._rank}"
            self._logger.info(f"reconfiguring for quorum_id={quorum.quorum_id} store_prefixed_addr={prefixed}")
            with trace_range("tft.configure"):
                # every member of the quorum is in the group, recovering ones included
                self._pg.configure(prefixed, quorum.replica_rank, quorum.replica_world_size)
            self._quorum_id = quorum.quorum_id

        if not allow_heal:
            return
        if quorum.recover_dst_ranks:
            self._logger.info(f"peers need recovery from us {quorum.recover_dst_ranks}")
            with trace_range("tft.heal_send"):
                self._checkpoint_transport.send_checkpoint(
                    dst_ranks=quorum.recover_dst_ranks,
                    step=max_step,
                    state_dict=self._manager_state_dict(),
                    timeout=self._timeout,
                )
        if quorum.heal:
            self._healing = True
            src_addr = quorum.recover_src_manager_address
            self._logger.info(f"healing required, fetching checkpoint metadata from {src_addr} max_step={max_step}")
            with trace_range("tft.heal_recv"):
                # The same local rank of the source group registered this metadata.
                source = ManagerClient(src_addr, connect_timeout=self._connect_timeout)
                metadata = source.checkpoint_metadata(self._rank, timeout=self._timeout)
                assert quorum.recover_src_rank is not None, "must have a recover rank when healing"
                self._logger.info(f"fetching checkpoint from rank {quorum.recover_src_rank} with metadata {metadata}")
                # User state is only staged here: this is not the training thread.
                self._pending_state_dict = cast(
                    Dict[str, object],
                    self._checkpoint_transport.recv_checkpoint(
                        src_rank=quorum.recover_src_rank, metadata=metadata, step=max_step, timeout=self._timeout
                    ),
                )
            self.load_state_dict(cast(Dict[str, int], self._pending_state_dict["torchft"]))
            self._step = max_step

    def _apply_pending_state_dict(self) -> None:
        assert self._healing, "must be in healing state"
        assert self._quorum_future is not None, "must call step before should_commit"
        self._quorum_future.result()
        self._logger.info("applying pending state dict")
        assert self._pending_state_dict is not None, "checkpoint was not staged"
        assert self._load_state_dict is not None, "user load_state_dict is not initialized."
        self._load_state_dict(cast(T, self._pending_state_dict["user"]))  # type: ignore[misc]
        self._pending_state_dict = None
        self._logger.info("Loaded state dict.")

    # ------------------------------------------------------------------ commit
    def should_commit(self, timeout: Optional[timedelta] = None) -> bool:
        """Group-wide vote on whether the optimizer may step.  Call once per step on every rank.

        Waits for the outstanding allreduces, applies a staged recovery checkpoint,
        then asks the manager server, which answers True only if every rank of the
        replica group voted True.  Different replica groups may decide differently.
        """
        for work in self._pending_work:
            if self._errored is not None:
                break  # the step is lost already
            work.wait()
        self._pending_work = []

        if self._healing:
            self._apply_pending_state_dict()

        enough_replicas = self.num_participants() >= self._min_replica_size
        local_should_commit = enough_replicas and self._errored is None
        should_commit = self._client.should_commit(
            self._rank, self._step, local_should_commit, timeout=timeout or self._timeout
        )
        self._logger.info(
            f"should_commit={should_commit} enough_replicas={enough_replicas}, errored={self._errored}"
        )
        # From here on the weights may change, so peers must not read them any more.
        self._checkpoint_transport.disallow_checkpoint()
        if should_commit:
            self._step += 1
            self._batches_committed += self.num_participants()
        return should_commit

    # ------------------------------------------------------------------ state
    def load_state_dict(self, state_dict: Dict[str, int]) -> None:
        self._step = state_dict["step"]
        self._batches_committed = state_dict["batches_committed"]

    def _manager_state_dict(self) -> Dict[str, object]:
        assert self._user_state_dict is not None, "user state_dict is not initialized."
        return {"user": self._user_state_dict(), "torchft": self.state_dict()}

    def state_dict(self) -> Dict[str, int]:
        """Must be saved with (and restored from) every durable checkpoint."""
        return {"step": self._step, "batches_committed": self._batches_committed}

    def current_step(self) -> int:
        """Number of committed steps (optimizer steps); also the live-recovery version."""
        return self._step

    def batches_committed(self) -> int:
        """Total batches committed over all replica groups and steps (sum of participants per step)."""
        return self._batches_committed

    def num_participants(self) -> int:
        """Replicas contributing to the current step (the averaging divisor)."""
        assert self._participating_world_size >= 0, "internal error"
        return self._participating_world_size

    def is_participating(self) -> bool:
        """False for spares and for a replica that is still healing in async mode."""
        if self._participating_rank is None:
            return False
        if self._healing:
            assert self._use_async_quorum
            return False
        return True

    def replica_rank(self) -> int:
        """Rank of this replica group within the current quorum (all members, recovering included)."""
        return self._replica_rank

    def replica_world_size(self) -> int:
        return self._replica_world_size

    def replica_id(self) -> str:
        return self._replica_id


def _completed(value: T) -> "torch.futures.Future[T]":
    fut: torch.futures.Future = torch.futures.Future()
    fut.set_result(value)
    return fut


class _ManagerLogger:
    """Prefixes log lines with ``[replica_id/rank - step N]``."""

    def __init__(self, manager: Manager, replica_id: str, rank: int) -> None:
        self._logger = logging.getLogger(__name__)
        self._replica_id = replica_id
        self._rank = rank
        self._manager = manager

    def prefix(self) -> str:
        return f"[{self._replica_id}/{self._rank} - step {self._manager.current_step()}]"

    def info(self, msg: str) -> None:
        self._logger.info(f"{self.prefix()} {msg}")

    def warn(self, msg: str) -> None:
        self._logger.warning(f"{self.prefix()} {msg}")

    def exception(self, msg: str) -> None:
        self._logger.exception(f"{self.prefix()} {msg}")
