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

Internally the class is cut into four pieces: the *view* of the current quorum (who takes
part, at which rank), the *ledger* of committed steps, one *round* of quorum work that runs on
a worker thread (request, reconfiguration, serving and fetching recovery state), and the
*vote* at the end of the step.
"""

from __future__ import annotations

import logging
import os
import socket
import uuid
from concurrent.futures import Future as _ThreadFuture, ThreadPoolExecutor
from dataclasses import dataclass
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

# keys of the replica group's store through which rank 0 publishes its manager server
MANAGER_ADDR_KEY: str = "manager_addr"
REPLICA_ID_KEY: str = "replica_id"
# environment variable with the port of the manager server (rank 0; default: any free port)
MANAGER_PORT_ENV: str = "TORCHFT_MANAGER_PORT"

T = TypeVar("T")


class WorldSizeMode(Enum):
    """How the number of participating replicas is chosen.

    DYNAMIC: every replica of the quorum participates; gradients are divided by that count.
    FIXED_WITH_SPARES: at most ``min_replica_size`` replicas participate; the others are
    hot spares that contribute zeros but receive the averaged result.
    """

    DYNAMIC = 0
    FIXED_WITH_SPARES = 1


@dataclass
class _QuorumView:
    """What the last quorum means for this replica."""

    replica_rank: int = 0             # position among ALL members (recovering ones included)
    replica_world: int = 0
    active_rank: Optional[int] = None  # position among the members whose data counts; None = spare / behind
    active_world: int = 0


@dataclass
class _Ledger:
    step: int = 0     # committed steps = version of the weights
    batches: int = 0  # sum over committed steps of the replicas that took part

    def commit(self, participants: int) -> None:
        self.step += 1
        self.batches += participants

    def as_dict(self) -> Dict[str, int]:
        return {"step": self.step, "batches_committed": self.batches}


def _from_env(value, name: str, convert=str, zero_is_value: bool = False):
    """``value`` if given, else the environment variable ``name`` (KeyError when missing).
    Empty strings and, unless ``zero_is_value``, zeros count as "not given"."""
    given = value is not None and (zero_is_value or bool(value))
    return value if given else convert(os.environ[name])


def _done(value: T) -> "torch.futures.Future[T]":
    fut: torch.futures.Future = torch.futures.Future()
    fut.set_result(value)
    return fut


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
        # ---- configuration
        self._pg = pg
        self._use_async_quorum = use_async_quorum
        self._timeout, self._quorum_timeout, self._connect_timeout = timeout, quorum_timeout, connect_timeout
        self._min_replica_size = min_replica_size
        self._world_size_mode = world_size_mode
        self._load_state_dict, self._user_state_dict = load_state_dict, state_dict
        self._checkpoint_transport: CheckpointTransport[Dict[str, T]] = (
            checkpoint_transport if checkpoint_transport is not None else CheckpointServer[Dict[str, T]](timeout=timeout)
        )

        # ---- place in the replica group and its store
        self._rank: int = int(_from_env(rank, "RANK", int, zero_is_value=True))
        group_size = int(_from_env(world_size, "WORLD_SIZE", int))
        host = _from_env(store_addr, "MASTER_ADDR")
        store_port = int(_from_env(store_port, "MASTER_PORT", int))
        self._store = TCPStore(host_name=host, port=store_port, is_master=False, wait_for_workers=False)

        # ---- control plane: rank 0 hosts the group's manager server, every rank is its client
        self._manager: Optional[_ManagerServer] = None
        if self._rank == 0:
            self._manager = self._host_group_server(
                replica_id, lighthouse_addr, hostname, port, f"{host}:{store_port}", group_size, heartbeat_interval
            )
        self._client = ManagerClient(self._store.get(MANAGER_ADDR_KEY).decode("utf-8"), connect_timeout=connect_timeout)
        self._replica_id = self._store.get(REPLICA_ID_KEY).decode("utf-8")
        self._logger = _StepLogger(self)

        # ---- per-step state
        self._view = _QuorumView()
        self._ledger = _Ledger()
        self._quorum_id = -1
        self._errored: Optional[Exception] = None
        self._healing = False
        self._pending_state_dict: Optional[Dict[str, object]] = None
        self._pending_work: List[torch.futures.Future[object]] = []
        self._executor = ThreadPoolExecutor(max_workers=1, thread_name_prefix="async_quorum")
        self._quorum_future: Optional[_ThreadFuture] = None

        # Transports that can receive in place (NVLink) ask the manager for the live state.
        bind = getattr(self._checkpoint_transport, "bind_manager", None)
        if callable(bind):
            bind(self)

    def _host_group_server(self, replica_id, lighthouse_addr, hostname, port, store, group_size, heartbeat_interval):
        """Rank 0: starts the manager server of the replica group and publishes it in the group's store."""
        unique_id = (replica_id or "") + str(uuid.uuid4())  # a restarted group is a new member for the lighthouse
        listen_port = port if port is not None else int(os.environ.get(MANAGER_PORT_ENV, 0))
        server = _ManagerServer(
            replica_id=unique_id,
            lighthouse_addr=_from_env(lighthouse_addr, "TORCHFT_LIGHTHOUSE"),
            hostname=hostname,
            bind=f"[::]:{listen_port}",
            store_addr=store,
            world_size=group_size,
            heartbeat_interval=heartbeat_interval,
            connect_timeout=self._connect_timeout,
        )
        self._store.set(MANAGER_ADDR_KEY, server.address())
        self._store.set(REPLICA_ID_KEY, unique_id)
        return server

    # ------------------------------------------------------------------ lifecycle
    def set_state_dict_fns(self, load_state_dict: Callable[[T], None], state_dict: Callable[[], T]) -> None:
        self._load_state_dict, self._user_state_dict = load_state_dict, state_dict

    def shutdown(self, wait: bool = True) -> None:
        """Stops the checkpoint transport, the manager server (rank 0) and the quorum thread."""
        self._checkpoint_transport.shutdown(wait=wait)
        if self._manager is not None:
            self._manager.shutdown()
        self._executor.shutdown(wait=wait)

    # ------------------------------------------------------------------ collectives
    def _collective(self, launch, result: T, what: str) -> "torch.futures.Future[T]":
        """Common path of every cross-replica operation: wait for the quorum, skip once the step has
        failed, start the operation, and turn any failure into ``report_error`` + ``result``."""
        if self._errored is not None:
            return _done(result)
        self.wait_quorum()  # may itself surface a reconfiguration error
        if self._errored is not None:
            return _done(result)
        try:
            with trace_range(f"tft.{what}"):
                participants = max(self.num_participants(), 1)
                # a healing or spare replica is in the group but its data does not count
                work = launch(self._pg, participants, self.is_participating())
                finished = work.get_future()

            def hand_back(f: "torch.futures.Future[object]") -> T:
                f.value()
                return result

            return self.wrap_future(finished.then(hand_back), result)
        except Exception as e:  # noqa: BLE001 - recorded, the step is discarded
            self._logger.exception(f"got exception in {what} -- skipping remaining: {e}")
            self.report_error(e)
            return _done(result)

    def allreduce(self, tensor: torch.Tensor) -> "torch.futures.Future[torch.Tensor]":
        """Averages ``tensor`` in place over the participating replicas.

        Returns a future that completes with the tensor.  Errors are recorded, not
        raised: after the first one the remaining calls of this step return
        immediately and the tensor contents must be considered garbage until the next
        successful step.
        """
        return self._collective(
            lambda pg, n, contribute: pg.allreduce_scaled(tensor, 1.0 / n, contribute=contribute), tensor, "allreduce"
        )

    def run_collective(self, launch, result: T) -> "torch.futures.Future[T]":
        """Runs a fused collective with the bookkeeping of ``allreduce``.

        ``launch(pg, num_participants, contribute)`` starts the operation on the process group and
        returns its work object.  Waits for the quorum first, does nothing once the step has
        failed, and turns failures into ``report_error`` + ``result``.
        """
        return self._collective(launch, result, "collective")

    def report_error(self, e: Exception) -> None:
        """Marks the current step as failed; it will not commit and the group reconfigures."""
        self._errored = e

    def _abort_process_group(self) -> None:
        """Ends what the process group still has in flight, where the group can do that.

        Called once the host has given up on a collective (its future failed or ran into the
        manager's timeout): a kernel of the NVLink group that still waits for a peer returns within
        milliseconds instead of sitting out its own, longer, device-side budget, and an NCCL
        communicator is torn down as the reference does on reconfiguration
        (torchft/process_group.py:265-268).  The step is lost either way and the next quorum asks
        for a reconfiguration, which re-arms the group.
        """
        abort = getattr(self._pg, "abort", None)
        if callable(abort):
            try:
                abort()
            except Exception as e:  # noqa: BLE001 - best effort; the step is discarded anyway
                self._logger.warn(f"abort of the process group failed: {e}")

    def errored(self) -> Optional[Exception]:
        return self._errored

    def wrap_future(
        self, fut: "torch.futures.Future[T]", default: T, timeout: Optional[timedelta] = None
    ) -> "torch.futures.Future[T]":
        """Adds a deadline to ``fut`` and converts failures into ``report_error`` + ``default``."""

        def absorb(f: "torch.futures.Future[T]") -> T:
            try:
                return f.value()
            except Exception as e:  # noqa: BLE001 - recorded, the step is discarded
                self._logger.exception(f"got exception in future -- skipping remaining: {e}")
                self.report_error(e)
                self._abort_process_group()
                return default

        guarded = future_timeout(fut, timeout if timeout is not None else self._timeout).then(absorb)
        self._pending_work.append(cast("torch.futures.Future[object]", guarded))
        return guarded

    # ------------------------------------------------------------------ quorum round
    def start_quorum(
        self, allow_heal: bool = True, shrink_only: bool = False, timeout: Optional[timedelta] = None
    ) -> None:
        """Begins a new step: computes the quorum (in the background in async mode).

        ``allow_heal`` must be the same on every replica.  In sync mode a recovering
        replica has its state loaded before this returns and takes part in the step;
        in async mode loading is deferred to ``should_commit`` on the calling thread.
        """
        if self._quorum_future is not None:
            self._quorum_future.result()  # the previous round must be over
        # A failed step can leave the communicator out of step with its peers (one side gave up
        # on a collective the other side never started).  Ask for a fresh quorum id: every member
        # then reconfigures even though the membership is unchanged.
        previous_step_failed = self._errored is not None
        self._errored, self._healing = None, False
        self._quorum_future = self._executor.submit(
            self._async_quorum,
            allow_heal=allow_heal,
            shrink_only=shrink_only,
            quorum_timeout=timeout if timeout is not None else self._quorum_timeout,
            force_reconfigure=previous_step_failed,
        )
        if self._use_async_quorum:
            return
        self.wait_quorum()
        if self._healing:
            # sync mode: the state is loaded here, on the caller's thread, so the step can be joined right away
            self._apply_pending_state_dict()
            self._healing = False

    def wait_quorum(self) -> None:
        """Blocks until the quorum, reconfiguration and checkpoint fetch of this step finished."""
        assert self._quorum_future is not None, "must call start_quorum before wait_quorum"
        self._quorum_future.result()

    def _async_quorum(
        self, allow_heal: bool, shrink_only: bool, quorum_timeout: timedelta, force_reconfigure: bool = False
    ) -> None:
        """One round on the worker thread: request, view, reconfiguration, recovery traffic."""
        extra = {"force_reconfigure": True} if force_reconfigure else {}
        with trace_range("tft.quorum"):
            quorum = self._client.quorum(
                rank=self._rank, step=self._ledger.step, checkpoint_metadata=self._checkpoint_transport.metadata(),
                shrink_only=shrink_only, timeout=quorum_timeout, **extra,
            )
        self._view = self._interpret(quorum, count_everyone=allow_heal and not self._use_async_quorum)
        if quorum.quorum_id != self._quorum_id:
            self._join_group(quorum)
        if not allow_heal:
            return
        if quorum.recover_dst_ranks:
            self._offer_state(quorum)
        if quorum.heal:
            self._fetch_state(quorum)

    def _interpret(self, quorum, count_everyone: bool) -> _QuorumView:
        """Who contributes this step.  With synchronous healing every member is up to date by the time
        data is exchanged, so all of them count; otherwise only the members at the newest step do."""
        view = _QuorumView(replica_rank=quorum.replica_rank, replica_world=quorum.replica_world_size)
        if count_everyone:
            view.active_rank, view.active_world = quorum.replica_rank, quorum.replica_world_size
        else:
            view.active_rank, view.active_world = quorum.max_rank, quorum.max_world_size
        if self._world_size_mode == WorldSizeMode.FIXED_WITH_SPARES:
            cap = self._min_replica_size
            view.active_world = min(view.active_world, cap)
            if view.active_rank is not None and view.active_rank >= cap:
                view.active_rank = None  # a hot spare: receives the result, contributes nothing
        return view

    def _join_group(self, quorum) -> None:
        """Membership changed: point the process group at the new peers (recovering ones included)."""
        rendezvous = f"{quorum.store_address}/torchft/{quorum.quorum_id}/{self._rank}"
        self._logger.info(f"reconfiguring for quorum_id={quorum.quorum_id} store_prefixed_addr={rendezvous}")
        with trace_range("tft.configure"):
            self._pg.configure(rendezvous, quorum.replica_rank, quorum.replica_world_size)
        self._quorum_id = quorum.quorum_id

    def _offer_state(self, quorum) -> None:
        """Peers that are behind were assigned to this replica: let them read the live state."""
        self._logger.info(f"peers need recovery from us {quorum.recover_dst_ranks}")
        with trace_range("tft.heal_send"):
            self._checkpoint_transport.send_checkpoint(
                dst_ranks=quorum.recover_dst_ranks, step=quorum.max_step, state_dict=self._manager_state_dict(),
                timeout=self._timeout,
            )

    def _fetch_state(self, quorum) -> None:
        """This replica is behind: fetch the state of its assigned source and stage it."""
        self._healing = True
        source_addr, source_rank, version = quorum.recover_src_manager_address, quorum.recover_src_rank, quorum.max_step
        self._logger.info(f"healing required, fetching checkpoint metadata from {source_addr} max_step={version}")
        assert source_rank is not None, "must have a recover rank when healing"
        with trace_range("tft.heal_recv"):
            # the same local rank of the source group registered the metadata we need
            peer = ManagerClient(source_addr, connect_timeout=self._connect_timeout)
            where = peer.checkpoint_metadata(self._rank, timeout=self._timeout)
            self._logger.info(f"fetching checkpoint from rank {source_rank} with metadata {where}")
            staged = self._checkpoint_transport.recv_checkpoint(
                src_rank=source_rank, metadata=where, step=version, timeout=self._timeout
            )
        # User state is only staged: this is not the training thread.  The counters can move now.
        self._pending_state_dict = cast(Dict[str, object], staged)
        self.load_state_dict(cast(Dict[str, int], self._pending_state_dict["torchft"]))
        self._ledger.step = version

    def _apply_pending_state_dict(self) -> None:
        assert self._healing, "must be in healing state"
        assert self._quorum_future is not None, "must call step before should_commit"
        self._quorum_future.result()
        staged, self._pending_state_dict = self._pending_state_dict, None
        assert staged is not None, "checkpoint was not staged"
        assert self._load_state_dict is not None, "user load_state_dict is not initialized."
        self._logger.info("applying pending state dict")
        self._load_state_dict(cast(T, staged["user"]))  # type: ignore[misc]
        self._logger.info("Loaded state dict.")

    # ------------------------------------------------------------------ vote
    def should_commit(self, timeout: Optional[timedelta] = None) -> bool:
        """Group-wide vote on whether the optimizer may step.  Call once per step on every rank.

        Waits for the outstanding allreduces, applies a staged recovery checkpoint,
        then asks the manager server, which answers True only if every rank of the
        replica group voted True.  Different replica groups may decide differently.
        """
        outstanding, self._pending_work = self._pending_work, []
        for work in outstanding:
            if self._errored is not None:
                break  # the step is lost already
            work.wait()
        if self._healing:
            self._apply_pending_state_dict()

        participants = self.num_participants()
        quorate = participants >= self._min_replica_size
        my_vote = quorate and self._errored is None
        decision = self._client.should_commit(
            self._rank, self._ledger.step, my_vote, timeout=timeout if timeout is not None else self._timeout
        )
        self._logger.info(f"should_commit={decision} enough_replicas={quorate}, errored={self._errored}")
        # From here on the weights may change, so peers must not read them any more.
        self._checkpoint_transport.disallow_checkpoint()
        if decision:
            self._ledger.commit(participants)
        return decision

    # ------------------------------------------------------------------ state and accessors
    def load_state_dict(self, state_dict: Dict[str, int]) -> None:
        self._ledger = _Ledger(step=state_dict["step"], batches=state_dict["batches_committed"])

    def state_dict(self) -> Dict[str, int]:
        """Must be saved with (and restored from) every durable checkpoint."""
        return self._ledger.as_dict()

    def _manager_state_dict(self) -> Dict[str, object]:
        """What a recovering peer receives: the user's state plus the counters above."""
        assert self._user_state_dict is not None, "user state_dict is not initialized."
        return {"user": self._user_state_dict(), "torchft": self.state_dict()}

    def current_step(self) -> int:
        """Number of committed steps (optimizer steps); also the live-recovery version."""
        return self._ledger.step

    def batches_committed(self) -> int:
        """Total batches committed over all replica groups and steps (sum of participants per step)."""
        return self._ledger.batches

    def num_participants(self) -> int:
        """Replicas contributing to the current step (the averaging divisor)."""
        assert self._view.active_world >= 0, "internal error"
        return self._view.active_world

    def is_participating(self) -> bool:
        """False for spares and for a replica that is still healing in async mode."""
        if self._view.active_rank is None:
            return False
        if self._healing:
            assert self._use_async_quorum
            return False
        return True

    def replica_rank(self) -> int:
        """Rank of this replica group within the current quorum (all members, recovering included)."""
        return self._view.replica_rank

    def replica_world_size(self) -> int:
        return self._view.replica_world

    def replica_id(self) -> str:
        return self._replica_id


class _StepLogger:
    """Log lines of a manager carry ``[replica_id/rank - step N]`` in front."""

    def __init__(self, manager: Manager) -> None:
        self._log = logging.getLogger(__name__)
        self._owner = manager

    def _line(self, msg: str) -> str:
        m = self._owner
        return f"[{m._replica_id}/{m._rank} - step {m.current_step()}] {msg}"

    def info(self, msg: str) -> None:
        self._log.info(self._line(msg))

    def warn(self, msg: str) -> None:
        self._log.warning(self._line(msg))

    def exception(self, msg: str) -> None:
        self._log.exception(self._line(msg))
