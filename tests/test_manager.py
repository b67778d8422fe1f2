"""Manager state machine against a mocked manager client (no servers).

Scenarios follow the reference's manager_test.py: happy path, sync / async heal,
errors at queue and wait time, spares, allow_heal=False, wrap_future, numerics.
"""

from datetime import timedelta
from unittest.mock import MagicMock, patch

import pytest
import torch
from torch.distributed import TCPStore

from torchft_b200._control import QuorumResult
from torchft_b200.checkpointing import CheckpointServer
from torchft_b200.manager import MANAGER_ADDR_KEY, REPLICA_ID_KEY, Manager, WorldSizeMode
from torchft_b200.process_group import ProcessGroup, ProcessGroupDummy, _DummyWork


class RecordingPG(ProcessGroupDummy):
    """World-size-1 dummy that records configure calls and can be told to fail."""

    def __init__(self):
        super().__init__(0, 1)
        self.configured = []
        self.fail_allreduce = None
        self.fail_future = None

    def configure(self, store_addr, rank, world_size):
        super().configure(store_addr, rank, world_size)
        self.configured.append((store_addr, rank, world_size))

    def allreduce(self, tensors, opts):
        if self.fail_allreduce is not None:
            raise self.fail_allreduce
        if self.fail_future is not None:
            w = _DummyWork(tensors)
            w._done = torch.futures.Future()
            w._done.set_exception(self.fail_future)
            return w
        return super().allreduce(tensors, opts)


def quorum_result(**kw):
    q = QuorumResult()
    q.quorum_id = 123
    q.replica_rank = 1
    q.replica_world_size = 2
    q.recover_src_manager_address = "manager address"
    q.store_address = "store:1"
    q.max_step = 1
    q.max_rank = 1
    q.max_world_size = 2
    q.heal = False
    for k, v in kw.items():
        setattr(q, k, v)
    return q


@pytest.fixture
def env():
    created = []

    def make(use_async_quorum=True, min_replica_size=2, world_size_mode=WorldSizeMode.DYNAMIC, timeout=timedelta(seconds=10), transport=None):
        store = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
        # rank 1 of a 2-rank group: no manager server is started, only the client (mocked)
        store.set(MANAGER_ADDR_KEY, "dummy")
        store.set(REPLICA_ID_KEY, "dummy_id")
        pg = RecordingPG()
        load_sd = MagicMock()
        with patch("torchft_b200.manager.ManagerClient", autospec=True):
            manager = Manager(
                pg=pg,
                min_replica_size=min_replica_size,
                load_state_dict=load_sd,
                state_dict=lambda: {"user": "state"},
                use_async_quorum=use_async_quorum,
                world_size_mode=world_size_mode,
                timeout=timeout,
                store_addr="127.0.0.1",
                store_port=store.port,
                rank=1,
                world_size=2,
                checkpoint_transport=transport,
            )
        created.append((manager, store))
        return manager, pg, load_sd

    yield make
    for manager, _ in created:
        manager.shutdown(wait=False)


def test_state_dict_round_trip(env):
    manager, _, _ = env()
    assert manager.state_dict() == {"step": 0, "batches_committed": 0}
    manager.load_state_dict({"step": 1234, "batches_committed": 2345})
    assert manager.current_step() == 1234 and manager.batches_committed() == 2345


def test_user_state_dict_fns(env):
    manager, _, _ = env()
    assert manager._manager_state_dict() == {"user": {"user": "state"}, "torchft": {"step": 0, "batches_committed": 0}}
    manager.set_state_dict_fns(lambda sd: None, lambda: {"new": 1})
    assert manager._manager_state_dict()["user"] == {"new": 1}


def test_happy_path(env):
    manager, pg, load_sd = env()
    manager._client.quorum.return_value = quorum_result()
    manager._client.should_commit.return_value = True
    assert manager._quorum_id == -1 and manager.current_step() == 0

    manager.start_quorum()
    t = torch.tensor([2.0, 4.0])
    manager.allreduce(t).wait()
    assert torch.allclose(t, torch.tensor([1.0, 2.0]))  # divided by 2 participants
    assert manager.should_commit()
    assert manager._quorum_id == 123
    assert manager.current_step() == 1
    assert manager.batches_committed() == 2
    assert pg.configured == [("store:1/torchft/123/1", 1, 2)]
    assert manager.is_participating() and manager.num_participants() == 2
    assert load_sd.call_count == 0

    # same quorum id: no second configure
    manager.start_quorum()
    assert manager.should_commit()
    assert len(pg.configured) == 1
    assert manager.current_step() == 2 and manager.batches_committed() == 4


def _self_serving_transport(manager_holder):
    """A real HTTP transport that the healing manager fetches from (loop-back)."""
    return CheckpointServer(timeout=timedelta(seconds=10))


def test_heal_sync(env):
    transport = CheckpointServer(timeout=timedelta(seconds=10))
    manager, pg, load_sd = env(use_async_quorum=False, min_replica_size=2, transport=transport)
    manager._client.quorum.return_value = quorum_result(
        recover_src_rank=0, max_step=20, max_rank=None, max_world_size=2, heal=True
    )
    manager._client.should_commit.return_value = True
    # the "peer" is our own transport serving step 20
    transport.send_checkpoint([1], 20, {"user": {"w": 1}, "torchft": {"step": 20, "batches_committed": 40}}, timedelta(seconds=10))
    with patch("torchft_b200.manager.ManagerClient", autospec=True) as client_cls:
        client_cls.return_value.checkpoint_metadata.return_value = transport.metadata()
        manager.start_quorum()
    # sync mode: state applied inside start_quorum, replica takes part in the step
    assert not manager._healing
    assert manager.current_step() == 20
    load_sd.assert_called_once_with({"w": 1})
    assert manager.is_participating() and manager.num_participants() == 2
    t = torch.tensor([4.0])
    manager.allreduce(t).wait()
    assert torch.allclose(t, torch.tensor([2.0]))
    assert manager.should_commit()
    assert manager.current_step() == 21 and manager.batches_committed() == 42


def test_heal_async_zero_gradients(env):
    transport = CheckpointServer(timeout=timedelta(seconds=10))
    manager, pg, load_sd = env(use_async_quorum=True, min_replica_size=1, transport=transport)
    manager._client.quorum.return_value = quorum_result(
        recover_src_rank=0, max_step=20, max_rank=None, max_world_size=1, heal=True
    )
    manager._client.should_commit.return_value = True
    transport.send_checkpoint([1], 20, {"user": {"w": 2}, "torchft": {"step": 20, "batches_committed": 0}}, timedelta(seconds=10))
    with patch("torchft_b200.manager.ManagerClient", autospec=True) as client_cls:
        client_cls.return_value.checkpoint_metadata.return_value = transport.metadata()
        manager.start_quorum()
        manager.wait_quorum()
    assert manager._healing and not manager.is_participating()
    assert manager.num_participants() == 1
    assert load_sd.call_count == 0  # deferred to the training thread
    t = torch.tensor([5.0])
    manager.allreduce(t).wait()
    assert torch.equal(t, torch.tensor([0.0]))  # contributes zeros
    assert manager.should_commit()
    load_sd.assert_called_once_with({"w": 2})
    assert manager.current_step() == 21


def test_heal_async_not_enough_participants(env):
    transport = CheckpointServer(timeout=timedelta(seconds=10))
    manager, pg, load_sd = env(use_async_quorum=True, min_replica_size=2, transport=transport)
    manager._client.quorum.return_value = quorum_result(
        recover_src_rank=0, max_step=20, max_rank=None, max_world_size=1, heal=True
    )
    manager._client.should_commit.return_value = False
    transport.send_checkpoint([1], 20, {"user": {}, "torchft": {"step": 20, "batches_committed": 0}}, timedelta(seconds=10))
    with patch("torchft_b200.manager.ManagerClient", autospec=True) as client_cls:
        client_cls.return_value.checkpoint_metadata.return_value = transport.metadata()
        manager.start_quorum()
        manager.wait_quorum()
    assert not manager.should_commit()
    # local vote was False: 1 participant < min_replica_size 2
    args = manager._client.should_commit.call_args
    assert args[0][2] is False
    assert manager.current_step() == 20  # healed but not advanced


def test_allreduce_error_at_queue_time_then_recovery(env):
    manager, pg, _ = env()
    manager._client.quorum.return_value = quorum_result(max_step=1)
    manager._client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    manager.start_quorum()
    manager.allreduce(torch.tensor([1.0])).wait()
    assert manager.should_commit()

    pg.fail_allreduce = RuntimeError("injected failure")
    manager.start_quorum()
    manager.allreduce(torch.tensor([1.0])).wait()
    assert isinstance(manager.errored(), RuntimeError)
    # later allreduces of the step are skipped outright
    manager.allreduce(torch.tensor([1.0])).wait()
    assert not manager.should_commit()
    assert manager.current_step() == 1

    pg.fail_allreduce = None
    manager._client.quorum.return_value = quorum_result(quorum_id=124, max_step=1)
    manager.start_quorum()  # clears the error, new quorum id reconfigures
    assert manager.errored() is None
    manager.allreduce(torch.tensor([1.0])).wait()
    assert manager.should_commit()
    assert len(pg.configured) == 2 and manager.current_step() == 2


def test_allreduce_error_at_wait_time(env):
    manager, pg, _ = env()
    manager._client.quorum.return_value = quorum_result()
    manager._client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    pg.fail_future = RuntimeError("async failure")
    manager.start_quorum()
    t = torch.tensor([3.0])
    out = manager.allreduce(t).wait()  # does not raise
    assert out is t
    assert "async failure" in str(manager.errored())
    assert not manager.should_commit()


def test_fixed_with_spares(env):
    manager, pg, _ = env(min_replica_size=2, world_size_mode=WorldSizeMode.FIXED_WITH_SPARES)
    manager._client.quorum.return_value = quorum_result(replica_rank=2, replica_world_size=3, max_rank=2, max_world_size=3)
    manager._client.should_commit.return_value = True
    manager.start_quorum()
    manager.wait_quorum()
    assert manager.num_participants() == 2
    assert not manager.is_participating()  # third replica is a spare
    t = torch.tensor([7.0])
    manager.allreduce(t).wait()
    assert torch.equal(t, torch.tensor([0.0]))
    assert manager.should_commit()
    assert manager.batches_committed() == 2
    assert pg.configured == [("store:1/torchft/123/1", 2, 3)]


def test_allow_heal_false(env):
    manager, pg, load_sd = env(use_async_quorum=False)
    manager._client.quorum.return_value = quorum_result(
        replica_rank=0, recover_src_rank=1, recover_dst_ranks=[], max_step=20, max_rank=None, max_world_size=1, heal=True
    )
    manager._client.should_commit.return_value = True
    manager.start_quorum(allow_heal=False)
    assert not manager._healing
    assert not manager.is_participating()  # behind and not healed: contributes zeros
    assert manager.num_participants() == 1
    assert manager.current_step() == 0 and load_sd.call_count == 0


def test_wrap_future_error_and_timeout(env):
    manager, _, _ = env(timeout=timedelta(seconds=0.05))
    manager._client.quorum.return_value = quorum_result()
    fut = torch.futures.Future()
    wrapped = manager.wrap_future(fut, 2)
    fut.set_exception(RuntimeError("injected failure"))
    assert wrapped.value() == 2
    assert "injected failure" in str(manager.errored())
    assert len(manager._pending_work) == 1

    manager._errored = None
    never = torch.futures.Future()
    wrapped = manager.wrap_future(never, "default")
    assert wrapped.wait() == "default"
    assert isinstance(manager.errored(), TimeoutError)


def test_timeouts_are_plumbed(env):
    manager, _, _ = env(timeout=timedelta(seconds=13))
    manager._quorum_timeout = timedelta(seconds=12)
    manager._client.quorum.return_value = quorum_result()
    manager._client.should_commit.return_value = True
    manager.start_quorum()
    manager.wait_quorum()
    assert manager._client.quorum.call_args.kwargs["timeout"] == timedelta(seconds=12)
    manager.start_quorum(timeout=timedelta(seconds=2))
    manager.wait_quorum()
    assert manager._client.quorum.call_args.kwargs["timeout"] == timedelta(seconds=2)
    manager.should_commit()
    assert manager._client.should_commit.call_args.kwargs["timeout"] == timedelta(seconds=13)
    manager.should_commit(timeout=timedelta(seconds=3))
    assert manager._client.should_commit.call_args.kwargs["timeout"] == timedelta(seconds=3)


def test_send_checkpoint_to_recovering_peers(env):
    transport = MagicMock()
    transport.metadata.return_value = "meta"
    manager, _, _ = env(transport=transport)
    manager._client.quorum.return_value = quorum_result(recover_dst_ranks=[0], max_step=5)
    manager._client.should_commit.return_value = True
    manager.start_quorum()
    manager.wait_quorum()
    kwargs = transport.send_checkpoint.call_args.kwargs
    assert kwargs["dst_ranks"] == [0] and kwargs["step"] == 5
    assert kwargs["state_dict"]["user"] == {"user": "state"}
    manager.should_commit()
    assert transport.disallow_checkpoint.call_count == 1


def test_run_collective_bookkeeping(env):
    """A fused collective gets the allreduce treatment: quorum first, participants passed, errors recorded."""
    manager, pg, _ = env()
    manager._client.quorum.return_value = quorum_result()
    manager._client.should_commit.return_value = True
    manager.start_quorum()
    seen = {}

    def launch(group, n, contribute):
        seen.update(pg=group, n=n, contribute=contribute)
        return _DummyWork([torch.zeros(1)])

    assert manager.run_collective(launch, "result").wait() == "result"
    assert seen == {"pg": pg, "n": 2, "contribute": True}
    assert manager.errored() is None and manager.should_commit()

    # a launch that raises: recorded, the default comes back, the step does not commit
    manager.start_quorum()

    def broken(group, n, contribute):
        raise RuntimeError("launch failed")

    assert manager.run_collective(broken, "fallback").wait() == "fallback"
    assert isinstance(manager.errored(), RuntimeError)
    # once the step has failed further collectives are skipped
    seen.clear()
    manager.run_collective(launch, None).wait()
    assert seen == {}
    manager._client.should_commit.return_value = False
    assert not manager.should_commit()


def test_step_accounting_over_random_histories(env):
    """Whatever mix of failed collectives, refused commits and changing quorum sizes: the step counts
    committed steps only, batches_committed adds the participants of committed steps, and an error
    never leaks into the next step."""
    import random

    manager, pg, _ = env(min_replica_size=1)
    rng = random.Random(11)
    step, batches, quorum_id = 0, 0, 100
    for _ in range(60):
        if rng.random() < 0.3:
            quorum_id += 1  # membership changed
        world = rng.randint(1, 4)
        manager._client.quorum.return_value = quorum_result(
            quorum_id=quorum_id, replica_rank=0, replica_world_size=world, max_rank=0, max_world_size=world, max_step=step)
        fail = rng.random() < 0.25
        vote = rng.random() < 0.8
        pg.fail_future = RuntimeError("injected") if fail else None
        manager._client.should_commit.return_value = vote and not fail
        manager.start_quorum()
        assert manager.errored() is None
        t = torch.ones(3)
        manager.allreduce(t).wait()
        committed = manager.should_commit()
        # the manager votes False after an error whatever the group would answer
        sent_vote = manager._client.should_commit.call_args.kwargs.get("should_commit", None)
        if sent_vote is None:
            sent_vote = manager._client.should_commit.call_args.args[2]
        assert sent_vote == (not fail)
        assert committed == (vote and not fail)
        if committed:
            step += 1
            batches += world
        assert manager.current_step() == step and manager.batches_committed() == batches
    pg.fail_future = None
