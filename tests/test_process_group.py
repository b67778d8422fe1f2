"""Process-group conformance tests on CPU (gloo) -- the generic helper runs every
collective of the torchft contract against each backend, as the reference's
process_group_test.py does."""

import gc
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta
from unittest.mock import MagicMock, create_autospec

import pytest
import torch
import torch.distributed as dist
from torch.distributed import ReduceOp, TCPStore
from torch.distributed.distributed_c10d import AllgatherOptions, AllreduceOptions, BroadcastOptions

from torchft_b200.manager import Manager
from torchft_b200.process_group import (
    ErrorSwallowingProcessGroupWrapper,
    ManagedProcessGroup,
    ProcessGroup,
    ProcessGroupBabyGloo,
    ProcessGroupDummy,
    ProcessGroupGloo,
    ProcessGroupWrapper,
    _DummyWork,
    _ErrorSwallowingWork,
    _ManagedWork,
)


def make_store():
    return TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)


def check_collectives(pg: ProcessGroup, example: torch.Tensor) -> None:
    """Runs allreduce / allgather / broadcast (+wait and future) on a world-size-1 group."""
    shape, dtype = example.shape, example.dtype

    def check(t):
        assert t.shape == shape and t.dtype == dtype

    at = example.clone()
    opts = AllreduceOptions()
    opts.reduceOp = ReduceOp.SUM
    work = pg.allreduce([at], opts)
    work.wait()
    fut = work.get_future()
    fut.wait()
    check(at)
    work = pg.allreduce([at], ReduceOp.SUM)
    work.wait()
    work.get_future().wait()

    out = [[torch.empty_like(example)]]
    work = pg.allgather(out, [example.clone()], AllgatherOptions())
    work.wait()
    work.get_future().wait()
    check(out[0][0])
    assert torch.equal(out[0][0], example)

    bt = example.clone()
    bopts = BroadcastOptions()
    bopts.rootRank = 0
    work = pg.broadcast([bt], bopts)
    work.wait()
    work.get_future().wait()
    work = pg.broadcast_one(bt, 0)
    work.wait()
    check(bt)


def test_gloo_conformance_and_reconfigure():
    store = make_store()
    pg = ProcessGroupGloo()
    pg.configure(f"127.0.0.1:{store.port}/prefix", 0, 1)
    assert pg.size() == 1
    check_collectives(pg, torch.randn((2, 3)))
    # reconfigure onto a fresh prefix
    pg.configure(f"127.0.0.1:{store.port}/prefix2", 0, 1)
    check_collectives(pg, torch.randn((4,)))
    assert pg.getBackendName() == "torchft-gloo"


def test_gloo_configure_timeout():
    store = make_store()
    pg = ProcessGroupGloo(timeout=timedelta(seconds=0.05))
    with pytest.raises(RuntimeError, match="(timeout after 50ms|Socket Timeout|timed out|Timed out)"):
        pg.configure(f"127.0.0.1:{store.port}/prefix", 0, 2)


def test_use_before_configure():
    pg = ProcessGroupGloo()
    with pytest.raises(RuntimeError, match="before configure"):
        pg.allreduce([torch.ones(1)], ReduceOp.SUM)


def test_dummy():
    pg = ProcessGroupDummy(0, 1)
    pg.configure("x", 0, 1)
    assert pg.configure_count == 1
    check_collectives(pg, torch.randn(3))
    assert pg.getBackendName() == "torchft-dummy"
    m = torch.nn.parallel.DistributedDataParallel(torch.nn.Linear(3, 4), process_group=pg)
    m(torch.rand(2, 3)).sum().backward()


def test_allreduce_scaled_generic_path():
    store = make_store()
    pg = ProcessGroupGloo()
    pg.configure(f"127.0.0.1:{store.port}/s", 0, 1)
    t = torch.full((8,), 6.0)
    w = pg.allreduce_scaled(t, 0.5)
    w.wait()
    assert torch.allclose(t, torch.full((8,), 3.0))
    w.wait()  # scaling is applied once
    assert torch.allclose(t, torch.full((8,), 3.0))
    t = torch.full((8,), 6.0)
    pg.allreduce_scaled(t, 0.5).get_future().wait()
    assert torch.allclose(t, torch.full((8,), 3.0))
    t = torch.full((8,), 6.0)
    pg.allreduce_scaled(t, 0.5, contribute=False).wait()
    assert torch.equal(t, torch.zeros(8))


def test_gloo_two_ranks_threads():
    store = make_store()
    addr = f"127.0.0.1:{store.port}/two"

    def run(rank):
        pg = ProcessGroupGloo()
        pg.configure(addr, rank, 2)
        t = torch.full((4,), float(rank + 1))
        pg.allreduce_scaled(t, 0.5, contribute=(rank == 0)).wait()
        return t

    with ThreadPoolExecutor(2) as ex:
        a, b = list(ex.map(run, range(2)))
    # only rank 0 contributes: (1 + 0) * 0.5
    assert torch.allclose(a, torch.full((4,), 0.5)) and torch.allclose(b, a)


def test_baby_gloo_conformance_and_reconfigure():
    store = make_store()
    pg = ProcessGroupBabyGloo(timeout=timedelta(seconds=20))
    try:
        pg.configure(f"127.0.0.1:{store.port}/baby", 0, 1)
        assert pg.size() == 1
        check_collectives(pg, torch.randn((2, 3)))
        gc.collect()
        assert pg.num_active_work() == 0  # no leaked work handles in the child
        first = pg._p
        pg.configure(f"127.0.0.1:{store.port}/baby2", 0, 1)
        assert not first.is_alive()  # old child was killed
        check_collectives(pg, torch.randn((3,)))
        assert pg.getBackendName() == "torchft-baby-gloo"
    finally:
        pg.shutdown()


def test_baby_gloo_start_timeout():
    store = make_store()
    pg = ProcessGroupBabyGloo(timeout=timedelta(seconds=0.5))
    try:
        with pytest.raises((TimeoutError, RuntimeError)):
            pg.configure(f"127.0.0.1:{store.port}/never", 0, 2)  # second rank never joins
    finally:
        pg.shutdown()


def test_baby_gloo_two_ranks():
    store = make_store()
    addr = f"127.0.0.1:{store.port}/baby_two"

    def run(rank):
        pg = ProcessGroupBabyGloo(timeout=timedelta(seconds=30))
        try:
            pg.configure(addr, rank, 2)
            t = torch.full((3,), float(rank + 1))
            pg.allreduce([t], ReduceOp.SUM).wait()
            return t.clone()
        finally:
            pg.shutdown()

    with ThreadPoolExecutor(2) as ex:
        a, b = list(ex.map(run, range(2)))
    assert torch.equal(a, torch.full((3,), 3.0)) and torch.equal(a, b)


def test_baby_dead_child_detected():
    store = make_store()
    pg = ProcessGroupBabyGloo(timeout=timedelta(seconds=20))
    try:
        pg.configure(f"127.0.0.1:{store.port}/dead", 0, 1)
        pg._p.kill()
        pg._p.join()
        with pytest.raises(RuntimeError, match="child process .* is dead"):
            pg.allreduce([torch.ones(1)], ReduceOp.SUM)
    finally:
        pg.shutdown()


def test_error_swallowing_wrapper():
    inner = ProcessGroupDummy(0, 1)
    pg = ErrorSwallowingProcessGroupWrapper(inner)
    check_collectives(pg, torch.randn(3))
    t = torch.zeros(2)
    work = pg.allreduce([t], ReduceOp.SUM)
    assert isinstance(work, _ErrorSwallowingWork)
    work.wait()
    work.get_future().wait()

    err = RuntimeError("injected")
    pg.report_error(err)
    assert pg.error() is err
    work = pg.allreduce([t], ReduceOp.SUM)
    assert isinstance(work, _DummyWork)
    work.wait()

    pg.configure("addr", 0, 1)  # clears the error, delegates to the inner group
    assert pg.error() is None and inner.configure_count == 1
    assert isinstance(pg.allreduce([t], ReduceOp.SUM), _ErrorSwallowingWork)


def test_error_swallowing_catches_failures():
    inner = MagicMock(spec=ProcessGroupDummy)
    inner.allreduce.side_effect = RuntimeError("kaboom")
    pg = ErrorSwallowingProcessGroupWrapper(inner)
    work = pg.allreduce([torch.zeros(1)], ReduceOp.SUM)
    assert isinstance(work, _DummyWork)
    assert isinstance(pg.error(), RuntimeError)


def test_managed_process_group():
    manager = create_autospec(Manager)
    manager.errored.return_value = None
    manager._pg = ProcessGroupDummy(0, 1)
    manager.num_participants.return_value = 123
    pg = ManagedProcessGroup(manager)
    manager.wrap_future.side_effect = lambda fut, default: fut

    t = torch.zeros(2, 3)
    work = pg.allreduce([t], ReduceOp.SUM)
    assert isinstance(work, _ManagedWork)
    work.wait()
    work.get_future().wait()
    assert pg.size() == 123
    assert manager.report_error.call_count == 0
    assert manager.wrap_future.call_count == 1
    assert manager.wait_quorum.call_count == 1

    manager.errored.return_value = RuntimeError("step failed")
    assert isinstance(pg.allreduce([t], ReduceOp.SUM), _DummyWork)


def test_managed_process_group_averages_over_participants_and_mutes_a_healing_replica():
    """c10d hands the reduction as a ReduceOp object inside AllreduceOptions (that is what FSDP2 does);
    AVG must divide by the participants, and a replica that is still healing must add zeros."""
    store = make_store()
    inner = ProcessGroupGloo()
    inner.configure(f"127.0.0.1:{store.port}/managed_avg", 0, 1)
    manager = create_autospec(Manager)
    manager.errored.return_value = None
    manager._pg = inner
    manager.num_participants.return_value = 4
    manager.is_participating.return_value = True
    manager.wrap_future.side_effect = lambda fut, default: fut
    pg = ManagedProcessGroup(manager)
    opts = AllreduceOptions()
    opts.reduceOp = ReduceOp.AVG
    t = torch.full((8,), 6.0)
    pg.allreduce([t], opts).wait()
    assert torch.allclose(t, torch.full((8,), 1.5))  # one member, four participants
    opts.reduceOp = ReduceOp.SUM
    t = torch.full((8,), 6.0)
    pg.allreduce([t], opts).wait()
    assert torch.allclose(t, torch.full((8,), 6.0))
    manager.is_participating.return_value = False
    t = torch.full((8,), 6.0)
    pg.allreduce([t], opts).wait()
    assert torch.equal(t, torch.zeros(8))
    assert manager.report_error.call_count == 0


def test_register_for_functional_collectives(tmp_path):
    """A registered group resolves through c10d's registry (needs a default group)."""
    store = make_store()
    dist.init_process_group(backend="gloo", rank=0, world_size=1, store=store)
    try:
        store_addr = f"127.0.0.1:{store.port}/reg"
        pg = ProcessGroupGloo()
        pg.configure(store_addr, 0, 1)
        registered = pg.register("test_group")
        from torch.distributed import _functional_collectives as fc

        t = torch.ones(3)
        out = fc.all_reduce(t, "sum", registered)
        assert torch.equal(torch.as_tensor(out), torch.ones(3))
    finally:
        dist.destroy_process_group()
