"""End-to-end fault-injection tests on CPU: a real lighthouse, real manager servers, one
thread per replica group (and per rank), gloo process groups.  A failure is an
exception raised in a rank's training loop between steps; the whole replica group is
then restarted, gets a new replica id and heals from the survivor.  The oracle is
equality of the final state dicts across replicas.  Structure follows the reference's
manager_integ_test.py (FailureInjector / Runner)."""

import copy
import threading
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from contextlib import ExitStack
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Any, Callable, Dict, List, Set, Tuple

import pytest
import torch
import torch.distributed as dist
from torch import nn, optim

from torchft_b200._control import Lighthouse
from torchft_b200.ddp import DistributedDataParallel
from torchft_b200.local_sgd import DiLoCo, LocalSGD
from torchft_b200.manager import Manager
from torchft_b200.models.lenet import LeNet
from torchft_b200.optim import OptimizerWrapper
from torchft_b200.process_group import ProcessGroupGloo


class InjectedFailure(Exception):
    """Raised inside a rank's training loop to stand for the loss of that rank."""


class FailureInjector:
    """A plan of one-shot failures, keyed by (rank, step); shared by the threads of a replica group.

    ``fail_at`` adds a point to the plan; ``check`` is called by every rank at every step and raises once
    when that rank reaches a planned step (the entry is consumed, so the restarted group passes the same
    step unharmed).  ``count`` says how many failures fired.
    """

    def __init__(self) -> None:
        self._guard = threading.Lock()
        self._plan: Set[Tuple[int, int]] = set()
        self.count = 0

    def fail_at(self, rank: int, step: int) -> "FailureInjector":
        with self._guard:
            self._plan.add((rank, step))
        return self

    def check(self, rank: int, step: int) -> None:
        with self._guard:
            due = (rank, step) in self._plan
            if due:
                self._plan.discard((rank, step))
                self.count += 1
        if due:
            raise InjectedFailure(f"injected failure rank={rank} step={step}")


@dataclass
class Runner:
    replica_id: int
    lighthouse_address: str
    failure_injector: FailureInjector
    train_loop: Callable[..., Dict[str, Any]]
    world_size: int = 1
    attempts: int = 3
    manager_args: Dict[str, object] = field(default_factory=dict)
    train_loop_args: Dict[str, Any] = field(default_factory=dict)

    def _replica_main(self) -> List[Dict[str, Any]]:
        store = dist.TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
        with ThreadPoolExecutor(max_workers=self.world_size, thread_name_prefix=f"replica{self.replica_id}") as ex:
            futs = [
                ex.submit(self.train_loop, rank=rank, store_port=store.port, runner=self, **self.train_loop_args)
                for rank in range(self.world_size)
            ]
            for fut in as_completed(futs):
                try:
                    fut.result()
                except Exception:
                    ex.shutdown(wait=False, cancel_futures=True)
                    raise
            return [f.result() for f in futs]

    def run_replica(self) -> List[Dict[str, Any]]:
        for _ in range(self.attempts):
            try:
                return self._replica_main()
            except InjectedFailure:
                continue  # the group restarts as a whole
        raise RuntimeError("ran out of attempts")


def make_manager(runner: Runner, rank: int, store_port: int, pg, load_state_dict, state_dict, **kw) -> Manager:
    args = dict(
        pg=pg,
        min_replica_size=2,
        load_state_dict=load_state_dict,
        state_dict=state_dict,
        replica_id=str(runner.replica_id),
        store_addr="127.0.0.1",
        store_port=store_port,
        rank=rank,
        world_size=runner.world_size,
        lighthouse_addr=runner.lighthouse_address,
        port=0,
        timeout=timedelta(seconds=20),
        quorum_timeout=timedelta(seconds=30),
    )
    args.update(runner.manager_args)
    args.update(kw)
    return Manager(**args)


def ddp_train_loop(rank: int, store_port: int, runner: Runner, total_steps: int = 4, model_fn=None, batch_fn=None) -> Dict[str, Any]:
    with ExitStack() as stack:
        def load_state_dict(sd):
            m.load_state_dict(sd["model"])
            optimizer.load_state_dict(sd["optim"])

        def state_dict():
            return {"model": m.state_dict(), "optim": optimizer.state_dict()}

        pg = ProcessGroupGloo(timeout=timedelta(seconds=20))
        manager = make_manager(runner, rank, store_port, pg, load_state_dict, state_dict)
        stack.callback(lambda: manager.shutdown(wait=False))

        torch.manual_seed(1234 + runner.replica_id)  # different init per replica: healing must fix it
        base = model_fn() if model_fn else nn.Sequential(nn.Linear(3, 4), nn.Sigmoid())
        m = DistributedDataParallel(manager, base)
        optimizer = OptimizerWrapper(manager, optim.AdamW(m.parameters(), lr=1e-3) if model_fn else optim.Adam(m.parameters()))
        criterion = nn.CrossEntropyLoss()

        while True:
            step = manager.current_step()
            gen = torch.Generator().manual_seed(step * 100 + runner.replica_id)
            if batch_fn:
                inputs, labels = batch_fn(gen)
            else:
                inputs = torch.rand(2, 3, generator=gen)
                labels = torch.randint(4, (2,), generator=gen)
            optimizer.zero_grad()
            loss = criterion(m(inputs), labels)
            loss.backward()
            optimizer.step()
            if manager.current_step() >= total_steps:
                break
            runner.failure_injector.check(rank, manager.current_step())
        return {k: v.detach().clone() if isinstance(v, torch.Tensor) else copy.deepcopy(v) for k, v in state_dict()["model"].items()}


def run_groups(lighthouse, injectors, train_loop, world_size=1, manager_args=None, **loop_args):
    with ThreadPoolExecutor(max_workers=len(injectors)) as ex:
        futs = []
        for replica_id, inj in enumerate(injectors):
            runner = Runner(
                replica_id=replica_id,
                lighthouse_address=lighthouse.address(),
                failure_injector=inj,
                train_loop=train_loop,
                world_size=world_size,
                manager_args=manager_args or {},
                train_loop_args=loop_args,
            )
            futs.append(ex.submit(runner.run_replica))
        return [f.result(timeout=240) for f in futs]


def assert_replicas_equal(results):
    """Local rank r of every replica group must hold the same state (ranks of one group
    are different shards in general, so they are only compared across groups)."""
    for rank, ref in enumerate(results[0]):
        for group in results[1:]:
            for k in ref:
                torch.testing.assert_close(group[rank][k], ref[k], msg=f"mismatch in {k} (local rank {rank})")


@pytest.fixture
def lighthouse():
    lh = Lighthouse(bind="[::]:0", min_replicas=2, join_timeout_ms=10000)
    yield lh
    lh.shutdown()


def test_ddp_healthy(lighthouse):
    results = run_groups(lighthouse, [FailureInjector(), FailureInjector()], ddp_train_loop)
    assert_replicas_equal(results)


@pytest.mark.parametrize("use_async_quorum", [True, False])
def test_ddp_recovery(lighthouse, use_async_quorum):
    injectors = [FailureInjector(), FailureInjector().fail_at(0, 2)]
    results = run_groups(lighthouse, injectors, ddp_train_loop, manager_args={"use_async_quorum": use_async_quorum}, total_steps=5)
    assert_replicas_equal(results)
    assert injectors[1].count == 1


def test_ddp_recovery_multi_rank(lighthouse):
    injectors = [FailureInjector(), FailureInjector().fail_at(0, 2).fail_at(1, 2)]
    results = run_groups(lighthouse, injectors, ddp_train_loop, world_size=2, total_steps=5)
    assert_replicas_equal(results)


def test_lenet_kill_and_heal():
    """LeNet DDP, 2 groups x 1 rank, AdamW 1e-3, batch 64 of synthetic 3x32x32 images;
    replica 1 dies after step 50 of 100, rejoins and heals; final weights must agree."""
    lh = Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=10000, quorum_tick_ms=100)
    try:
        def batch(gen):
            return torch.randn(64, 3, 32, 32, generator=gen), torch.randint(10, (64,), generator=gen)

        injectors = [FailureInjector(), FailureInjector().fail_at(0, 50)]
        results = run_groups(
            lh, injectors, ddp_train_loop, manager_args={"min_replica_size": 1}, total_steps=100, model_fn=LeNet, batch_fn=batch
        )
        assert injectors[1].count == 1
        assert_replicas_equal(results)
    finally:
        lh.shutdown()


def local_sgd_train_loop(rank: int, store_port: int, runner: Runner, total_steps: int = 4, diloco: bool = False) -> Dict[str, Any]:
    with ExitStack() as stack:
        def load_state_dict(sd):
            m.load_state_dict(sd["model"])
            inner.load_state_dict(sd["inner"])
            if diloco:
                outer.load_state_dict(sd["outer"])
                for name, t in sd["backup"].items():
                    algo._backup_parameters[name].copy_(t)

        def state_dict():
            sd = {"model": m.state_dict(), "inner": inner.state_dict()}
            if diloco:
                sd["outer"] = outer.state_dict()
                sd["backup"] = {k: v.clone() for k, v in algo._backup_parameters.items()}
            return sd

        pg = ProcessGroupGloo(timeout=timedelta(seconds=20))
        manager = make_manager(runner, rank, store_port, pg, load_state_dict, state_dict, use_async_quorum=False)
        stack.callback(lambda: manager.shutdown(wait=False))

        torch.manual_seed(42 if diloco else 1234 + runner.replica_id)
        m = nn.Sequential(nn.Linear(3, 4), nn.Sigmoid())
        inner = optim.AdamW(m.parameters(), lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95))
        if diloco:
            outer = optim.SGD(m.parameters(), lr=0.7, momentum=0.9, nesterov=True)
            algo = DiLoCo(manager, m, inner, outer, sync_every=2)
        else:
            algo = LocalSGD(manager, m, inner, sync_every=2)
        criterion = nn.CrossEntropyLoss()
        with algo:
            while True:
                gen = torch.Generator().manual_seed(manager.current_step() * 100 + algo._local_step + runner.replica_id)
                inputs = torch.rand(2, 3, generator=gen)
                labels = torch.randint(4, (2,), generator=gen)
                inner.zero_grad()
                criterion(m(inputs), labels).backward()
                inner.step()
                if manager.current_step() >= total_steps:
                    break
                runner.failure_injector.check(rank, manager.current_step())
        out = {k: v.detach().clone() for k, v in m.state_dict().items()}
        for k, v in algo._backup_parameters.items():
            out["backup." + k] = v.detach().clone()
        return out


def test_local_sgd_recovery(lighthouse):
    injectors = [FailureInjector(), FailureInjector().fail_at(0, 2)]
    results = run_groups(lighthouse, injectors, local_sgd_train_loop, total_steps=4)
    assert_replicas_equal(results)
    assert injectors[1].count == 1


def test_diloco_healthy(lighthouse):
    results = run_groups(lighthouse, [FailureInjector(), FailureInjector()], local_sgd_train_loop, total_steps=4, diloco=True)
    assert_replicas_equal(results)


def test_diloco_recovery(lighthouse):
    injectors = [FailureInjector(), FailureInjector().fail_at(0, 2)]
    results = run_groups(lighthouse, injectors, local_sgd_train_loop, total_steps=5, diloco=True)
    assert_replicas_equal(results)
    assert injectors[1].count == 1


def test_quorum_and_commit_timeouts_surface_fast():
    lh = Lighthouse(bind="[::]:0", min_replicas=2)
    store = dist.TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
    manager = Manager(
        pg=ProcessGroupGloo(),
        min_replica_size=2,
        load_state_dict=lambda x: None,
        state_dict=lambda: None,
        store_addr="127.0.0.1",
        store_port=store.port,
        rank=0,
        world_size=2,
        lighthouse_addr=lh.address(),
        port=0,
        use_async_quorum=False,
    )
    try:
        t0 = time.time()
        with pytest.raises(TimeoutError, match="status: Cancelled, message.*Timeout expired"):
            manager.start_quorum(timeout=timedelta(seconds=0.01))
        assert time.time() - t0 < 1.0
        t0 = time.time()
        with pytest.raises(TimeoutError, match="status: Cancelled, message.*Timeout expired"):
            manager.should_commit(timeout=timedelta(seconds=0.01))
        assert time.time() - t0 < 1.0
    finally:
        manager.shutdown(wait=False)
        lh.shutdown()
