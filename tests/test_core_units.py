"""Unit tests of futures, checkpoint transport, optimizer wrapper, sampler, DDP hook.

Scenarios follow the reference's futures_test.py, checkpointing_test.py, optim_test.py,
data_test.py and ddp_test.py.
"""

import os
import threading
import time
import urllib.error
from datetime import timedelta
from unittest.mock import MagicMock, create_autospec

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.futures import Future

from torchft_b200.checkpointing import CheckpointServer, _timed_acquire
from torchft_b200.data import DistributedSampler
from torchft_b200.ddp import DistributedDataParallel, PureDistributedDataParallel
from torchft_b200.futures import future_timeout, future_wait
from torchft_b200.manager import Manager
from torchft_b200.optim import OptimizerWrapper


# ------------------------------------------------------------------ futures
def test_future_wait_result_and_timeout():
    fut = Future()
    with pytest.raises(TimeoutError, match="future did not complete within"):
        future_wait(fut, timedelta(seconds=0.01))
    fut = Future()
    fut.set_result(1)
    assert future_wait(fut, timedelta(seconds=1.0)) == 1
    fut = Future()
    fut.set_exception(RuntimeError("test"))
    with pytest.raises(RuntimeError, match="test"):
        future_wait(fut, timedelta(seconds=1.0))


def test_future_timeout_fires():
    fut = Future()
    timed = future_timeout(fut, timedelta(seconds=0.01))
    with pytest.raises(TimeoutError, match="future did not complete within"):
        timed.wait()


def test_future_timeout_passes_result_and_exception():
    fut = Future()
    timed = future_timeout(fut, timedelta(seconds=10))
    fut.set_result(5)
    assert timed.wait() == 5
    fut = Future()
    timed = future_timeout(fut, timedelta(seconds=10))
    fut.set_exception(RuntimeError("boom"))
    with pytest.raises(RuntimeError, match="boom"):
        timed.wait()


def test_future_timeout_many_deadlines_in_order():
    futs = [Future() for _ in range(20)]
    timed = [future_timeout(f, timedelta(seconds=0.3 + 0.001 * i)) for i, f in enumerate(futs)]
    futs[3].set_result("ok")
    assert timed[3].wait() == "ok"
    for i, t in enumerate(timed):
        if i == 3:
            continue
        with pytest.raises(TimeoutError):
            t.wait()


# ------------------------------------------------------------------ checkpoint server
def test_checkpoint_server_round_trip_and_gate():
    expected = {"state": "dict", "tensor": torch.arange(5)}
    server = CheckpointServer(timeout=timedelta(seconds=10))
    try:
        server.send_checkpoint(dst_ranks=[], step=1234, state_dict=expected, timeout=timedelta(seconds=10))
        meta = server.metadata()
        assert meta.endswith("/checkpoint/")
        out = server.recv_checkpoint(src_rank=0, metadata=meta, step=1234, timeout=timedelta(seconds=10))
        assert out["state"] == "dict" and torch.equal(out["tensor"], expected["tensor"])

        # wrong step -> 400
        with pytest.raises(urllib.error.HTTPError, match="Error 400"):
            server.recv_checkpoint(src_rank=0, metadata=meta, step=1, timeout=timedelta(seconds=10))

        # closed gate -> the request blocks until the (short) client timeout
        server.disallow_checkpoint()
        with pytest.raises((TimeoutError, urllib.error.URLError, OSError)):
            server.recv_checkpoint(src_rank=0, metadata=meta, step=1234, timeout=timedelta(seconds=0.2))
    finally:
        server.shutdown()


def test_checkpoint_server_serves_views_of_one_arena():
    """State kept as bf16 and fp32 views of ONE byte buffer (a heap) is sent tensor by tensor."""
    arena = torch.zeros(1 << 16, dtype=torch.uint8)
    a = arena[:1024].view(torch.bfloat16)
    b = arena[4096 : 4096 + 4096].view(torch.float32)
    a.copy_(torch.arange(512).to(torch.bfloat16))
    b.copy_(torch.arange(1024).float())
    server = CheckpointServer(timeout=timedelta(seconds=10))
    try:
        server.send_checkpoint([], 3, {"p": [a], "m": b}, timedelta(seconds=10))
        out = server.recv_checkpoint(0, server.metadata(), 3, timedelta(seconds=10))
        assert torch.equal(out["p"][0], a) and torch.equal(out["m"], b)
        assert out["m"].untyped_storage().nbytes() == b.numel() * 4  # not the whole arena
    finally:
        server.shutdown()


def test_checkpoint_server_gate_blocks_until_allowed():
    server = CheckpointServer(timeout=timedelta(seconds=10))
    try:
        result = {}

        def fetch():
            result["v"] = server.recv_checkpoint(0, server.metadata(), 7, timedelta(seconds=10))

        t = threading.Thread(target=fetch)
        t.start()
        time.sleep(0.2)
        assert "v" not in result  # still gated
        server.send_checkpoint([1], 7, {"x": 1}, timedelta(seconds=10))
        t.join(timeout=10)
        assert result["v"] == {"x": 1}
    finally:
        server.shutdown()


def test_timed_acquire():
    lock = threading.Lock()
    with _timed_acquire(lock, timedelta(seconds=1)):
        assert lock.locked()
        with pytest.raises(TimeoutError, match="timed out acquiring lock after"):
            with _timed_acquire(lock, timedelta(seconds=0.01)):
                pass
    assert not lock.locked()


# ------------------------------------------------------------------ optimizer wrapper
def test_optimizer_wrapper_gates_step():
    manager = create_autospec(Manager)
    m = nn.Linear(3, 4)
    base = torch.optim.AdamW(m.parameters())
    optim = OptimizerWrapper(manager, base)
    optim.add_param_group({"params": nn.Linear(2, 2).parameters(), "lr": 1})
    assert len(optim.param_groups) == 2
    optim.load_state_dict(optim.state_dict())

    optim.zero_grad()
    assert manager.start_quorum.call_count == 1

    m(torch.rand(2, 3)).sum().backward()
    before = [p.detach().clone() for p in m.parameters()]
    manager.should_commit.return_value = False
    optim.step()
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
    manager.should_commit.return_value = True
    optim.step()
    assert manager.should_commit.call_count == 2
    assert not all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
    assert optim.state is base.state


# ------------------------------------------------------------------ sampler
def test_distributed_sampler_arithmetic():
    dataset = list(range(1000))
    sampler = DistributedSampler(dataset, replica_group=1, num_replica_groups=2, rank=3, num_replicas=4, shuffle=False)
    assert sampler.global_rank == 3 + 1 * 4
    assert sampler.global_world_size == 8
    it = iter(sampler)
    assert next(it) == 7
    assert next(it) == 15
    assert len(sampler) == 125


# ------------------------------------------------------------------ DDP
def _manager_mock_allreduce():
    manager = create_autospec(Manager)
    calls = []

    def allreduce(t):
        calls.append(t.numel())
        f = Future()
        f.set_result(t)
        return f

    manager.allreduce = allreduce
    return manager, calls


def test_ddp_routes_buckets_through_manager():
    manager, calls = _manager_mock_allreduce()
    m = nn.Linear(3, 4)
    ddp = DistributedDataParallel(manager, m)
    ddp(torch.rand(2, 3)).mean().backward()
    assert sum(calls) == sum(p.numel() for p in m.parameters())
    for p in m.parameters():
        assert p.grad is not None


def test_pure_ddp_hooks_every_parameter():
    manager, calls = _manager_mock_allreduce()
    m = nn.Linear(3, 4)
    ddp = PureDistributedDataParallel(manager, m)
    ddp(torch.rand(2, 3)).mean().backward()
    assert sorted(calls) == sorted(p.numel() for p in m.parameters())


# ------------------------------------------------------------------ durable checkpoints
def test_durable_checkpoint_round_trip(tmp_path):
    from unittest.mock import MagicMock

    from torchft_b200.utils.durable import latest_step, load_checkpoint, save_checkpoint

    manager = MagicMock()
    manager.current_step.return_value = 7
    manager.state_dict.return_value = {"step": 7, "batches_committed": 14}
    model = nn.Linear(3, 2)
    for rank in (0, 1):
        path = save_checkpoint(str(tmp_path), manager, {"model": model.state_dict(), "rank": rank}, rank=rank,
                               dataloader_state={"position": 70})
        assert path.endswith(f"step0000000007/rank{rank:05d}.pt")
    # a newer step that only rank 0 finished writing does not count for a two-rank job
    manager.current_step.return_value = 9
    manager.state_dict.return_value = {"step": 9, "batches_committed": 18}
    save_checkpoint(str(tmp_path), manager, {"model": model.state_dict(), "rank": 0}, rank=0)
    assert latest_step(str(tmp_path), world_size=2) == 7 and latest_step(str(tmp_path), world_size=1) == 9
    assert not [f for f in os.listdir(tmp_path / "step0000000007") if f.startswith(".tmp-")]

    restored = MagicMock()
    out = load_checkpoint(str(tmp_path), restored, rank=1, world_size=2)
    restored.load_state_dict.assert_called_once_with({"step": 7, "batches_committed": 14})
    assert out["user"]["rank"] == 1 and out["dataloader"] == {"position": 70}
    assert torch.equal(out["user"]["model"]["weight"], model.state_dict()["weight"])
    assert load_checkpoint(str(tmp_path / "nothing"), restored) is None


def test_checkpoint_gate_counts_readers_and_close_waits_for_them():
    """Two peers stream at once; closing the gate returns only after both have left."""
    from torchft_b200.checkpointing import _Gate

    gate = _Gate()
    with pytest.raises(TimeoutError):
        with gate.reading(timedelta(seconds=0.05)):
            pass
    gate.open(5, {"w": 1})
    inside = threading.Barrier(3)
    leave = threading.Event()
    seen = []

    def reader():
        with gate.reading(timedelta(seconds=5)) as (step, state):
            seen.append((step, state["w"]))
            inside.wait(timeout=5)
            leave.wait(timeout=5)

    readers = [threading.Thread(target=reader) for _ in range(2)]
    for t in readers:
        t.start()
    inside.wait(timeout=5)  # both readers are in at the same time
    closed = threading.Event()
    closer = threading.Thread(target=lambda: (gate.close(), closed.set()))
    closer.start()
    time.sleep(0.1)
    assert not closed.is_set()  # readers still streaming
    leave.set()
    closer.join(timeout=5)
    assert closed.is_set() and seen == [(5, 1), (5, 1)]
    with pytest.raises(TimeoutError):
        with gate.reading(timedelta(seconds=0.05)):
            pass


def test_optimizer_wrapper_is_a_proxy_that_lr_schedulers_accept():
    """A scheduler built on the wrapper changes the wrapped optimizer's learning rate, and its
    re-binding of ``step`` neither bypasses the commit vote nor recurses."""
    manager = create_autospec(Manager)
    manager.should_commit.return_value = True
    layer = nn.Linear(2, 2)
    base = torch.optim.SGD(layer.parameters(), lr=1.0)
    optim = OptimizerWrapper(manager, base)
    assert isinstance(optim, torch.optim.Optimizer)
    scheduler = torch.optim.lr_scheduler.StepLR(optim, step_size=1, gamma=0.5)
    optim.zero_grad()
    layer(torch.ones(2)).sum().backward()
    before = layer.weight.detach().clone()
    optim.step()
    scheduler.step()
    assert manager.should_commit.call_count == 1
    assert not torch.equal(layer.weight, before)
    assert base.param_groups[0]["lr"] == 0.5 and optim.param_groups is base.param_groups
    optim.defaults["marker"] = 1  # attributes that are not the wrapper's own live on the wrapped optimizer
    assert base.defaults["marker"] == 1

    manager.should_commit.return_value = False
    before = layer.weight.detach().clone()
    optim.step()
    assert torch.equal(layer.weight, before)


def test_pure_ddp_remove_hooks_and_sampler_bounds():
    manager = create_autospec(Manager)
    model = PureDistributedDataParallel(manager, nn.Linear(3, 1))
    model(torch.ones(3)).sum().backward()
    assert manager.allreduce.call_count == 2
    model.remove_hooks()
    model(torch.ones(3)).sum().backward()
    assert manager.allreduce.call_count == 2

    with pytest.raises(ValueError):
        DistributedSampler(list(range(8)), replica_group=2, num_replica_groups=2, rank=0, num_replicas=2)
    with pytest.raises(ValueError):
        DistributedSampler(list(range(8)), replica_group=0, num_replica_groups=2, rank=2, num_replicas=2)


def test_fused_adamw_matches_torch_and_keeps_its_state_tensors():
    """The plain-arithmetic path (parameters that are not bf16 CUDA tensors) against ``torch.optim.AdamW``;
    the state dict hands out the live fp32 moments and loading copies into them in place."""
    from torchft_b200.optim import FusedAdamW

    torch.manual_seed(0)
    ours = [nn.Parameter(torch.randn(17, 5)), nn.Parameter(torch.randn(33))]
    theirs = [nn.Parameter(p.detach().clone()) for p in ours]
    kw = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    a, b = FusedAdamW(ours, **kw), torch.optim.AdamW(theirs, **kw)
    assert all(a.state[p]["exp_avg"].dtype == torch.float32 for p in ours)  # allocated before the first step
    for _ in range(5):
        for p, q in zip(ours, theirs):
            g = torch.randn_like(p)
            p.grad, q.grad = g, g.clone()
        a.step()
        b.step()
    for p, q in zip(ours, theirs):
        assert torch.allclose(p, q, rtol=1e-5, atol=1e-6)
        assert torch.allclose(a.state[p]["exp_avg_sq"], b.state[q]["exp_avg_sq"], rtol=1e-5, atol=1e-8)

    fresh = [nn.Parameter(torch.zeros_like(p)) for p in ours]
    c = FusedAdamW(fresh, **kw)
    kept = [c.state[p]["exp_avg"] for p in fresh]
    c.load_state_dict(a.state_dict())
    assert c.param_groups[0]["step"] == 5 and c.param_groups[0]["betas"] == (0.9, 0.95)
    for p, q, t in zip(fresh, ours, kept):
        assert c.state[p]["exp_avg"] is t and torch.equal(t, a.state[q]["exp_avg"])
    # behind the fault-tolerance wrapper the step is gated by the commit vote
    manager = create_autospec(Manager)
    manager.should_commit.return_value = False
    wrapped = OptimizerWrapper(manager, a)
    before = ours[0].detach().clone()
    wrapped.step()
    assert torch.equal(ours[0], before)
    with pytest.raises(ValueError):
        FusedAdamW(ours, lr=-1.0)


def test_peer_mappings_are_shared_and_closed_with_the_last_user(monkeypatch):
    """``_PeerMappings`` opens a peer's heap once per process however many users map it and closes it when the
    last one lets go (the peer's GPU memory stays allocated for as long as a mapping exists).  The CUDA-IPC
    calls are replaced by a fake here."""
    import contextlib
    import ctypes

    from torchft_b200.parallel import nvlink

    calls = []

    class FakeLib:
        @staticmethod
        def tft_p2p_peer_open(handle, out):
            calls.append(("open", bytes(handle)))
            ctypes.cast(out, ctypes.POINTER(ctypes.c_void_p))[0] = 0x1000 * len(calls)
            return 0

        @staticmethod
        def tft_p2p_peer_close(ptr):
            calls.append(("close", ptr.value))
            return 0

    monkeypatch.setattr(nvlink, "_lib_p2p", lambda: FakeLib)
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    monkeypatch.setattr(nvlink._PeerMappings, "_table", {})
    dev = torch.device("cuda", 0)
    a = nvlink._PeerMappings.acquire(b"peer-a", dev)
    assert nvlink._PeerMappings.acquire(b"peer-a", dev) == a  # second user: same mapping, no second open
    b = nvlink._PeerMappings.acquire(b"peer-b", dev)
    assert a != b and nvlink._PeerMappings.open_count() == 2 and [c[0] for c in calls] == ["open", "open"]
    nvlink._PeerMappings.release(b"peer-a", dev)
    assert nvlink._PeerMappings.open_count() == 2  # one user of peer-a is left
    nvlink._PeerMappings.release(b"peer-a", dev)
    assert nvlink._PeerMappings.open_count() == 1 and calls[-1] == ("close", a)
    nvlink._PeerMappings.release(b"peer-a", dev)  # unknown handle: nothing to do
    nvlink._PeerMappings.release(b"peer-b", dev)
    assert nvlink._PeerMappings.open_count() == 0 and calls[-1] == ("close", b)


def test_api_reference_pages_name_importable_modules():
    """Every ``automodule`` of the Sphinx pages under ``docs/source`` can be imported (the docs job would fail otherwise)."""
    import importlib
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pages = os.path.join(root, "docs", "source")
    names = []
    for page in sorted(os.listdir(pages)):
        if page.endswith(".rst"):
            with open(os.path.join(pages, page)) as f:
                names += re.findall(r"^\.\. automodule:: (\S+)", f.read(), flags=re.M)
    assert len(names) >= 20
    for name in names:
        importlib.import_module(name)
    with open(os.path.join(pages, "index.rst")) as f:
        listed = set(re.findall(r"^    (\w+)$", f.read(), flags=re.M))
    assert listed == {p[:-4] for p in os.listdir(pages) if p.endswith(".rst")} - {"index"}
