"""LocalSGD / DiLoCo unit tests with a mocked Manager, the parameter server round trip and
the managed device mesh (4 gloo processes).  Scenarios follow the reference's
local_sgd_test.py, parameter_server_test.py and device_mesh_test.py."""

import io
import os
import time
from datetime import timedelta
from unittest.mock import Mock, create_autospec

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn, optim

from torchft_b200.local_sgd import DiLoCo, LocalSGD
from torchft_b200.manager import Manager
from torchft_b200.parameter_server import ParameterServer
from torchft_b200.process_group import ProcessGroupGloo, ft_init_device_mesh


class Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.model = nn.Sequential(nn.Linear(3, 4), nn.Tanh(), nn.Linear(4, 2))  # no dead units: every parameter gets a gradient

    def forward(self, x):
        return self.model(x)


def mock_manager(use_async_quorum=True):
    manager = create_autospec(Manager)
    manager._use_async_quorum = use_async_quorum

    def allreduce(t):
        f = torch.futures.Future()
        f.set_result(t)
        return f

    manager.allreduce.side_effect = allreduce
    return manager


def params_copy(m):
    return {n: p.detach().clone() for n, p in m.named_parameters()}


def test_local_sgd_sync_every_and_rollback():
    model = Tiny()
    opt = optim.SGD(model.parameters(), lr=0.1)
    manager = mock_manager()
    manager.should_commit.return_value = True
    with LocalSGD(manager, model, opt, sync_every=2) as sgd:
        assert sgd._local_step == 0
        start = params_copy(model)
        x = torch.rand(5, 3)
        for expected_quorums, expected_local in [(0, 1), (1, 0)]:
            opt.zero_grad()
            model(x).sum().backward()
            opt.step()
            assert manager.start_quorum.call_count == expected_quorums
            assert sgd._local_step == expected_local
        # committed: backup == current parameters
        for n, p in model.named_parameters():
            torch.testing.assert_close(sgd._backup_parameters[n], p.detach())
            assert not torch.equal(p.detach(), start[n])
        # bucketed: a handful of allreduces, not one per tensor
        assert manager.allreduce.call_count == 1

        committed = params_copy(model)
        manager.should_commit.return_value = False
        for _ in range(2):
            opt.zero_grad()
            model(x).sum().backward()
            opt.step()
        # not committed: rolled back to the last synchronised weights
        for n, p in model.named_parameters():
            torch.testing.assert_close(p.detach(), committed[n])


def test_local_sgd_restores_on_exception():
    model = Tiny()
    opt = optim.SGD(model.parameters(), lr=0.1)
    manager = mock_manager()
    start = params_copy(model)
    with pytest.raises(RuntimeError, match="boom"):
        with LocalSGD(manager, model, opt, sync_every=100):
            opt.zero_grad()
            model(torch.rand(5, 3)).sum().backward()
            opt.step()
            raise RuntimeError("boom")
    for n, p in model.named_parameters():
        torch.testing.assert_close(p.detach(), start[n])


def test_diloco_requires_sync_quorum():
    model = Tiny()
    with pytest.raises(ValueError, match="synchronous quorum"):
        DiLoCo(mock_manager(True), model, optim.SGD(model.parameters(), lr=0.1), optim.SGD(model.parameters(), lr=0.5), sync_every=2)


def test_diloco_matches_manual_outer_step():
    torch.manual_seed(0)
    model = Tiny()
    inner = optim.AdamW(model.parameters(), lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95))
    outer = optim.SGD(model.parameters(), lr=0.7, momentum=0.9, nesterov=True)
    manager = mock_manager(False)
    manager.should_commit.return_value = True
    global0 = params_copy(model)
    with DiLoCo(manager, model, inner, outer, sync_every=2) as diloco:
        x = torch.rand(5, 3)
        for _ in range(2):
            inner.zero_grad()
            model(x).sum().backward()
            inner.step()
        assert manager.start_quorum.call_count == 1 and diloco._local_step == 0
    # single replica: averaged pseudo-gradient == own delta; first Nesterov step:
    # buf = g ; step = g + mu*buf ; new = global - lr*step
    # We cannot see the pre-sync local weights any more, but new global and backup must agree
    for n, p in model.named_parameters():
        torch.testing.assert_close(diloco._backup_parameters[n], p.detach())
        assert not torch.equal(p.detach(), global0[n])
        buf = outer.state[p]["momentum_buffer"]
        # new = global0 - lr*(1+mu)*g with buf == g  =>  g = (global0 - new)/(lr*(1+mu))
        g = (global0[n] - p.detach()) / (0.7 * 1.9)
        torch.testing.assert_close(buf, g, rtol=1e-4, atol=1e-6)


def test_diloco_no_commit_restores_global():
    model = Tiny()
    inner = optim.SGD(model.parameters(), lr=0.1)
    outer = optim.SGD(model.parameters(), lr=0.7, momentum=0.9, nesterov=True)
    manager = mock_manager(False)
    manager.should_commit.return_value = False
    global0 = params_copy(model)
    with DiLoCo(manager, model, inner, outer, sync_every=1):
        inner.zero_grad()
        model(torch.rand(5, 3)).sum().backward()
        inner.step()
    for n, p in model.named_parameters():
        torch.testing.assert_close(p.detach(), global0[n])
        assert p.grad is None


class EchoPS(ParameterServer):
    @classmethod
    def new_process_group(cls):
        return ProcessGroupGloo(timeout=timedelta(seconds=20))

    def forward(self, session_id, pg):
        data = torch.zeros(2, 3)
        pg.broadcast_one(data, 1).wait()  # from the client
        data += 23
        pg.broadcast_one(data, 0).wait()  # back to the client


def test_parameter_server_round_trip():
    ps = EchoPS(port=0)
    try:
        assert ps.address().endswith("/new_session")
        pg = EchoPS.new_session(ps.address())
        data = torch.full((2, 3), 12.0)
        pg.broadcast_one(data, 1).wait()
        pg.broadcast_one(data, 0).wait()
        assert torch.equal(data, torch.full((2, 3), 35.0))
        # the session leaves the server's table when its forward() has returned
        deadline = time.monotonic() + 5
        while ps.open_sessions() and time.monotonic() < deadline:
            time.sleep(0.01)
        assert ps.open_sessions() == 0
    finally:
        ps.shutdown()


def _mesh_worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    manager = Mock(spec=Manager)
    manager._pg = ProcessGroupGloo()
    manager.num_participants.return_value = 0
    mesh = ft_init_device_mesh(
        device_type="cpu",
        mesh_shape=(2, world),
        mesh_dim_names=("dp_replicate", "dp_shard"),
        replicate_dim=0,
        manager=manager,
    )
    assert mesh.ndim == 2
    assert mesh.mesh_dim_names == ("dp_replicate", "dp_shard")
    replicate_group = mesh.get_group("dp_replicate")
    assert mesh["dp_replicate"].get_group() is replicate_group
    assert mesh.get_group(0) is replicate_group
    assert mesh.get_group("dp_shard").size() == world
    assert mesh["dp_shard"].size() == world
    assert mesh.size(1) == world and mesh.get_local_rank("dp_shard") == rank
    assert mesh.get_rank() == rank
    for n, expect in [(0, 1), (1, 1), (2, 2)]:
        manager.num_participants.return_value = n
        assert mesh["dp_replicate"].size() == expect
        assert mesh.size() == expect * world
        flat = mesh._flatten("dp")
        assert flat.size() == expect * world
        assert flat.get_local_rank() == rank  # replicate rank 0 in its size-1 registered group
    manager.num_participants.return_value = 2
    assert mesh.shape == (2, world)
    assert mesh.get_coordinate() == [0, rank]
    assert mesh.get_local_rank("dp_replicate") == 0
    sub = mesh[("dp_replicate", "dp_shard")]
    assert sub.ndim == 2 and sub.replicate_dim == 0
    # meshes travel inside checkpoints
    buf = io.BytesIO()
    torch.save(mesh, buf)
    buf.seek(0)
    loaded = torch.load(buf, weights_only=False)
    assert loaded.mesh_dim_names == mesh.mesh_dim_names and loaded.replicate_pg is mesh.replicate_pg
    dist.destroy_process_group()


def test_managed_device_mesh_four_processes():
    from torch.distributed import TCPStore

    probe = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
    port = probe.port
    del probe
    mp.spawn(_mesh_worker, args=(4, port), nprocs=4, join=True)


def _fsdp_worker(rank, world, port):
    """HSDP from stock FSDP2: shard dimension on a real gloo mesh, replicate dimension managed."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor import DTensor

    manager = Mock(spec=Manager)
    manager._pg = ProcessGroupGloo()
    manager.num_participants.return_value = 1
    manager.errored.return_value = None
    mesh = ft_init_device_mesh(
        device_type="cpu", mesh_shape=(2, world), mesh_dim_names=("dp_replicate", "dp_shard"), replicate_dim=0, manager=manager
    )
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    reference = [p.detach().clone() for p in model.parameters()]
    fully_shard(model, mesh=mesh)
    assert all(isinstance(p, DTensor) for p in model.parameters())
    x = torch.randn(8, 16, generator=torch.Generator().manual_seed(rank))
    model(x).sum().backward()
    # the replicate-dimension reduction went through the manager's process group view
    assert manager.wait_quorum.call_count >= 1
    for p, ref in zip(model.parameters(), reference):
        assert p.grad is not None and isinstance(p.grad, DTensor)
        assert p.grad.to_local().numel() * world >= ref.numel()  # row-sharded over the shard dimension
    dist.destroy_process_group()


def test_fsdp2_over_managed_mesh_two_processes():
    from torch.distributed import TCPStore

    probe = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
    port = probe.port
    del probe
    mp.spawn(_fsdp_worker, args=(2, port), nprocs=2, join=True)
