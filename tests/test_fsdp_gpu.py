"""HSDP composed from stock FSDP2 and the managed replicate dimension, on four GPUs.

Two replica groups of two GPUs.  Inside a group ``fully_shard`` shards over an ordinary NCCL mesh
dimension; across the groups the gradient all-reduce goes through ``ManagedProcessGroup`` ->
``Manager`` -> ``ProcessGroupNVLink`` (the fused peer-memory kernel).  One optimizer step runs
through the fault-tolerant wrapper and the resulting gradients are compared with a single-process
fp32 computation over all four batches.  Same scenario as the reference's torchft/fsdp_test.py:38-74,
which uses a mocked manager; here the manager, the lighthouse and the collectives are real.
"""

import os
import sys
from datetime import timedelta

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    try:
        import torch.distributed as dist
        from torch import nn
        from torch.distributed import TCPStore
        from torch.distributed.fsdp import fully_shard

        from torchft_b200 import _control
        from torchft_b200.device_mesh import ft_init_device_mesh
        from torchft_b200.manager import Manager
        from torchft_b200.optim import OptimizerWrapper
        from torchft_b200.parallel.nvlink import ProcessGroupNVLink

        _control.set_log_enabled(False)
        torch.cuda.set_device(rank)
        group_size = world // 2
        group, group_rank = divmod(rank, group_size)
        rendezvous = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
        lighthouse = None
        if rank == 0:
            lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=2, join_timeout_ms=30000, quorum_tick_ms=10)
            rendezvous.set("lighthouse", lighthouse.address())
        # one store per replica group: torch.distributed inside the group and the manager both use it
        if group_rank == 0:
            group_store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
            rendezvous.set(f"group_port/{group}", str(group_store.port))
        group_port = int(rendezvous.get(f"group_port/{group}").decode())
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(group_port), RANK=str(group_rank),
                          WORLD_SIZE=str(group_size))
        dist.init_process_group(
            "nccl", store=dist.PrefixStore("c10d", TCPStore("127.0.0.1", group_port, is_master=False, wait_for_workers=False)),
            rank=group_rank, world_size=group_size)  # no device_id: groups created later (the managed
        # replicate dimension) would inherit it, and c10d then asks the group for a native CUDA backend

        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(128, 256, bias=False), nn.Tanh(), nn.Linear(256, 64, bias=False)).cuda()
        reference = nn.Sequential(nn.Linear(128, 256, bias=False), nn.Tanh(), nn.Linear(256, 64, bias=False)).cuda()
        reference.load_state_dict(model.state_dict())

        manager = Manager(
            pg=ProcessGroupNVLink(timeout=timedelta(seconds=30)),
            load_state_dict=lambda sd: None, state_dict=lambda: {},  # same seed everywhere: nothing to transfer
            min_replica_size=2, timeout=timedelta(seconds=60), quorum_timeout=timedelta(seconds=60),
            rank=group_rank, world_size=group_size, store_addr="127.0.0.1", store_port=group_port,
            lighthouse_addr=rendezvous.get("lighthouse").decode(), replica_id=f"fsdp_{group}_", hostname="127.0.0.1",
        )
        mesh = ft_init_device_mesh(device_type="cuda", mesh_shape=(2, group_size),
                                   mesh_dim_names=("dp_replicate", "dp_shard"), replicate_dim=0, manager=manager)
        fully_shard(model, mesh=mesh)
        # lr 0: the steps commit but leave the weights alone, so step 2 can be checked against them
        optimizer = OptimizerWrapper(manager, torch.optim.SGD(model.parameters(), lr=0.0))

        batches = [torch.randn(4, 128, generator=torch.Generator().manual_seed(100 + r)).cuda() for r in range(world)]
        # Step 1 is the initial weight sync: the second replica group heals and only the first one's
        # gradients count.  From step 2 on both groups participate.
        for step in (1, 2):
            optimizer.zero_grad()  # starts the quorum
            model(batches[rank]).pow(2).mean().backward()
            grads = [p.grad.to_local().clone() for p in model.parameters()]
            optimizer.step()  # should_commit, then the wrapped step
            torch.cuda.synchronize()
            assert manager.errored() is None, f"step {step}: {manager.errored()!r}"
            assert manager.current_step() == step, (manager.current_step(), step)
        assert manager.num_participants() == 2

        # the same gradient, computed here from all four batches without any sharding
        sum(reference(b).pow(2).mean() for b in batches).div(world).backward()
        for g, p_ref in zip(grads, reference.parameters()):
            rows = p_ref.grad.shape[0] // group_size
            want = p_ref.grad[group_rank * rows : (group_rank + 1) * rows]
            err = (g - want).abs().max().item() / max(want.abs().max().item(), 1e-12)
            assert err < 1e-4, f"sharded gradient differs from the unsharded one by {err}"
        rendezvous.set(f"done/{rank}", b"1")
        for r in range(world):
            rendezvous.get(f"done/{r}")
        manager.shutdown(wait=False)
        if lighthouse is not None:
            lighthouse.shutdown()
        dist.destroy_process_group()
        q.put((rank, True, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback

        q.put((rank, False, f"{e}\n{traceback.format_exc()}"))


def test_fully_shard_over_managed_mesh_with_nvlink_replicate_dimension():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    from torch.distributed import TCPStore

    store = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 4, store.port, q)) for r in range(4)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, ok, payload in sorted(results):
        assert ok, f"rank {rank} failed: {payload}"
