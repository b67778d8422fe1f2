"""NVLink peer-memory collectives and the torchft-nvlink process group on 2+ GPUs.

Every rank is its own process on its own GPU.  The failure test makes a rank stay away
from a collective (a host-side decision); the survivor's bounded device-side wait runs out
and is reported as an error status -- no GPU is ever faulted or hung.
"""

import os
import sys
from datetime import timedelta

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need_gpus(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _spawn(fn, world, *args):
    from torch.distributed import TCPStore

    store = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, store.port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        r, ok, payload = q.get(timeout=300)
        results[r] = (ok, payload)
    for p in procs:
        p.join(timeout=60)
    for r in range(world):
        ok, payload = results[r]
        assert ok, f"rank {r} failed: {payload}"
    return [results[r][1] for r in range(world)]


def _entry(fn, rank, world, port, q, *args):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    try:
        torch.cuda.set_device(rank)
        out = fn(rank, world, port, *args)
        q.put((rank, True, out))
    except Exception as e:  # noqa: BLE001
        import traceback

        q.put((rank, False, f"{e}\n{traceback.format_exc()}"))


def _collectives(rank, world, port):
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.parallel.nvlink import NVLinkCommunicator, SymmetricHeap

    store = PrefixStore("t1", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False))
    heap = SymmetricHeap.get(256 << 20)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=20))
    comm.configure(store, rank, world, "epoch-a")
    for dtype in (torch.bfloat16, torch.float32):
        for n in (8, 1000 * 8, (1 << 20) + 8 * 3):
            t = heap.alloc(n, dtype)
            vals = [torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1234 + r)) for r in range(world)]
            t.copy_(vals[rank].to(dtype))
            comm.allreduce_(t, 1.0 / world)
            ref = sum(v.to(dtype).float() for v in vals) / world
            err = (t.float() - ref).abs().max().item()
            assert err < (2e-2 if dtype == torch.bfloat16 else 1e-5), (dtype, n, err)
            # non-contributing rank: zeros instead of its data
            t.copy_(vals[rank].to(dtype))
            comm.allreduce_(t, 1.0, contribute=(rank != 0))
            ref = sum(v.to(dtype).float() for r, v in enumerate(vals) if r != 0)
            err = (t.float() - ref).abs().max().item()
            assert err < (4e-2 if dtype == torch.bfloat16 else 1e-5), ("contrib", dtype, n, err)
    # one-shot variant for small buffers (every rank reduces everything; one block)
    small = NVLinkCommunicator(heap, timeout=timedelta(seconds=20), oneshot_max_bytes=128 << 10)
    small.configure(PrefixStore("t1os", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)), rank, world, 0)
    for dtype, n in ((torch.bfloat16, 8), (torch.bfloat16, 65536), (torch.float32, 1000 * 4), (torch.float32, 32768)):
        t = heap.alloc(n, dtype)
        vals = [torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7 + r)) for r in range(world)]
        t.copy_(vals[rank].to(dtype))
        small.allreduce_(t, 1.0 / world)
        ref = sum(v.to(dtype).float() for v in vals) / world
        err = (t.float() - ref).abs().max().item()
        assert err < (2e-2 if dtype == torch.bfloat16 else 1e-5), ("one-shot", dtype, n, err)
        t.copy_(vals[rank].to(dtype))
        small.allreduce_(t, 1.0, contribute=(rank != 0))
        ref = sum(v.to(dtype).float() for r, v in enumerate(vals) if r != 0)
        err = (t.float() - ref).abs().max().item()
        assert err < (4e-2 if dtype == torch.bfloat16 else 1e-5), ("one-shot, muted rank", dtype, n, err)
    small.check()
    # allreduce with the copy engines moving the data: same result as the kernel to rounding
    big = NVLinkCommunicator(heap, timeout=timedelta(seconds=20), copy_engine_min_bytes=1 << 16)
    big.configure(PrefixStore("t1ce", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)), rank, world, 0)
    for dtype, n in ((torch.bfloat16, (1 << 20) + 8 * 3), (torch.float32, 1 << 18)):
        t = heap.alloc(n, dtype)
        vals = [torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(99 + r)) for r in range(world)]
        t.copy_(vals[rank].to(dtype))
        big.allreduce_(t, 1.0 / world)
        ref = sum(v.to(dtype).float() for v in vals) / world
        err = (t.float() - ref).abs().max().item()
        assert err < (2e-2 if dtype == torch.bfloat16 else 1e-5), ("copy engine", dtype, err)
        t.copy_(vals[rank].to(dtype))
        big.allreduce_(t, 1.0, contribute=(rank != 0))
        ref = sum(v.to(dtype).float() for r, v in enumerate(vals) if r != 0)
        err = (t.float() - ref).abs().max().item()
        assert err < (4e-2 if dtype == torch.bfloat16 else 1e-5), ("copy engine, muted rank", dtype, err)
    big.check()
    # reduce-scatter + all-gather == allreduce
    n = world * 4096
    full = heap.alloc(n, torch.bfloat16)
    vals = [torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(77 + r)).to(torch.bfloat16) for r in range(world)]
    full.copy_(vals[rank])
    comm.reduce_scatter_(full, 1.0)
    ref = sum(v.float() for v in vals)
    sl = slice(rank * 4096, (rank + 1) * 4096)
    assert (full[sl].float() - ref[sl]).abs().max().item() < 4e-2
    # copy-engine variant: same summation order, so the same bits
    by_kernel = full[sl].clone()
    comm.barrier()  # everybody has read what it needed before the buffers are refilled
    full.copy_(vals[rank])
    comm.reduce_scatter_(full, 1.0, engine="copy")
    assert torch.equal(full[sl], by_kernel)
    comm.all_gather_(full)
    assert (full.float() - ref).abs().max().item() < 4e-2
    # the same exchange by the copy engines, pulled and pushed
    for engine in ("copy", "copy-push"):
        mine = full[sl].clone()
        full.zero_()
        full[sl] = mine
        comm.all_gather_(full, engine)
        assert (full.float() - ref).abs().max().item() < 4e-2, engine
    b = heap.alloc(1024, torch.float32)
    b.fill_(float(rank + 1))
    comm.broadcast_(b, world - 1)
    assert torch.all(b == float(world)).item()
    comm.barrier()
    comm.check()
    # reconfigure onto a new epoch (same peers) and go again
    store2 = PrefixStore("t2", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False))
    comm.configure(store2, (rank + 1) % world, world, "epoch-b")
    t = heap.alloc(4096, torch.float32)
    t.fill_(1.0)
    comm.allreduce_(t, 1.0)
    assert torch.all(t == float(world)).item()
    comm.check()
    return "ok"


def test_nvlink_collectives_two_gpus():
    _need_gpus(2)
    _spawn(_collectives, 2)


def test_nvlink_collectives_four_gpus():
    _need_gpus(4)
    _spawn(_collectives, 4)


def _process_group(rank, world, port):
    from torch.distributed import ReduceOp

    from torchft_b200.parallel.nvlink import ProcessGroupNVLink

    pg = ProcessGroupNVLink(timeout=timedelta(seconds=20))
    pg.configure(f"127.0.0.1:{port}/pg/1", rank, world)
    assert pg.size() == world and pg.getBackendName() == "torchft-nvlink"
    t = torch.full((1000,), float(rank + 1), device="cuda")  # not in the heap: staged
    w = pg.allreduce([t], ReduceOp.SUM)
    w.get_future().wait()
    assert torch.all(t == sum(range(1, world + 1))).item()
    t = torch.full((4099,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
    w = pg.allreduce_scaled(t, 0.5, contribute=True)
    w.wait()
    torch.cuda.synchronize()
    assert torch.allclose(t.float(), torch.full((4099,), 0.5 * sum(range(1, world + 1)), device="cuda"))
    outs = [[torch.empty(5, device="cuda") for _ in range(world)]]
    pg.allgather(outs, [torch.full((5,), float(rank), device="cuda")]).get_future().wait()
    for r in range(world):
        assert torch.all(outs[0][r] == float(r)).item()
    b = torch.full((7,), float(rank), device="cuda")
    pg.broadcast_one(b, 1).get_future().wait()
    assert torch.all(b == 1.0).item()
    return "ok"


def test_process_group_nvlink():
    _need_gpus(2)
    _spawn(_process_group, 2)


def _peer_absent(rank, world, port):
    """Rank 1 stays away from the second collective; rank 0's device-side wait must run out cleanly."""
    import time

    from torch.distributed import ReduceOp, TCPStore

    from torchft_b200.parallel.nvlink import ProcessGroupNVLink, _PeerMappings

    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    pg = ProcessGroupNVLink(timeout=timedelta(seconds=1))
    pg.configure(f"127.0.0.1:{port}/absent/1", rank, world)
    # the first collective of a membership meets on the host; do it together
    first = torch.ones(1024, device="cuda")
    pg.allreduce([first], ReduceOp.SUM).get_future().wait()
    assert torch.all(first == float(world)).item()
    if rank == 0:
        t = torch.ones(1024, device="cuda")
        t0 = time.time()
        fut = pg.allreduce([t], ReduceOp.SUM).get_future()
        with pytest.raises(TimeoutError, match="device-side wait gave up"):
            fut.wait()
        assert time.time() - t0 < 10
        store.set("rank0_done", b"1")
        # the context is still healthy: reconfigure alone and keep going
        assert _PeerMappings.open_count() == 1
        pg.configure(f"127.0.0.1:{port}/absent/2", 0, 1)
        # the peer that left is unmapped: its GPU memory is not pinned by this process any more
        assert _PeerMappings.open_count() == 0
        t = torch.ones(8, device="cuda")
        pg.allreduce_scaled(t, 0.5).get_future().wait()
        assert torch.all(t == 0.5).item()
    else:
        store.get("rank0_done")  # leave only between steps, nothing in flight
    return "ok"


def test_absent_peer_times_out_without_hanging():
    _need_gpus(2)
    _spawn(_peer_absent, 2)


def _host_gives_up_first(rank, world, port):
    """The manager's (host) timeout is far shorter than the device budget: when it fires, the manager
    aborts the process group and the waiting kernel returns at once with status 3 (aborted)."""
    import time

    from torch.distributed import TCPStore

    from torchft_b200 import _control
    from torchft_b200.manager import Manager
    from torchft_b200.parallel.nvlink import ProcessGroupNVLink

    _control.set_log_enabled(False)
    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    lighthouse = None
    if rank == 0:
        lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=world, join_timeout_ms=20000, quorum_tick_ms=10)
        store.set("lighthouse", lighthouse.address())
    group_store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    pg = ProcessGroupNVLink(timeout=timedelta(seconds=20))  # device-side budget
    state = {"w": torch.zeros(4, device="cuda")}
    manager = Manager(
        pg=pg, load_state_dict=lambda sd: state.update(sd), state_dict=lambda: dict(state), min_replica_size=world,
        timeout=timedelta(seconds=1),  # host-side budget
        quorum_timeout=timedelta(seconds=30), rank=0, world_size=1, store_addr="127.0.0.1",
        store_port=group_store.port, lighthouse_addr=store.get("lighthouse").decode(), replica_id=f"abort_{rank}_",
        hostname="127.0.0.1",
    )
    # step 1 (quorum, first configuration, initial weight sync) gets a generous host budget
    manager._timeout = timedelta(seconds=30)
    for step in (1, 2):
        manager.start_quorum()
        t = torch.ones(1024, device="cuda")
        manager.allreduce(t).wait()
        assert manager.should_commit()
        # step 1 is the initial weight sync: the healing replica counts as a participant but sends zeros
        assert torch.all(t == (0.5 if step == 1 else 1.0)).item(), t[:4]
    # step 3: rank 1 joins the quorum but stays away from the allreduce (a host-side decision)
    manager._timeout = timedelta(seconds=1)
    manager.start_quorum()
    manager.wait_quorum()
    if rank == 0:
        t = torch.ones(1024, device="cuda")
        t0 = time.time()
        manager.allreduce(t).wait()  # never raises; completes when the host timeout fired
        torch.cuda.synchronize()  # the kernel itself is over, too: it saw the abort word
        elapsed = time.time() - t0
        assert isinstance(manager.errored(), Exception)
        assert elapsed < 6.0, f"kernel still waited {elapsed:.1f} s after the host had given up"
        assert pg.communicator.status() == 3, pg.communicator.status()
        assert not manager.should_commit()
        store.set("rank0_done", b"1")
    else:
        store.get("rank0_done")  # nothing of rank 1 is in flight while rank 0's wait is cut short
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    return "ok"


def test_manager_timeout_aborts_the_waiting_kernel():
    _need_gpus(2)
    _spawn(_host_gives_up_first, 2)


def _shard_peer_skips(rank, world, port):
    """One replica group sharded over two GPUs; in step 2 rank 1 stays away from the shard-group
    collectives.  Rank 0's bounded wait runs out, the status word turns that into a failed vote for the
    whole group, every rank renews the shard communicator, and step 3 commits again."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200 import _control
    from torchft_b200.manager import Manager
    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.parallel.hsdp import HSDPEngine
    from torchft_b200.parallel.nvlink import NVLinkCommunicator, NVLinkShardComm, ProcessGroupNVLink, SymmetricHeap

    _control.set_log_enabled(False)
    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    lighthouse = None
    if rank == 0:
        lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=20000, quorum_tick_ms=10)
        store.set("lighthouse", lighthouse.address())
    cfg = LlamaConfig.tiny()
    heap = SymmetricHeap.get(512 << 20)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=1))
    comm.bind(PrefixStore("grp", store), rank, world, "shard")
    shard = NVLinkShardComm(comm)
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=3)
    box = {}
    manager = Manager(
        pg=ProcessGroupNVLink(timeout=timedelta(seconds=10), heap=heap, staging_bytes=16 << 20),
        load_state_dict=lambda sd: box["e"].load_state_dict(sd), state_dict=lambda: box["e"].state_dict(),
        min_replica_size=1, timeout=timedelta(seconds=30), quorum_timeout=timedelta(seconds=30),
        rank=rank, world_size=world, store_addr="127.0.0.1", store_port=port,
        lighthouse_addr=store.get("lighthouse").decode(), replica_id="sharded_", hostname="127.0.0.1",
    )
    engine = HSDPEngine(model, model.units(), manager=manager, shard_comm=shard, lr=1e-3, alloc=heap.alloc)
    box["e"] = engine
    gen = torch.Generator().manual_seed(11 + rank)
    tokens = torch.randint(cfg.vocab_size, (1, 256), generator=gen).cuda()
    targets = torch.randint(cfg.vocab_size, (1, 256), generator=gen).cuda()

    engine.train_step(tokens, targets)
    assert manager.current_step() == 1
    engine.wait_optimizer()
    before = engine.flat_param.clone()
    real_rs, real_ag = shard.reduce_scatter_, shard.all_gather_
    if rank == 1:
        shard.reduce_scatter_ = lambda full, n: None  # stays away, on the host
        shard.all_gather_ = lambda full, n: None
    engine.train_step(tokens, targets)
    shard.reduce_scatter_, shard.all_gather_ = real_rs, real_ag
    assert manager.current_step() == 1, "a step with partial gradients must not commit"
    assert comm._generation == 1 and comm.status() == 0
    # the optimizer did not run: the owned parameter slices are what they were
    own = slice(0, 0)
    for u in engine.units:
        n = u.numel // world
        own = slice(u.offset + rank * n, u.offset + (rank + 1) * n)
        assert torch.equal(engine.flat_param[own], before[own])
    loss = engine.train_step(tokens, targets)
    assert manager.current_step() == 2
    assert torch.isfinite(loss).item()
    store.set(f"done/{rank}", b"1")
    for r in range(world):
        store.get(f"done/{r}")
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    return "ok"


def test_shard_peer_missing_fails_the_vote_and_the_group_recovers():
    _need_gpus(2)
    _spawn(_shard_peer_skips, 2)


def _ddp_buckets_in_heap(rank, world, port):
    """torch's DDP reducer allocates its gradient buckets by itself; built under the heap's memory pool they
    are heap tensors, so the NVLink group reduces them in place (no staging copies), and the averaged
    gradients match a single process that sees both batches."""
    from torch import nn
    from torch.distributed import TCPStore

    from torchft_b200 import _control
    from torchft_b200.ddp import DistributedDataParallel
    from torchft_b200.manager import Manager
    from torchft_b200.optim import OptimizerWrapper
    from torchft_b200.parallel.nvlink import ProcessGroupNVLink, SymmetricHeap

    _control.set_log_enabled(False)
    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    lighthouse = None
    if rank == 0:
        lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=world, join_timeout_ms=20000, quorum_tick_ms=10)
        store.set("lighthouse", lighthouse.address())
    group_store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    heap = SymmetricHeap.get(512 << 20)
    pg = ProcessGroupNVLink(timeout=timedelta(seconds=30), heap=heap, staging_bytes=1 << 20)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 512), nn.Tanh(), nn.Linear(512, 64)).cuda()
    reference = nn.Sequential(nn.Linear(256, 512), nn.Tanh(), nn.Linear(512, 64)).cuda()
    reference.load_state_dict(model.state_dict())
    manager = Manager(
        pg=pg, load_state_dict=lambda sd: model.load_state_dict(sd), state_dict=lambda: model.state_dict(),
        min_replica_size=world, timeout=timedelta(seconds=30), quorum_timeout=timedelta(seconds=30), rank=0, world_size=1,
        store_addr="127.0.0.1", store_port=group_store.port, lighthouse_addr=store.get("lighthouse").decode(),
        replica_id=f"ddp_{rank}_", hostname="127.0.0.1",
    )
    seen = []
    real = pg.allreduce_scaled

    def spy(tensor, scale, contribute=True):
        seen.append(heap.offset_of(tensor) is not None)
        return real(tensor, scale, contribute)

    pg.allreduce_scaled = spy
    with heap.allocating(64 << 20):
        ddp = DistributedDataParallel(manager, model, gradient_as_bucket_view=True, bucket_cap_mb=1)
    optimizer = OptimizerWrapper(manager, torch.optim.SGD(model.parameters(), lr=0.0))
    batches = [torch.randn(8, 256, generator=torch.Generator().manual_seed(40 + r)).cuda() for r in range(world)]
    for step in (1, 2):  # step 1 is the initial weight sync; from step 2 on both replicas count
        optimizer.zero_grad()
        ddp(batches[rank]).pow(2).mean().backward()
        optimizer.step()
        assert manager.errored() is None and manager.current_step() == step
    assert seen and all(seen), f"buckets outside the heap: {seen}"
    sum(reference(b).pow(2).mean() for b in batches).div(world).backward()
    for p, p_ref in zip(model.parameters(), reference.parameters()):
        err = (p.grad - p_ref.grad).abs().max().item() / max(p_ref.grad.abs().max().item(), 1e-12)
        assert err < 1e-5, err
    store.set(f"done/{rank}", b"1")
    for r in range(world):
        store.get(f"done/{r}")
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    return "ok"


def test_ddp_gradient_buckets_live_in_the_heap():
    _need_gpus(2)
    _spawn(_ddp_buckets_in_heap, 2)


def _hsdp_shards(rank, world, port):
    """One replica group sharded over `world` GPUs must match one GPU fed the concatenated batch."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.parallel.hsdp import HSDPEngine
    from torchft_b200.parallel.nvlink import NVLinkCommunicator, NVLinkShardComm, SymmetricHeap

    cfg = LlamaConfig.tiny()
    heap = SymmetricHeap.get(512 << 20)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    comm.configure(PrefixStore("hsdp", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)), rank, world, "hsdp")

    gen = torch.Generator().manual_seed(5)
    tokens = torch.randint(cfg.vocab_size, (world, 256), generator=gen).cuda()
    targets = torch.randint(cfg.vocab_size, (world, 256), generator=gen).cuda()

    ref_model = Llama(cfg, device="cuda")
    ref_model.init_weights(seed=3)
    ref = HSDPEngine(ref_model, ref_model.units(), lr=1e-3)
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=3)
    engine = HSDPEngine(model, model.units(), shard_comm=NVLinkShardComm(comm), lr=1e-3, alloc=heap.alloc)
    assert engine.exp_avg.numel() * world == engine.total
    for _ in range(3):
        ref.train_step(tokens, targets)
        engine.train_step(tokens[rank : rank + 1], targets[rank : rank + 1])
    torch.cuda.synchronize()
    comm.check()
    engine.gather_parameters()  # slices updated by the last step are exchanged at the start of the next one
    torch.cuda.synchronize()
    a, b = engine.flat_param.float(), ref.flat_param.float()
    err = (a - b).abs().max().item()
    assert err < 2e-2, f"sharded and single-GPU parameters differ by {err}"
    return "ok"


def test_hsdp_engine_sharded_matches_single_gpu():
    _need_gpus(2)
    _spawn(_hsdp_shards, 2)


def _replicas_with_manager(rank, world, port):
    """Two replica groups of one GPU: lighthouse quorum, step-0 heal over NVLink, fused allreduce."""
    from torch.distributed import TCPStore

    from torchft_b200 import _control
    from torchft_b200.manager import Manager
    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.parallel.hsdp import HSDPEngine
    from torchft_b200.parallel.nvlink import ProcessGroupNVLink, SymmetricHeap
    from torchft_b200.parallel.nvlink_heal import NVLinkCheckpointTransport

    _control.set_log_enabled(False)
    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    lighthouse = None
    if rank == 0:
        lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=world, join_timeout_ms=20000, quorum_tick_ms=10)
        store.set("lighthouse", lighthouse.address())
    lighthouse_addr = store.get("lighthouse").decode()
    group_store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)

    cfg = LlamaConfig.tiny()
    heap = SymmetricHeap.get(512 << 20)
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=100 + rank)  # replicas start DIFFERENT: the step-0 heal must fix that
    box = {}
    transport = NVLinkCheckpointTransport(heap, timeout=timedelta(seconds=30))
    manager = Manager(
        pg=ProcessGroupNVLink(timeout=timedelta(seconds=30), heap=heap, staging_bytes=16 << 20),
        load_state_dict=lambda sd: box["e"].load_state_dict(sd),
        state_dict=lambda: box["e"].state_dict(),
        min_replica_size=world,
        timeout=timedelta(seconds=30),
        quorum_timeout=timedelta(seconds=30),
        rank=0,
        world_size=1,
        store_addr="127.0.0.1",
        store_port=group_store.port,
        lighthouse_addr=lighthouse_addr,
        replica_id=f"replica_{rank}_",
        hostname="127.0.0.1",
        checkpoint_transport=transport,
    )
    engine = HSDPEngine(model, model.units(), manager=manager, lr=1e-3, alloc=heap.alloc)
    box["e"] = engine
    gen = torch.Generator().manual_seed(50 + rank)
    tokens = torch.randint(cfg.vocab_size, (1, 256), generator=gen).cuda()
    targets = torch.randint(cfg.vocab_size, (1, 256), generator=gen).cuda()
    for _ in range(4):
        engine.train_step(tokens, targets)
    torch.cuda.synchronize()
    assert manager.current_step() == 4, manager.current_step()
    digest = engine.flat_param.float().double().sum().item()
    store.set(f"digest/{rank}", str(digest))
    digests = [float(store.get(f"digest/{r}").decode()) for r in range(world)]
    pulled = transport.bytes_pulled
    store.set(f"done/{rank}", b"1")
    for r in range(world):
        store.get(f"done/{r}")
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    assert all(abs(d - digests[0]) <= 1e-6 * max(1.0, abs(digests[0])) for d in digests), digests
    return pulled


def test_two_replicas_quorum_heal_and_allreduce_on_gpus():
    _need_gpus(2)
    pulled = _spawn(_replicas_with_manager, 2)
    # exactly one of the two replicas healed from the other at step 0, GPU to GPU
    assert sorted(p > 0 for p in pulled) == [False, True]


def _ag_gemm(rank, world, port):
    """All-gather fused into the GEMM against an fp32 reference of the same product."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.parallel.nvlink import NVLinkCommunicator, SymmetricHeap

    store = PrefixStore("agg", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False))
    heap = SymmetricHeap.get(512 << 20)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=20))
    comm.configure(store, rank, world, "epoch-ag")
    for (M, N, K, copy_ctas) in ((256, 256 * world, 128, 2), (1000, 512 * world, 1024, 16), (4096, 1024 * world, 2048, 8)):
        w_all = torch.randn(N, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).to(torch.bfloat16)
        x = torch.randn(M, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9 + rank)).to(torch.bfloat16)
        w = heap.alloc(N * K, torch.bfloat16).view(N, K)
        rows = N // world
        for rep in range(2):  # twice: the second call starts from a gathered buffer that is reset first
            w.fill_(float("nan"))
            w[rank * rows : (rank + 1) * rows].copy_(w_all[rank * rows : (rank + 1) * rows])
            comm.barrier()  # nobody pulls before every rank wrote its rows
            y = comm.all_gather_linear(x, w, copy_ctas=copy_ctas)
            torch.cuda.synchronize()
            comm.check()
            assert torch.equal(w, w_all), "gathered weight differs"
            ref = x.float() @ w_all.float().t()
            err = (y.float() - ref).abs().max().item()
            assert err <= 0.02 * ref.abs().max().item() + 1e-2, (M, N, K, rep, err)
            comm.barrier()  # nobody resets its rows while a peer may still read them
    return "ok"


def test_all_gather_fused_gemm_two_gpus():
    _need_gpus(2)
    _spawn(_ag_gemm, 2)


def test_all_gather_fused_gemm_four_gpus():
    _need_gpus(4)
    _spawn(_ag_gemm, 4)


def _diloco_outer(rank, world, port):
    """One-kernel DiLoCo outer step against the same arithmetic in fp32 PyTorch."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.parallel.nvlink import NVLinkCommunicator, SymmetricHeap

    store = PrefixStore("dil", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False))
    heap = SymmetricHeap.get(256 << 20)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=20))
    comm.configure(store, rank, world, "epoch-diloco")
    lr, mu = 0.7, 0.9
    for dtype, n, tol in ((torch.bfloat16, 8 * 100003, 3e-2), (torch.float32, 4 * 50021, 1e-5)):
        gen = lambda seed: torch.Generator(device="cuda").manual_seed(seed)  # noqa: E731
        glob = torch.randn(n, device="cuda", generator=gen(3)).to(dtype)
        locals_ = [(glob.float() + 0.05 * torch.randn(n, device="cuda", generator=gen(10 + r))).to(dtype) for r in range(world)]
        local, grad = heap.alloc(n, dtype), heap.alloc(n, dtype)
        g_in, g_out = glob.clone(), torch.zeros_like(glob)
        m_in = torch.full((n,), 123.0, device="cuda")  # ignored on the first step
        m_out = torch.zeros(n, device="cuda")
        # step 1: everybody contributes, first use of the momentum
        local.copy_(locals_[rank])
        comm.diloco_outer_(local, grad, g_in, m_in, g_out, m_out, inv_n=1.0 / world, lr=lr, momentum=mu, nesterov=True, first=True)
        torch.cuda.synchronize()
        comm.check()
        g_ref = sum(x.float() for x in locals_) / world - glob.float()
        assert (grad.float() - g_ref).abs().max().item() < tol
        g_used = grad.float()  # the kernel keeps using the rounded average
        b_ref = g_used
        w_ref = glob.float() - lr * (g_used + mu * b_ref)
        assert (m_out - b_ref).abs().max().item() < 1e-6
        assert (g_out.float() - w_ref).abs().max().item() < tol
        assert torch.equal(g_in, glob), "inputs of a step must stay untouched until the commit"
        # step 2: rank 0 takes part without contributing; buffers swapped as after a commit
        locals2 = [(g_out.float() + 0.05 * torch.randn(n, device="cuda", generator=gen(20 + r))).to(dtype) for r in range(world)]
        # every rank needs identical inputs: rebuild them from rank-independent seeds and the shared reference
        w1 = w_ref.to(dtype)
        g_in2, m_in2 = w1.clone(), b_ref.clone()
        g_out2, m_out2 = torch.zeros_like(g_in2), torch.zeros_like(m_in2)
        locals2 = [(w1.float() + 0.05 * torch.randn(n, device="cuda", generator=gen(20 + r))).to(dtype) for r in range(world)]
        local.copy_(locals2[rank])
        contributors = [r for r in range(world) if r != 0]
        comm.diloco_outer_(local, grad, g_in2, m_in2, g_out2, m_out2, inv_n=1.0 / len(contributors), lr=lr, momentum=mu,
                           nesterov=True, first=False, contribute=(rank != 0))
        torch.cuda.synchronize()
        comm.check()
        g_ref2 = sum(locals2[r].float() for r in contributors) / len(contributors) - w1.float()
        assert (grad.float() - g_ref2).abs().max().item() < tol
        g_used2 = grad.float()
        b2 = mu * m_in2 + g_used2
        w2 = w1.float() - lr * (g_used2 + mu * b2)
        assert (m_out2 - b2).abs().max().item() < 1e-5
        assert (g_out2.float() - w2).abs().max().item() < tol
        comm.barrier()
    return "ok"


def test_diloco_outer_step_single_kernel_two_gpus():
    _need_gpus(2)
    _spawn(_diloco_outer, 2)


def _gemm_rs(rank, world, port):
    """Weight-gradient GEMM fused with the reduce-scatter against the fp32 sum of all ranks' products."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.parallel.nvlink import NVLinkCommunicator, SymmetricHeap

    heap = SymmetricHeap.get(1 << 30)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=20))
    comm.configure(PrefixStore("grs", TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)), rank, world, 0)

    def inputs(tokens, rows, cols, seed):
        out = []
        for r in range(world):
            g = torch.Generator(device="cuda").manual_seed(seed + r)
            out.append((torch.randn(tokens, rows, device="cuda", generator=g).to(torch.bfloat16),
                        torch.randn(tokens, cols, device="cuda", generator=g).mul(0.1).to(torch.bfloat16)))
        return out

    # (tokens, rows of the weight, columns); the first call needs the largest staging area
    for case, (tokens, rows, cols) in enumerate([(1024, 1024 * world, 1024), (512, 256 * world, 512), (200, 128 * world, 256)]):
        assert comm.can_fuse_wgrad(rows, cols)
        everyone = inputs(tokens, rows, cols, 10 * case)
        dy, x = everyone[rank]
        ref = sum(d.float().t() @ xx.float() for d, xx in everyone)
        share = rows // world
        mine = ref[rank * share : (rank + 1) * share]
        out = torch.empty(share, cols, device="cuda", dtype=torch.bfloat16)
        comm.wgrad_reduce_scatter(dy, x, out)
        torch.cuda.synchronize()
        comm.check()
        err = ((out.float() - mine).norm() / mine.norm()).item()
        assert err < 4e-3, f"case {case}: relative error {err}"
        # a second micro-batch accumulates into the shard
        comm.wgrad_reduce_scatter(dy, x, out, accumulate=True)
        torch.cuda.synchronize()
        comm.check()
        err = ((out.float() - 2 * mine).norm() / mine.norm()).item()
        assert err < 8e-3, f"case {case}: relative error after accumulation {err}"
    return "ok"


def test_wgrad_gemm_fused_with_reduce_scatter_two_gpus():
    _need_gpus(2)
    _spawn(_gemm_rs, 2)


def test_wgrad_gemm_fused_with_reduce_scatter_four_gpus():
    _need_gpus(4)
    _spawn(_gemm_rs, 4)


def _hsdp_fused_rs(rank, world, port):
    """Row-sharded projection matrices whose gradients are reduce-scattered inside the weight-gradient
    GEMM: same parameters after three steps as one GPU fed the concatenated batch."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.parallel.hsdp import HSDPEngine
    from torchft_b200.parallel.nvlink import NVLinkCommunicator, NVLinkShardComm, SymmetricHeap

    cfg = LlamaConfig.tiny(dim=512, n_heads=4, n_kv_heads=2, ffn_dim=1024)
    heap = SymmetricHeap.get(1 << 30)
    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    comm.bind(PrefixStore("frs", store), rank, world, "shard")
    rs = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    rs.bind(PrefixStore("frs", store), rank, world, "rs")
    calls = {"n": 0}
    inner = rs.wgrad_reduce_scatter

    def counted(*a, **kw):
        calls["n"] += 1
        return inner(*a, **kw)

    rs.wgrad_reduce_scatter = counted
    gen = torch.Generator().manual_seed(5)
    tokens = torch.randint(cfg.vocab_size, (world, 256), generator=gen).cuda()
    targets = torch.randint(cfg.vocab_size, (world, 256), generator=gen).cuda()
    ref_model = Llama(cfg, device="cuda")
    ref_model.init_weights(seed=3)
    ref = HSDPEngine(ref_model, ref_model.units(), lr=1e-3)
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=3)
    engine = HSDPEngine(model, model.units(per_weight=True), shard_comm=NVLinkShardComm(comm, gather_engine="copy"),
                        lr=1e-3, alloc=heap.alloc, fused_rs_comm=rs)
    assert sum(u.fused_rs for u in engine.units) == 4 * cfg.n_layers
    steps = 3
    for _ in range(steps):
        ref.train_step(tokens, targets)
        engine.train_step(tokens[rank : rank + 1], targets[rank : rank + 1])
    torch.cuda.synchronize()
    comm.check()
    rs.check()
    assert calls["n"] == steps * 4 * cfg.n_layers, calls
    engine.gather_parameters()
    torch.cuda.synchronize()
    for (name, p), (_, q) in zip(model.named_parameters(), ref_model.named_parameters()):
        err = (p.float() - q.float()).abs().max().item()
        assert err < 2e-2, f"{name}: sharded and single-GPU parameters differ by {err}"
    return "ok"


def test_hsdp_engine_fused_reduce_scatter_matches_single_gpu():
    _need_gpus(2)
    _spawn(_hsdp_fused_rs, 2)


def test_hsdp_engine_fused_reduce_scatter_four_gpus():
    _need_gpus(4)
    _spawn(_hsdp_fused_rs, 4)


def _hsdp_fused_gather(rank, world, port):
    """Row-sharded projection matrices gathered inside their first GEMM of the step: same result
    as one GPU fed the concatenated batch."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.parallel.hsdp import HSDPEngine
    from torchft_b200.parallel.nvlink import NVLinkCommunicator, NVLinkShardComm, SymmetricHeap

    cfg = LlamaConfig.tiny(dim=512, n_heads=4, n_kv_heads=2, ffn_dim=1024)
    heap = SymmetricHeap.get(1 << 30)
    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    comm.configure(PrefixStore("fg-shard", store), rank, world, "fg-shard")
    fused = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    fused.configure(PrefixStore("fg-fused", store), rank, world, "fg-fused")
    calls = {"n": 0}
    inner = fused.all_gather_linear

    def counted(*a, **kw):
        calls["n"] += 1
        return inner(*a, **kw)

    fused.all_gather_linear = counted

    gen = torch.Generator().manual_seed(5)
    tokens = torch.randint(cfg.vocab_size, (world, 256), generator=gen).cuda()
    targets = torch.randint(cfg.vocab_size, (world, 256), generator=gen).cuda()
    ref_model = Llama(cfg, device="cuda")
    ref_model.init_weights(seed=3)
    ref = HSDPEngine(ref_model, ref_model.units(), lr=1e-3)
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=3)
    engine = HSDPEngine(model, model.units(per_weight=True), shard_comm=NVLinkShardComm(comm), lr=1e-3, alloc=heap.alloc,
                        fused_gather_comm=fused)
    assert len(engine._fused_units) == 4 * cfg.n_layers
    steps = 3
    for _ in range(steps):
        ref.train_step(tokens, targets)
        engine.train_step(tokens[rank : rank + 1], targets[rank : rank + 1])
    torch.cuda.synchronize()
    comm.check()
    fused.check()
    assert calls["n"] == steps * 4 * cfg.n_layers, calls
    engine.gather_parameters()
    torch.cuda.synchronize()
    for (name, p), (_, q) in zip(model.named_parameters(), ref_model.named_parameters()):
        err = (p.float() - q.float()).abs().max().item()
        assert err < 2e-2, f"{name}: sharded and single-GPU parameters differ by {err}"
    return "ok"


def test_hsdp_engine_fused_gather_matches_single_gpu():
    _need_gpus(2)
    _spawn(_hsdp_fused_gather, 2)
