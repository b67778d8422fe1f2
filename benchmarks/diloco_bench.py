"""DiLoCo / LocalSGD on a Llama 1B-shape decoder: outer-step (sync) time and tokens/s.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/diloco_bench.py [--sync-every 100] [--syncs 3] [--arms fused,buckets,reference]

N replica groups of one GPU.  Inner optimizer AdamW (lr 3e-4, wd 0.1, betas .9/.95); outer optimizer
SGD (lr 0.7, momentum 0.9, Nesterov) on bf16 pseudo-gradients.  Arms:

* ``fused``: this repository's ``DiLoCo`` on ``ProcessGroupNVLink``: the outer step is ONE kernel
  (pseudo-gradient + allreduce over peer memory + Nesterov update) plus the pack / unpack copies;
* ``buckets``: this repository's ``DiLoCo`` on ``ProcessGroupNCCL``: pseudo-gradient kernel, bucketed
  NCCL allreduce + divide, Nesterov kernel;
* ``reference``: the reference's ``torchft.local_sgd.DiLoCo`` and ``Manager`` on its ``ProcessGroupNCCL``
  (``torchft/local_sgd.py:177-239``: per-parameter sub, allreduce, divide, restore copy,
  ``torch.optim.SGD.step``, host backup copy), when ``baseline/_ref`` exists.
* ``localsgd``: this repository's ``LocalSGD`` (plain parameter averaging) on ``ProcessGroupNVLink``.

Every arm trains the same model class (this repository's Llama with its kernels) so that the inner
steps cost the same and the sync time is what differs.  Sync time is host wall time around
``sync()`` with a device synchronise on both sides (it contains the quorum and the commit vote),
max over ranks, median over the syncs after the first.
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import sys
import time
from datetime import timedelta

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def bcast(obj, src=0):
    box = [obj]
    dist.broadcast_object_list(box, src=src)
    return box[0]


def run_arm(arm: str, args, rank: int, world: int, heap) -> dict:
    from torch.distributed import TCPStore

    from torchft_b200.models.llama import Llama, LlamaConfig

    device = torch.device("cuda", torch.cuda.current_device())
    cfg = LlamaConfig.llama_1b() if args.model == "llama_1b" else LlamaConfig.tiny()
    seq = cfg.max_seq_len
    model = Llama(cfg, device=device)
    model.init_weights(seed=11)
    inner = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    outer = torch.optim.SGD(model.parameters(), lr=0.7, momentum=0.9, nesterov=True)
    store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    timeout = timedelta(seconds=120)

    if arm == "reference":
        try:
            socket.getaddrinfo(socket.gethostname(), None)
        except OSError:
            socket.gethostname = lambda: "127.0.0.1"  # type: ignore[assignment]
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import torchft
        from torchft.local_sgd import DiLoCo as Algo
        from torchft.torchft import Lighthouse

        pg = torchft.process_group.ProcessGroupNCCL()
        manager_cls = torchft.Manager
    else:
        from torchft_b200 import _control
        from torchft_b200.local_sgd import DiLoCo, LocalSGD
        from torchft_b200.manager import Manager as manager_cls
        from torchft_b200.parallel.nvlink import ProcessGroupNVLink
        from torchft_b200.process_group import ProcessGroupNCCL

        _control.set_log_enabled(False)
        Lighthouse = _control.Lighthouse
        Algo = LocalSGD if arm == "localsgd" else DiLoCo
        pg = ProcessGroupNCCL() if arm == "buckets" else ProcessGroupNVLink(timeout=timedelta(seconds=60), heap=heap, staging_bytes=1 << 30)

    lighthouse = Lighthouse(bind="[::]:0", min_replicas=world, join_timeout_ms=60000, quorum_tick_ms=10) if rank == 0 else None
    lighthouse_addr = bcast(lighthouse.address() if lighthouse else None)
    manager = manager_cls(
        pg=pg, load_state_dict=lambda sd: model.load_state_dict(sd), state_dict=lambda: model.state_dict(),
        min_replica_size=world, use_async_quorum=False, timeout=timeout, quorum_timeout=timeout, rank=0, world_size=1,
        store_addr="127.0.0.1", store_port=store.port, lighthouse_addr=lighthouse_addr, replica_id=f"{arm}_{rank}_",
    )
    if arm == "localsgd":
        algo = Algo(manager, model, inner, sync_every=args.sync_every, backup_device=device)
    elif arm == "reference":
        algo = Algo(manager, model, inner, outer, sync_every=args.sync_every, backup_device=device)
    else:
        algo = Algo(manager, model, inner, outer, sync_every=args.sync_every, backup_device=device)
    single_kernel = bool(getattr(getattr(algo, "_fused", None), "single_kernel", False))

    gen = torch.Generator().manual_seed(rank)
    tokens = torch.randint(cfg.vocab_size, (args.batch, seq), generator=gen).to(device)
    targets = torch.randint(cfg.vocab_size, (args.batch, seq), generator=gen).to(device)

    sync_ms, inner_ms = [], []
    orig_sync = algo.sync

    def timed_sync() -> None:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        orig_sync()
        torch.cuda.synchronize()
        sync_ms.append((time.perf_counter() - t0) * 1e3)

    algo.sync = timed_sync  # type: ignore[method-assign]
    with algo:
        for _ in range(args.syncs):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(args.sync_every):
                inner.zero_grad(set_to_none=True)
                loss = model(tokens, targets)
                loss.backward()
                inner.step()
            torch.cuda.synchronize()
            inner_ms.append((time.perf_counter() - t0) * 1e3 - sync_ms[-1])
    final_loss = float(loss.item())
    checksum = float(sum(p.float().sum() for p in model.parameters()).item())
    t = torch.tensor([statistics.median(sync_ms[1:] or sync_ms), statistics.median(inner_ms[1:] or inner_ms)],
                     device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    committed = manager.current_step()
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    n_params = sum(p.numel() for p in model.parameters())
    per_round_s = (float(t[0]) + float(t[1])) / 1e3
    return {"arm": arm, "replicas": world, "model": args.model, "params": n_params, "sync_every": args.sync_every,
            "sync_ms": round(float(t[0]), 2), "inner_steps_ms": round(float(t[1]), 1),
            "tokens_per_s": round(world * args.batch * seq * args.sync_every / per_round_s, 1),
            "single_kernel": single_kernel, "committed_syncs": committed, "final_loss": round(final_loss, 4),
            "param_checksum": round(checksum, 2)}


def kernel_arm(rank: int, world: int, heap) -> dict:
    """Device time of the one-kernel outer step alone (CUDA events, max over ranks)."""
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.parallel.nvlink import NVLinkCommunicator

    store = PrefixStore("dk", TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), is_master=False,
                                       wait_for_workers=False))
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    comm.configure(store, rank, world, "diloco-kernel")
    n = 1498482688  # parameters of the Llama 1B shape
    local, grad = heap.alloc(n, torch.bfloat16), heap.alloc(n, torch.bfloat16)
    g = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    m = [torch.zeros(n, device="cuda") for _ in range(2)]
    local.normal_(0, 0.02)
    times = []
    for it in range(6):
        dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        comm.diloco_outer_(local, grad, g[it & 1], m[it & 1], g[1 - (it & 1)], m[1 - (it & 1)], inv_n=1.0 / world, lr=0.7,
                           momentum=0.9, nesterov=True, first=(it == 0))
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    comm.check()
    t = torch.tensor([statistics.median(times[2:])], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    link_bytes = 2.0 * n * (world - 1) / world          # per direction: chunk loads in, averaged chunk stores out
    hbm_bytes = n * (2 + 2 + 4 + 2 + 4) + 4.0 * n / world + 2.0 * n  # phase 2; phase 1 own chunk + global; gradient stores landing here
    roof_ms = (link_bytes / 770e9 + hbm_bytes / 6548.5e9) * 1e3  # the phases run one after the other
    return {"arm": "kernel", "replicas": world, "params": n, "kernel_ms": round(ms, 3), "roofline_ms": round(roof_ms, 3),
            "of_roofline": round(roof_ms / ms, 3)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama_1b", choices=["llama_1b", "tiny"])
    ap.add_argument("--sync-every", type=int, default=100)
    ap.add_argument("--syncs", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--arms", default="fused,buckets,reference,localsgd")
    ap.add_argument("--dump-after", type=float, default=0.0, help="dump all thread stacks after this many seconds")
    args = ap.parse_args()
    if args.dump_after > 0:
        import faulthandler

        faulthandler.dump_traceback_later(args.dump_after, exit=False)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("cpu:gloo,cuda:nccl" if "kernel" in args.arms else "gloo", timeout=timedelta(seconds=300))
    from torchft_b200.parallel.nvlink import SymmetricHeap

    heap = SymmetricHeap.get(12 << 30)
    for arm in args.arms.split(","):
        if arm == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "torchft")):
            if rank == 0:
                print(json.dumps({"arm": "reference", "unavailable": "baseline/_ref missing"}), flush=True)
            continue
        res = kernel_arm(rank, world, heap) if arm == "kernel" else run_arm(arm, args, rank, world, heap)
        if rank == 0:
            print(json.dumps(res), flush=True)
        dist.barrier()
        torch.cuda.empty_cache()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
