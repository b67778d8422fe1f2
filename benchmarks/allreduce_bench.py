"""Cross-replica gradient allreduce microbenchmark: fused NVLink kernel vs NCCL + divide.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29520 benchmarks/allreduce_bench.py [--max-mib 1024] [--abort-part]

For flat buffers from 1 KiB to --max-mib MiB in powers of two, bf16 and fp32, every rank averages
its buffer with the others:

* ``nvlink``: one launch of the fused peer-memory kernel (sum + 1/n scaling in the same pass)
  on a buffer in the symmetric heap -- what ``Manager.allreduce`` runs on ``ProcessGroupNVLink``;
  up to 128 KiB also ``nvlink_oneshot``, the one-block one-shot variant (every rank reduces the whole
  buffer), which is what the dispatch threshold ``oneshot_max_bytes`` is chosen from;
* ``nccl``: ``all_reduce(SUM)`` followed by the separate ``div_`` kernel -- what the reference's
  ``Manager.allreduce`` runs on ``ProcessGroupNCCL`` (``torchft/manager.py:274,287``).  NCCL runs
  with whatever ``NCCL_NVLS_ENABLE`` says; the JSON lines record it (unset = NCCL's default, which
  uses in-switch reduction where the fabric offers it).  NCCL reads the variable once per process,
  so the two NCCL rows of a table come from two runs.

Times are CUDA-event times per call (max over ranks) after warm-up.  Bus bandwidth uses the usual
2(n-1)/n factor.  Rank 0 prints one JSON line per (dtype, size).

``--abort-part`` adds the failure drill of the sweep (run it with ``NCCL_NVLS_ENABLE=0``): at 16 MiB the
last rank stays away from one collective -- a decision of its host code, nothing on a GPU is faulted --
the other ranks' bounded device-side wait runs out after ``--abort-timeout`` seconds and sets the status
word, everyone reconfigures onto a fresh store prefix and runs the next allreduce.  Reported: the time
from launching the doomed collective to reading the status, and from the status to the first
completed collective of the new membership.
"""

import argparse
import json
import os
import sys
import time
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mib", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--abort-part", action="store_true")
    ap.add_argument("--abort-timeout", type=float, default=1.0)
    ap.add_argument("--skip-nccl", action="store_true")
    args = ap.parse_args()

    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.parallel.nvlink import NVLinkCommunicator, SymmetricHeap

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    store = TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), is_master=False, wait_for_workers=False)
    heap = SymmetricHeap.get((args.max_mib << 20) + (64 << 20))
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=30), max_blocks=int(os.environ.get("TFT_BLOCKS", 64)))
    comm.configure(PrefixStore("arbench", store), rank, world, 0)
    oneshot = NVLinkCommunicator(heap, timeout=timedelta(seconds=30), oneshot_max_bytes=128 << 10)
    oneshot.configure(PrefixStore("arbench1", store), rank, world, 0)
    buf = heap.alloc(args.max_mib << 20, torch.uint8)
    ref = torch.empty(args.max_mib << 20, dtype=torch.uint8, device="cuda")
    nvls = os.environ.get("NCCL_NVLS_ENABLE", "default")

    def timed(fn, nbytes):
        iters = args.iters * (4 if nbytes <= (1 << 20) else 1)
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Both paths once before anything is timed: the first NCCL call builds its communicator and the
    # first launch of each kernel loads its code, neither of which belongs to the first row.
    warm_a, warm_b = buf[: 1 << 20].view(torch.float32), ref[: 1 << 20].view(torch.float32)
    warm_a.zero_()
    warm_b.zero_()
    for _ in range(3):
        comm.allreduce_(warm_a, 1.0 / world)
        if not args.skip_nccl:
            dist.all_reduce(warm_b)
            warm_b.div_(world)
    torch.cuda.synchronize()
    tiny_a, tiny_b = buf[:1024].view(torch.bfloat16), ref[:1024].view(torch.bfloat16)
    timed(lambda: comm.allreduce_(tiny_a, 1.0 / world), 1024)  # discarded: clocks and caches settle here
    if not args.skip_nccl:
        timed(lambda: (dist.all_reduce(tiny_b), tiny_b.div_(world)), 1024)

    for dtype in (torch.bfloat16, torch.float32):
        nbytes = 1024
        while nbytes <= (args.max_mib << 20):
            a = buf[:nbytes].view(dtype)
            b = ref[:nbytes].view(dtype)
            a.normal_()
            b.copy_(a)
            ours = timed(lambda: comm.allreduce_(a, 1.0 / world), nbytes)
            one = timed(lambda: oneshot.allreduce_(a, 1.0 / world), nbytes) if nbytes <= (128 << 10) else None
            nccl = None if args.skip_nccl else timed(lambda: (dist.all_reduce(b), b.div_(world)), nbytes)
            comm.check()
            if rank == 0:
                bus = 2 * (world - 1) / world * nbytes
                row = {"dtype": str(dtype).replace("torch.", ""), "bytes": nbytes, "ranks": world,
                       "nvlink_fused_us": round(ours * 1e3, 2), "nvlink_busbw_GBs": round(bus / ours / 1e6, 1),
                       "nccl_nvls": nvls}
                if one is not None:
                    row["nvlink_oneshot_us"] = round(one * 1e3, 2)
                if nccl is not None:
                    row.update({"nccl_plus_div_us": round(nccl * 1e3, 2), "nccl_busbw_GBs": round(bus / nccl / 1e6, 1),
                                "speedup": round(nccl / ours, 2)})
                print(json.dumps(row), flush=True)
            nbytes *= 2

    if args.abort_part:
        drill = NVLinkCommunicator(heap, timeout=timedelta(seconds=args.abort_timeout))
        drill.configure(PrefixStore("drill/0", store), rank, world, 0)
        t = buf[: 16 << 20].view(torch.float32)
        t.fill_(1.0)
        drill.allreduce_(t, 1.0 / world)  # a good one first
        torch.cuda.synchronize()
        dist.barrier()
        absent = rank == world - 1
        t0 = time.perf_counter()
        if not absent:
            drill.allreduce_(t, 1.0 / world)
        torch.cuda.synchronize()
        status = drill.status()
        t_status = time.perf_counter()
        assert absent or status != 0, "the wait should have run out"
        # every member, the absentee included, moves to the next membership and goes again
        drill.configure(PrefixStore("drill/1", store), rank, world, 1)
        t.fill_(1.0)
        drill.allreduce_(t, 1.0 / world)
        torch.cuda.synchronize()
        t_good = time.perf_counter()
        ok = drill.status() == 0 and bool((t == 1.0).all().item())
        # rank 0 is one of the ranks that waited; the absentee's own clock only shows how long it sat in
        # the store waiting for the others to give up
        times = torch.tensor([t_status - t0, t_good - t_status], device="cuda", dtype=torch.float64)
        dist.broadcast(times, src=0)
        flags = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if rank == 0:
            print(json.dumps({
                "abort_drill": {"ranks": world, "absent_rank": world - 1, "device_budget_s": args.abort_timeout,
                                "status_on_waiting_ranks": status,
                                "launch_to_status_s": round(float(times[0]), 3),
                                "status_to_first_good_collective_s": round(float(times[1]), 3),
                                "recovered": bool(flags.item())}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
