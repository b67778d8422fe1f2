"""Cross-replica gradient allreduce microbenchmark: fused NVLink kernel vs NCCL + divide.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29520 benchmarks/allreduce_bench.py [--max-mib 1024]

For flat buffers from 1 KiB to --max-mib MiB (powers of four), bf16 and fp32, every rank
averages its buffer with the others:

* ``nvlink``: one launch of the fused peer-memory kernel (sum + 1/n scaling in the same pass)
  on a buffer in the symmetric heap -- what ``Manager.allreduce`` runs on ``ProcessGroupNVLink``;
* ``nccl``: ``all_reduce(SUM)`` followed by the separate ``div_`` kernel -- what the reference's
  ``Manager.allreduce`` runs on ``ProcessGroupNCCL`` (``torchft/manager.py:274,287``).

Times are CUDA-event times per call (max over ranks), after warm-up.  Bus bandwidth uses the
usual 2(n-1)/n factor.  Rank 0 prints one JSON line per (dtype, size).
"""

import argparse
import json
import os
import sys
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mib", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()

    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.parallel.nvlink import NVLinkCommunicator, SymmetricHeap

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    store = TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), is_master=False, wait_for_workers=False)
    heap = SymmetricHeap.get((args.max_mib << 20) + (64 << 20))
    comm = NVLinkCommunicator(heap, timeout=timedelta(seconds=30), max_blocks=int(os.environ.get("TFT_BLOCKS", 64)))
    comm.configure(PrefixStore("arbench", store), rank, world, "arbench")
    buf = heap.alloc(args.max_mib << 20, torch.uint8)
    ref = torch.empty(args.max_mib << 20, dtype=torch.uint8, device="cuda")

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / args.iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for dtype in (torch.bfloat16, torch.float32):
        nbytes = 1024
        while nbytes <= (args.max_mib << 20):
            a = buf[:nbytes].view(dtype)
            b = ref[:nbytes].view(dtype)
            a.normal_()
            b.copy_(a)
            ours = timed(lambda: comm.allreduce_(a, 1.0 / world))
            nccl = timed(lambda: (dist.all_reduce(b), b.div_(world)))
            comm.check()
            if rank == 0:
                bus = 2 * (world - 1) / world * nbytes
                print(json.dumps({
                    "dtype": str(dtype).replace("torch.", ""), "bytes": nbytes, "ranks": world,
                    "nvlink_fused_us": round(ours * 1e3, 2), "nccl_plus_div_us": round(nccl * 1e3, 2),
                    "nvlink_busbw_GBs": round(bus / ours / 1e6, 1), "nccl_busbw_GBs": round(bus / nccl / 1e6, 1),
                    "speedup": round(nccl / ours, 2),
                }), flush=True)
            nbytes *= 4
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
