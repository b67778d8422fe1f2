"""All-gather fused into the GEMM vs. the unfused pair, on the linear layers of Llama-3-8B.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/ag_gemm_bench.py

Per rank: ``Y = X @ W.T`` with ``W [N, K]`` row-sharded over the ranks.  Arms:

* ``fused``: ``NVLinkCommunicator.all_gather_linear`` (one kernel: peer pulls + tcgen05 GEMM);
* ``unfused``: this repository's all-gather kernel followed by its GEMM kernel;
* ``nccl+cublas``: ``dist.all_gather_into_tensor`` followed by ``torch.matmul`` (what FSDP2 does).

Times are CUDA events on the launching stream, max over ranks, inputs rotated through more
than 126 MB so weights do not stay in L2 between iterations.  The roofline per shape is the
slower of FLOPs / measured GEMM peak and remote bytes / 770 GB/s.
"""

from __future__ import annotations

import json
import os
import sys
from datetime import timedelta

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", timeout=timedelta(seconds=120))
    from torch.distributed import PrefixStore, TCPStore

    from torchft_b200.ops.gemm import gemm
    from torchft_b200.parallel.nvlink import NVLinkCommunicator, SymmetricHeap

    store = PrefixStore("agb", TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), is_master=False,
                                        wait_for_workers=False))
    heap = SymmetricHeap.get(3 << 30)
    fused = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    fused.configure(PrefixStore("f", store), rank, world, "agb-f")
    plain = NVLinkCommunicator(heap, timeout=timedelta(seconds=30), max_blocks=64)
    plain.configure(PrefixStore("p", store), rank, world, "agb-p")
    peak = 1.36e15
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak = float(json.load(f).get("bf16_tflops_sustained", 1360.0)) * 1e12
    except Exception:  # noqa: BLE001
        pass

    M = 4096
    shapes = [("wqkv", 6144, 4096), ("wo", 4096, 4096), ("w13", 28672, 4096), ("w2", 4096, 14336)]
    copies = 3  # rotate buffers: 3 x (W + X + Y) exceeds L2 for every shape
    rows = []
    for name, N, K in shapes:
        if N % (256 * world):
            continue
        ws = [heap.alloc(N * K, torch.bfloat16).view(N, K) for _ in range(copies)]
        xs = [torch.randn(M, K, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        ys = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
        for w in ws:
            w.normal_(0, 0.02)
        shard = [w[rank * (N // world):(rank + 1) * (N // world)] for w in ws]
        gathered = [torch.empty(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]

        def run_fused(i):
            fused.all_gather_linear(xs[i], ws[i], out=ys[i], copy_ctas=int(os.environ.get("COPY_CTAS", "16")))

        def run_unfused(i):
            plain.all_gather_(ws[i].view(-1))
            gemm(xs[i], ws[i], ys[i])

        def run_nccl(i):
            dist.all_gather_into_tensor(gathered[i].view(-1), shard[i].reshape(-1))
            torch.matmul(xs[i], gathered[i].t(), out=ys[i])

        def run_gemm_only(i):
            gemm(xs[i], ws[i], ys[i])

        res = {}
        for label, fn in (("gemm_only", run_gemm_only), ("fused", run_fused), ("unfused", run_unfused), ("nccl+cublas", run_nccl)):
            for i in range(4):
                fn(i % copies)
            torch.cuda.synchronize()
            dist.barrier()
            iters = 12
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(iters):
                fn(i % copies)
            stop.record()
            torch.cuda.synchronize()
            t = torch.tensor([start.elapsed_time(stop) / iters], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[label] = t.item()
        fused.check()
        plain.check()
        flops = 2.0 * M * N * K
        remote = N * K * 2 * (world - 1) / world
        roof_ms = max(flops / peak, remote / 770e9) * 1e3
        rows.append({"layer": name, "M": M, "N": N, "K": K, **{k: round(v, 4) for k, v in res.items()},
                     "roofline_ms": round(roof_ms, 4), "fused_of_roofline": round(roof_ms / res["fused"], 3),
                     "fused_tflops": round(flops / res["fused"] / 1e9, 1)})
        del ws, xs, ys, gathered
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
