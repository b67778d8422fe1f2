"""Weight-gradient GEMM fused with the reduce-scatter vs. the unfused pairs, on the projections of
Llama-3-8B at 4096 tokens per rank.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 benchmarks/gemm_rs_bench.py

Per rank: ``dW = dY.T @ X`` (``dY [tokens, rows]``, ``X [tokens, cols]``), summed over the ranks, rank r
keeping rows ``[r * rows / world, (r + 1) * rows / world)``.  Arms:

* ``fused``: ``NVLinkCommunicator.wgrad_reduce_scatter`` (one kernel: tcgen05 GEMM whose epilogue sends
  each tile to its owner, ``csrc/kernels/gemm_rs.cu``);
* ``unfused``: this repository's GEMM into a full-size gradient buffer followed by its reduce-scatter
  kernel (what ``HSDPEngine`` does without ``fused_rs_comm``);
* ``nccl+cublas``: ``torch.matmul`` followed by ``dist.reduce_scatter_tensor`` (what FSDP2 does; NCCL
  with whatever ``NCCL_NVLS_ENABLE`` says);
* ``gemm_only``: the local product alone, for scale.

Times are CUDA events on the launching stream, max over ranks; operands rotate through three copies so
that nothing is served from L2.  The roofline per shape is the slower of FLOPs / measured sustained GEMM
rate and bytes that must leave this GPU, ``(world - 1) / world * rows * cols * 2``, over 770 GB/s.
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

    store = PrefixStore("grsb", TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), is_master=False,
                                         wait_for_workers=False))
    heap = SymmetricHeap.get(3 << 30)
    fused = NVLinkCommunicator(heap, timeout=timedelta(seconds=30))
    fused.configure(PrefixStore("f", store), rank, world, 0)
    plain = NVLinkCommunicator(heap, timeout=timedelta(seconds=30), max_blocks=64)
    plain.configure(PrefixStore("p", store), rank, world, 0)
    peak = 1.36e15
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak = float(json.load(f).get("bf16_tflops_sustained", 1360.0)) * 1e12
    except Exception:  # noqa: BLE001
        pass

    tokens = 4096
    shapes = [("w13", 28672, 4096), ("wqkv", 6144, 4096), ("wo", 4096, 4096), ("w2", 4096, 14336)]  # largest first
    copies = 3
    fused.reserve_wgrad_staging(28672, 4096)
    full_heap = heap.alloc(28672 * 4096, torch.bfloat16)  # unfused arm: the gradient buffer peers read from
    rows_out = []
    for name, rows, cols in shapes:
        if not fused.can_fuse_wgrad(rows, cols):
            continue
        dys = [torch.randn(tokens, rows, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        xs = [torch.randn(tokens, cols, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        share = rows // world
        shard = torch.empty(share, cols, device="cuda", dtype=torch.bfloat16)
        full = full_heap[: rows * cols].view(rows, cols)
        full_local = torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16)

        def run_fused(i):
            fused.wgrad_reduce_scatter(dys[i], xs[i], shard)

        def run_unfused(i):
            gemm(dys[i], xs[i], full, a_kmajor=False, b_kmajor=False)
            plain.reduce_scatter_(full.view(-1), 1.0)

        def run_nccl(i):
            torch.matmul(dys[i].t(), xs[i], out=full_local)
            dist.reduce_scatter_tensor(shard.view(-1), full_local.view(-1))

        def run_gemm_only(i):
            gemm(dys[i], xs[i], full_local, a_kmajor=False, b_kmajor=False)

        res = {}
        for label, fn in (("gemm_only", run_gemm_only), ("fused", run_fused), ("unfused", run_unfused),
                          ("nccl+cublas", run_nccl)):
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
        flops = 2.0 * tokens * rows * cols
        remote = rows * cols * 2 * (world - 1) / world
        roof_ms = max(flops / peak, remote / 770e9) * 1e3
        rows_out.append({"layer": name, "rows": rows, "cols": cols, "tokens": tokens, "ranks": world,
                         **{k + "_ms": round(v, 4) for k, v in res.items()},
                         "bytes_over_link_MB": round(remote / 1e6, 1), "link_ms_at_770GBs": round(remote / 770e9 * 1e3, 4),
                         "roofline_ms": round(roof_ms, 4), "fused_of_roofline": round(roof_ms / res["fused"], 3),
                         "fused_vs_unfused": round(res["unfused"] / res["fused"], 3),
                         "fused_vs_nccl_cublas": round(res["nccl+cublas"] / res["fused"], 3)})
        del dys, xs, shard, full_local
    if rank == 0:
        for r in rows_out:
            print(json.dumps(r))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
