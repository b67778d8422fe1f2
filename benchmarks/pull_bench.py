"""Bandwidth of the heal data path alone: one GPU pulls a buffer out of a peer's symmetric heap.

    python benchmarks/pull_bench.py [--max-mib 4096]

Two processes, one per GPU.  Rank 1 owns the source buffer; rank 0 maps rank 1's heap and pulls with the
two engines of ``NVLinkCheckpointTransport`` (``pull_copy_kernel`` on the SMs, ``cudaMemcpyAsync`` on a copy
engine).  CUDA events on the pulling stream, after warm-up; GB/s = bytes / time.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from datetime import timedelta

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def worker(rank: int, port: int, max_mib: int) -> None:
    import torch
    from torch.distributed import TCPStore

    from torchft_b200.parallel.nvlink import SymmetricHeap, _PeerMappings
    from torchft_b200.parallel.nvlink_heal import NVLinkCheckpointTransport

    torch.cuda.set_device(rank)
    store = TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    nbytes = max_mib << 20
    heap = SymmetricHeap.get(nbytes + (64 << 20))
    buf = heap.alloc(nbytes, torch.uint8)
    if rank == 1:
        buf.fill_(7)
        torch.cuda.synchronize()
        store.set("handle", heap.handle)
        store.set("offset", str(heap.offset_of(buf)))
        store.get("done")  # leave only when the reader has unmapped the heap
        return
    transport = NVLinkCheckpointTransport(heap, timeout=timedelta(seconds=60))
    handle = bytes(store.get("handle"))
    src = _PeerMappings.acquire(handle, heap.device) + int(store.get("offset"))
    stream = transport._stream
    size = 16 << 20
    while size <= nbytes:
        row = {"MiB": size >> 20}
        for engine, floor in (("kernel", 1 << 62), ("copy_engine", 0)):
            transport.copy_engine_min_bytes = floor
            dst = buf[:size]
            with torch.cuda.stream(stream):
                for _ in range(3):
                    transport._pull(dst, src, size)
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(stream)
                for _ in range(5):
                    transport._pull(dst, src, size)
                end.record(stream)
            stream.synchronize()
            ms = start.elapsed_time(end) / 5
            row[f"{engine}_ms"] = round(ms, 4)
            row[f"{engine}_GBps"] = round(size / ms / 1e6, 1)
        assert int(buf[size - 1]) == 7
        print(json.dumps(row), flush=True)
        size *= 4
    _PeerMappings.release(handle, heap.device)
    transport.shutdown(wait=False)
    store.set("done", b"1")


def main() -> None:
    import torch.multiprocessing as mp
    from torch.distributed import TCPStore

    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mib", type=int, default=4096)
    args = ap.parse_args()
    store = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
    mp.spawn(worker, args=(store.port, args.max_mib), nprocs=2, join=True)


if __name__ == "__main__":
    main()
