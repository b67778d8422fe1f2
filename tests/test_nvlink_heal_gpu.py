"""NVLink checkpoint transport: manifest + peer-memory pull, gate and lease semantics."""

import time
import urllib.error
from datetime import timedelta

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_loopback_pull_gate_and_lease():
    from torchft_b200.parallel.nvlink import SymmetricHeap
    from torchft_b200.parallel.nvlink_heal import NVLinkCheckpointTransport

    heap = SymmetricHeap.get(256 << 20)
    src_a = heap.alloc(1 << 20, torch.bfloat16)
    src_b = heap.alloc(12345, torch.float32)
    src_a.copy_(torch.randn(1 << 20, device="cuda").to(torch.bfloat16))
    src_b.copy_(torch.randn(12345, device="cuda"))
    outside = torch.arange(10, device="cuda")  # not in the heap: travels inside the manifest
    state = {"user": {"a": src_a.view(1024, 1024), "b": [src_b], "outside": outside, "lr": 0.1}, "torchft": {"step": 7, "batches_committed": 14}}

    t = NVLinkCheckpointTransport(heap, timeout=timedelta(seconds=10))
    try:
        # gate closed: a request waits (and here runs into its own short timeout)
        with pytest.raises((TimeoutError, urllib.error.URLError, OSError)):
            t.recv_checkpoint(0, t.metadata(), 7, timedelta(seconds=0.3))

        t.send_checkpoint([1], 7, state, timedelta(seconds=10))
        with pytest.raises(urllib.error.HTTPError):
            t.recv_checkpoint(0, t.metadata(), 6, timedelta(seconds=5))  # wrong step -> 400

        out = t.recv_checkpoint(0, t.metadata(), 7, timedelta(seconds=10))
        assert torch.equal(out["user"]["a"], src_a.view(1024, 1024)) and out["user"]["a"].data_ptr() != src_a.data_ptr()
        assert torch.equal(out["user"]["b"][0], src_b)
        assert torch.equal(out["user"]["outside"].cuda(), outside) and out["user"]["lr"] == 0.1
        assert out["torchft"] == {"step": 7, "batches_committed": 14}

        # in-place receive into live tensors
        dst_a = torch.zeros(1024, 1024, device="cuda", dtype=torch.bfloat16)
        dst_b = torch.zeros(12345, device="cuda")
        t.set_receive_targets(lambda: {"user": {"a": dst_a, "b": [dst_b], "outside": None, "lr": 0.0}, "torchft": {}})
        out = t.recv_checkpoint(0, t.metadata(), 7, timedelta(seconds=10))
        assert out["user"]["a"].data_ptr() == dst_a.data_ptr() and torch.equal(dst_a, src_a.view(1024, 1024))
        assert torch.equal(dst_b, src_b)

        # the gate closes only after the lease of a running copy is returned
        t.disallow_checkpoint()
        with pytest.raises((TimeoutError, urllib.error.URLError, OSError)):
            t.recv_checkpoint(0, t.metadata(), 7, timedelta(seconds=0.3))
    finally:
        t.shutdown()


def test_http_checkpoint_is_ordered_after_kernels_still_queued():
    """The HTTP transport copies on a stream of its own; the copy must still see the values that
    kernels queued BEFORE send_checkpoint produce (here: a long spin followed by a fill)."""
    from torchft_b200.checkpointing import CheckpointServer

    param = torch.zeros(1 << 20, device="cuda")
    server = CheckpointServer(timeout=timedelta(seconds=30))
    try:
        torch.cuda._sleep(2_000_000_000)  # about a second of GPU time ahead of the write
        param.fill_(7.0)
        server.send_checkpoint([1], 3, {"user": {"p": param}, "torchft": {"step": 3, "batches_committed": 3}},
                               timedelta(seconds=30))
        got = server.recv_checkpoint(0, server.metadata(), 3, timedelta(seconds=30))
        server.disallow_checkpoint()
        assert got["user"]["p"].device.type == "cpu"
        assert bool((got["user"]["p"] == 7.0).all())
    finally:
        server.shutdown(wait=False)
