"""The NCCL process groups on real GPUs: in-process (ProcessGroupNCCL) and in a child process
(ProcessGroupBabyNCCL).  Same scenarios as the reference's torchft/process_group_test.py:145-170
(NCCL, reconfigured), :270-285 (BabyNCCL API surface) and :301-333 (BabyNCCL on two GPUs).

NVLS is switched off for NCCL in every process these tests start: ranks come and go between the
cases, and a rank that leaves while bound to an NVLink multicast object disturbs the other GPUs.
"""

import gc
import os
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta

import pytest
import torch
from torch import nn
from torch.distributed import ReduceOp, TCPStore

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

from test_process_group import check_collectives  # noqa: E402 - the conformance helper of the CPU tests

pytestmark = pytest.mark.gpu


def _store():
    return TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)


def test_nccl_conformance_ddp_and_two_reconfigurations():
    from torchft_b200.process_group import ProcessGroupNCCL

    store = _store()
    pg = ProcessGroupNCCL(timeout=timedelta(seconds=30))
    assert pg.getBackendName() == "torchft-nccl"
    for attempt in range(3):  # configure, then reconfigure twice onto fresh prefixes
        pg.configure(f"127.0.0.1:{store.port}/nccl{attempt}", 0, 1)
        assert pg.size() == 1
        check_collectives(pg, torch.tensor([2], device="cuda"))
        check_collectives(pg, torch.randn(2, 3, device="cuda"))
        if attempt == 0:
            m = torch.nn.parallel.DistributedDataParallel(nn.Linear(3, 4).cuda(), process_group=pg)
            m(torch.rand(2, 3, device="cuda")).sum().backward()
        t = torch.full((8,), 6.0, device="cuda")
        pg.allreduce_scaled(t, 0.5).wait()
        assert torch.allclose(t, torch.full_like(t, 3.0))
        torch.cuda.synchronize()


def test_baby_nccl_api_surface_and_work_bookkeeping():
    from torchft_b200.process_group import ProcessGroupBabyNCCL

    store = _store()
    pg = ProcessGroupBabyNCCL(timeout=timedelta(seconds=60))
    try:
        pg.configure(f"127.0.0.1:{store.port}/baby", 0, 1)
        assert pg.getBackendName() == "torchft-baby-nccl"
        check_collectives(pg, torch.randn((2, 3), device="cuda"))
        torch.cuda.synchronize()
        gc.collect()  # no work handle of the parent is alive any more ...
        assert pg.num_active_work() == 0  # ... so the child dropped its side too
    finally:
        pg.shutdown()


def test_baby_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from torchft_b200.process_group import ProcessGroupBabyNCCL

    store = _store()
    addr = f"127.0.0.1:{store.port}/baby2"
    groups = []

    def run(rank):
        pg = ProcessGroupBabyNCCL(timeout=timedelta(seconds=60))
        groups.append(pg)
        pg.configure(addr, rank, 2)
        assert pg.size() == 2
        torch.cuda.set_device(rank)  # the child must follow the tensor's device, not a default
        t = torch.tensor([rank + 1.0], device="cuda")
        return t, pg.allreduce([t], ReduceOp.SUM)

    try:
        with ThreadPoolExecutor(max_workers=2) as ex:
            fa, fb = ex.submit(run, 0), ex.submit(run, 1)
            (at, aw), (bt, bw) = fa.result(), fb.result()
        aw.wait()
        bw.get_future().wait()
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        assert at.cpu().item() == 3.0 and bt.cpu().item() == 3.0
    finally:
        for pg in groups:
            pg.shutdown()
