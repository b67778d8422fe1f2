"""Fault-tolerant data parallelism across replica groups.

``DistributedDataParallel`` reuses torch's bucketing reducer but routes every gradient
bucket through ``Manager.allreduce`` (average over the replicas of the current quorum,
errors recorded instead of raised).  ``PureDistributedDataParallel`` is the hook-only
variant without buckets.  Parity: the reference's ``torchft/ddp.py:32-97``.
"""

from typing import TYPE_CHECKING

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import parallel

from torchft_b200.process_group import ProcessGroupDummy

if TYPE_CHECKING:
    from torchft_b200.manager import Manager


class DistributedDataParallel(parallel.DistributedDataParallel):
    """torch DDP whose gradient communication goes through a ``Manager``.

    The module itself is built on a world-size-1 dummy group, so the constructor's
    parameter verification and broadcast do nothing (initial weights are synchronised
    by the step-0 heal).  Bucket layout is frozen (``find_unused_parameters=True`` stops
    the reducer from rebuilding buckets), because a replica that joins later must see
    exactly the same buckets as the ones already training.
    """

    def __init__(self, manager: "Manager", module: nn.Module, **kwargs: object) -> None:
        pg = ProcessGroupDummy(0, 1)
        super().__init__(
            module,
            process_group=pg,
            find_unused_parameters=True,  # keeps the first bucket assignment for good
            **kwargs,  # type: ignore[arg-type]
        )
        self.register_comm_hook(manager, self._comm_hook)

    @staticmethod
    def _comm_hook(state: "Manager", bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
        return state.allreduce(bucket.buffer())


class PureDistributedDataParallel(nn.Module):
    """Per-parameter allreduce from ``post_accumulate_grad`` hooks; no buckets, no reducer."""

    def __init__(self, manager: "Manager", module: nn.Module) -> None:
        super().__init__()
        self.module = module

        def post_grad_hook(p: torch.Tensor) -> None:
            if p.grad is not None:
                manager.allreduce(p.grad)

        for p in module.parameters():
            p.register_post_accumulate_grad_hook(post_grad_hook)

    def forward(self, *args: object) -> object:
        return self.module(*args)
