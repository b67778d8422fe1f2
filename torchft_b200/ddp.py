"""Fault-tolerant data parallelism across replica groups.

``DistributedDataParallel`` reuses torch's bucketing reducer but routes every gradient
bucket through ``Manager.allreduce`` (average over the replicas of the current quorum,
errors recorded instead of raised).  ``PureDistributedDataParallel`` is the hook-only
variant without buckets.  Parity: the reference's ``torchft/ddp.py:32-97``.
"""

from typing import TYPE_CHECKING, Any, List

import torch
from torch import nn
from torch.distributed import GradBucket
from torch.nn.parallel import DistributedDataParallel as _TorchDDP
from torch.utils.hooks import RemovableHandle

from torchft_b200.process_group import ProcessGroupDummy

if TYPE_CHECKING:
    from torchft_b200.manager import Manager


def _reduce_bucket(manager: "Manager", bucket: GradBucket) -> torch.futures.Future[torch.Tensor]:
    """DDP communication hook: one flat bucket, averaged over the live replica groups, in place.

    torch inspects the annotations of a hook at registration, so they are real objects, not strings.
    """
    return manager.allreduce(bucket.buffer())


class DistributedDataParallel(_TorchDDP):
    """torch DDP whose gradient communication goes through a ``Manager``.

    The module itself is built on a world-size-1 dummy group, so the constructor's
    parameter verification and broadcast do nothing (initial weights are synchronised
    by the step-0 heal).  Bucket layout is frozen (``find_unused_parameters=True`` stops
    the reducer from rebuilding buckets), because a replica that joins later must see
    exactly the same buckets as the ones already training.
    """

    def __init__(self, manager: "Manager", module: nn.Module, **kwargs: Any) -> None:
        kwargs["process_group"] = ProcessGroupDummy(0, 1)
        kwargs["find_unused_parameters"] = True  # keeps the first bucket assignment for good
        super().__init__(module, **kwargs)
        self.register_comm_hook(manager, _reduce_bucket)


class PureDistributedDataParallel(nn.Module):
    """Per-parameter allreduce from ``post_accumulate_grad`` hooks; no buckets, no reducer.

    Each gradient is handed to the manager the moment autograd has finished accumulating it, so
    communication overlaps the rest of the backward pass; ``Manager.should_commit`` waits for all of it.
    """

    def __init__(self, manager: "Manager", module: nn.Module) -> None:
        super().__init__()
        self.module = module
        self._handles: List[RemovableHandle] = []

        def reduce_when_ready(param: torch.Tensor) -> None:
            grad = param.grad
            if grad is None:
                return
            manager.allreduce(grad)

        for param in module.parameters():
            if param.requires_grad:
                self._handles.append(param.register_post_accumulate_grad_hook(reduce_when_ready))

    def remove_hooks(self) -> None:
        """Detaches the gradient hooks (the wrapped module then trains without communication)."""
        while self._handles:
            self._handles.pop().remove()

    def forward(self, *args: Any, **kwargs: Any) -> Any:
        return self.module(*args, **kwargs)
