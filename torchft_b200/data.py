"""Data sharding across replica groups.

``DistributedSampler`` shards a dataset over ``num_replica_groups x num_replicas``
workers.  The mapping is static, so when a replica group is down its shard is simply
not visited: this sampler is lossy by design and fits jobs where exact epoch
boundaries do not matter.  Dataloader state is per replica group and must be
checkpointed with the model.  Same arithmetic as the reference's
``torchft/data.py:24-77``.
"""

from __future__ import annotations

from typing import Optional

import torch.distributed as dist
from torch.utils import data


class DistributedSampler(data.distributed.DistributedSampler):
    def __init__(
        self,
        dataset: data.Dataset,
        replica_group: int,
        num_replica_groups: int,
        rank: Optional[int] = None,
        num_replicas: Optional[int] = None,
        **kwargs: object,
    ) -> None:
        """
        Args:
            replica_group: index of this replica group
            num_replica_groups: maximum number of replica groups of the job
            rank / num_replicas: local rank and size inside the group (default: the
                default process group's)
        """
        if rank is None:
            rank = dist.get_rank()
        if num_replicas is None:
            num_replicas = dist.get_world_size()
        self.global_rank: int = rank + num_replicas * replica_group
        self.global_world_size: int = num_replicas * num_replica_groups
        super().__init__(dataset, rank=self.global_rank, num_replicas=self.global_world_size, **kwargs)  # type: ignore[arg-type]
