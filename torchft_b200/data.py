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
        group_size = dist.get_world_size() if num_replicas is None else num_replicas
        local_rank = dist.get_rank() if rank is None else rank
        if not 0 <= replica_group < num_replica_groups:
            raise ValueError(f"replica_group {replica_group} outside [0, {num_replica_groups})")
        if not 0 <= local_rank < group_size:
            raise ValueError(f"rank {local_rank} outside [0, {group_size})")
        # groups are laid out one after the other: group g owns global ranks [g * size, (g + 1) * size)
        self.global_world_size: int = num_replica_groups * group_size
        self.global_rank: int = replica_group * group_size + local_rank
        super().__init__(dataset, num_replicas=self.global_world_size, rank=self.global_rank, **kwargs)  # type: ignore[arg-type]
