"""Example: fault-tolerant data-parallel training of a small CNN.

Start a lighthouse, then one process (or one torchrun job) per replica group:

    python -m torchft_b200.lighthouse --min_replicas 1 --join_timeout_ms 10000 &
    REPLICA_GROUP_ID=0 NUM_REPLICA_GROUPS=2 TORCHFT_LIGHTHOUSE=http://127.0.0.1:29510 \
        torchrun --master-addr 127.0.0.1 --master-port 29600 --nproc-per-node 1 train_ddp.py
    REPLICA_GROUP_ID=1 NUM_REPLICA_GROUPS=2 TORCHFT_LIGHTHOUSE=http://127.0.0.1:29510 \
        torchrun --master-addr 127.0.0.1 --master-port 29601 --nproc-per-node 1 train_ddp.py

Kill either job at any time and start it again: it rejoins the quorum, pulls the weights
and optimizer state from the survivor and continues.  Data is synthetic (CIFAR-10 shaped)
so the example runs without a dataset; swap ``SyntheticImages`` for a real one.

Same role as the reference's ``train_ddp.py`` (LeNet-style CNN, batch 64, AdamW).
"""

import logging
import os
import sys
from datetime import timedelta

import torch
from torch import nn, optim
from torch.utils.data import DataLoader, Dataset

from torchft_b200 import DistributedDataParallel, DistributedSampler, Manager, Optimizer, ProcessGroupGloo
from torchft_b200.models.lenet import LeNet

logging.basicConfig(level=logging.INFO)


class SyntheticImages(Dataset):
    def __init__(self, n: int = 50000) -> None:
        self.n = n

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i: int):
        g = torch.Generator().manual_seed(i)
        return torch.randn(3, 32, 32, generator=g), int(torch.randint(10, (1,), generator=g))


def main() -> None:
    replica_group = int(os.environ.get("REPLICA_GROUP_ID", 0))
    num_replica_groups = int(os.environ.get("NUM_REPLICA_GROUPS", 2))
    total_steps = int(os.environ.get("TOTAL_STEPS", 10000))
    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)

    dataset = SyntheticImages()
    # Shards the data over replica groups x ranks; a group that is down simply skips its shard.
    sampler = DistributedSampler(
        dataset,
        replica_group=replica_group,
        num_replica_groups=num_replica_groups,
        rank=int(os.environ.get("RANK", 0)),
        num_replicas=int(os.environ.get("WORLD_SIZE", 1)),
        shuffle=True,
    )
    loader = DataLoader(dataset, batch_size=64, sampler=sampler, num_workers=0)

    def load_state_dict(state):
        model.load_state_dict(state["model"])
        optimizer.load_state_dict(state["optim"])

    def state_dict():
        return {"model": model.state_dict(), "optim": optimizer.state_dict()}

    if use_cuda:
        # peer-memory collectives with bounded waits (GPUs of one NVLink domain) ...
        from torchft_b200.parallel.nvlink import ProcessGroupNVLink

        pg = ProcessGroupNVLink(timeout=timedelta(seconds=5))
    else:
        # ... or Gloo over TCP on CPU
        pg = ProcessGroupGloo(timeout=timedelta(seconds=5))

    manager = Manager(
        pg=pg,
        min_replica_size=1,
        load_state_dict=load_state_dict,
        state_dict=state_dict,
        replica_id=f"train_ddp_{replica_group}",
        timeout=timedelta(seconds=10),
    )

    model = LeNet().to(device)
    model = DistributedDataParallel(manager, model)
    optimizer = Optimizer(manager, optim.AdamW(model.parameters()))
    criterion = nn.CrossEntropyLoss()
    print(model)

    # Durable checkpoints (optional): besides model and optimizer they hold manager.state_dict()
    # (step and batches_committed).  One replica group writes; every group reads after a full restart.
    ckpt_dir = os.environ.get("CHECKPOINT_DIR")
    ckpt_every = int(os.environ.get("CHECKPOINT_EVERY", 100))
    if ckpt_dir:
        from torchft_b200.utils.durable import load_checkpoint, save_checkpoint

        restored = load_checkpoint(ckpt_dir, manager, rank=int(os.environ.get("RANK", 0)),
                                   world_size=int(os.environ.get("WORLD_SIZE", 1)))
        if restored is not None:
            load_state_dict(restored["user"])
            print(f"resumed from step {manager.current_step()}")
    last_saved = manager.current_step()
    while True:
        for inputs, labels in loader:
            inputs, labels = inputs.to(device), labels.to(device)
            optimizer.zero_grad()  # starts the quorum for this step
            loss = criterion(model(inputs), labels)
            loss.backward()  # gradients are averaged over the live replica groups
            optimizer.step()  # applied only if every rank of the group voted to commit
            if manager.current_step() % 100 == 0:
                print(f"[{manager.current_step()}] loss = {loss.item():.4f} participants = {manager.num_participants()}")
            if ckpt_dir and replica_group == 0 and manager.current_step() >= last_saved + ckpt_every:
                save_checkpoint(ckpt_dir, manager, state_dict(), rank=int(os.environ.get("RANK", 0)))
                last_saved = manager.current_step()
            if manager.current_step() >= total_steps:
                manager.shutdown(wait=False)
                sys.exit(0)


if __name__ == "__main__":
    main()
