"""Durable (on-disk) checkpoints to go with the live recovery of ``Manager``.

Live recovery copies state between replicas that are up; a job that loses ALL replicas needs a
checkpoint on disk.  The reference leaves that to the user and only notes what has to be in it
(``torchft/manager.py:83-84,619-629``, ``train_ddp.py:141-148``): the user state, the manager's
``state_dict()`` (step and batches committed) and the data loader position.  These two helpers
write and read exactly that, one file per rank, atomically.

    save_checkpoint(dir, manager, {"model": model.state_dict(), "optim": opt.state_dict()}, rank=rank)
    state = load_checkpoint(dir, manager, rank=rank)      # restores the manager, returns the user state

Every replica group holds the same weights after a committed step, so ONE group saving is
enough: call ``save_checkpoint`` where ``manager.replica_rank() == 0`` (or any fixed group) and,
after a full restart, load the same files in every group.
"""

from __future__ import annotations

import os
import tempfile
from typing import Any, Dict, Optional

import torch


def _path(directory: str, step: int, rank: int) -> str:
    return os.path.join(directory, f"step{step:010d}", f"rank{rank:05d}.pt")


def save_checkpoint(directory: str, manager, user_state: Dict[str, Any], rank: int = 0,
                    dataloader_state: Optional[Dict[str, Any]] = None) -> str:
    """Writes ``<directory>/step<N>/rank<R>.pt`` for the manager's current step; returns the path.

    Call it between ``should_commit()`` of one step and ``start_quorum()`` of the next, when the state is
    consistent.  The file appears under its final name only when it is complete.
    """
    step = manager.current_step()
    path = _path(directory, step, rank)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    payload = {"user": user_state, "torchft": manager.state_dict(), "dataloader": dataloader_state}
    fd, tmp = tempfile.mkstemp(dir=os.path.dirname(path), prefix=".tmp-")
    try:
        with os.fdopen(fd, "wb") as f:
            torch.save(payload, f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise
    return path


def latest_step(directory: str, world_size: int = 1) -> Optional[int]:
    """Newest step for which all ``world_size`` rank files exist (a partly written step is skipped)."""
    if not os.path.isdir(directory):
        return None
    steps = []
    for name in os.listdir(directory):
        if name.startswith("step") and name[4:].isdigit():
            step = int(name[4:])
            if all(os.path.exists(_path(directory, step, r)) for r in range(world_size)):
                steps.append(step)
    return max(steps) if steps else None


def load_checkpoint(directory: str, manager, rank: int = 0, step: Optional[int] = None, world_size: int = 1,
                    map_location: Any = "cpu") -> Optional[Dict[str, Any]]:
    """Loads the given (default: newest complete) step, restores ``manager`` and returns
    ``{"user": ..., "dataloader": ...}``; ``None`` when there is no checkpoint."""
    if step is None:
        step = latest_step(directory, world_size)
    if step is None:
        return None
    payload = torch.load(_path(directory, step, rank), map_location=map_location, weights_only=False)
    manager.load_state_dict(payload["torchft"])
    return {"user": payload["user"], "dataloader": payload.get("dataloader")}
