"""LocalSGD and DiLoCo: replicas train independently and synchronise every ``sync_every`` steps.

Both are context managers around an (inner) optimizer.  After every ``sync_every``
optimizer steps the quorum is computed and

* ``LocalSGD`` averages the parameters over the replicas;
* ``DiLoCo`` averages the pseudo-gradients (local weights minus the last global
  weights) and applies an outer optimizer (typically Nesterov SGD) to the global
  weights.

A copy of the last synchronised weights is kept; when a synchronisation does not
commit (an error, too few replicas) the weights are rolled back to it, so
"no commit => weights untouched" holds exactly as for per-step training.

Differences from the reference (``torchft/local_sgd.py:26-239``), which allreduces each
parameter tensor on its own and keeps the backup in host memory:

* parameters are packed into flat per-dtype buckets, so a synchronisation is a handful
  of large collectives instead of one per tensor;
* the backup lives on the parameters' device by default (``backup_device=None``) --
  180 GB of HBM makes the host round trip pointless; pass ``torch.device("cpu")`` for
  the host-memory behaviour;
* on CUDA with SGD as the outer optimizer, ``DiLoCo`` uses fused kernels: one for
  pseudo-gradient + cross-replica average, one for the Nesterov update of parameters,
  backup and momentum in a single pass (``torchft_b200.ops.outer_step``).
"""

from __future__ import annotations

import logging
from types import TracebackType
from typing import Callable, Dict, List, Optional, Tuple, Type

import torch
from torch import nn, optim
from torch.utils.hooks import RemovableHandle

from torchft_b200.manager import Manager

logger: logging.Logger = logging.getLogger(__name__)


class _FlatBuckets:
    """Flat per-(dtype, device) buffers mirroring a list of parameters."""

    def __init__(self, params: List[torch.Tensor], device: Optional[torch.device], pin_memory: bool,
                 alloc: Optional[Callable[[int, torch.dtype], torch.Tensor]] = None) -> None:
        """``alloc(numel, dtype)``, when given, provides the CUDA buffers (e.g. from a symmetric heap so
        that peer-memory collectives reduce them in place); it may raise to fall back to ``torch.zeros``."""
        self.params = params
        self.groups: Dict[Tuple[torch.dtype, torch.device], List[int]] = {}
        for i, p in enumerate(params):
            self.groups.setdefault((p.dtype, p.device), []).append(i)
        self.flat: Dict[Tuple[torch.dtype, torch.device], torch.Tensor] = {}
        self.views: List[Optional[torch.Tensor]] = [None] * len(params)
        for key, idxs in self.groups.items():
            dtype, pdev = key
            total = sum(params[i].numel() for i in idxs)
            # 16-byte aligned sub-tensors keep vectorised kernels happy
            align = max(16 // params[idxs[0]].element_size(), 1)
            offsets = []
            cursor = 0
            for i in idxs:
                offsets.append(cursor)
                cursor += (params[i].numel() + align - 1) // align * align
            total = cursor
            dev = device if device is not None else pdev
            buf = None
            if alloc is not None and dev.type == "cuda":
                try:
                    buf = alloc(total, dtype)
                except RuntimeError as e:  # heap too small: ordinary memory works too, through staging
                    logger.info(f"flat bucket of {total} elements does not fit the peer heap ({e}); using device memory")
            if buf is None:
                buf = torch.zeros(total, dtype=dtype, device=dev)
            if pin_memory and dev.type == "cpu" and torch.cuda.is_available():
                buf = buf.pin_memory()
            self.flat[key] = buf
            for i, off in zip(idxs, offsets):
                self.views[i] = buf[off : off + params[i].numel()].view(params[i].shape)

    def copy_from_params(self, non_blocking: bool = True) -> None:
        with torch.no_grad():
            for i, p in enumerate(self.params):
                self.views[i].copy_(p.data, non_blocking=non_blocking)  # type: ignore[union-attr]

    def copy_to_params(self, non_blocking: bool = False) -> None:
        with torch.no_grad():
            for i, p in enumerate(self.params):
                p.data.copy_(self.views[i], non_blocking=non_blocking)  # type: ignore[arg-type]


class LocalSGD:
    """Periodic parameter averaging (https://arxiv.org/abs/1805.09767), fault tolerant.

    The quorum is computed at each synchronisation.  If a replica fails between two
    synchronisations the survivors notice at the next one; a step whose
    synchronisation fails is rolled back to the previous synchronised weights.  In
    async-quorum mode a joining replica discards its first ``sync_every`` steps while
    it recovers; in sync mode the checkpoint is loaded before the first step.
    """

    def __init__(
        self,
        manager: Manager,
        model: nn.Module,
        optimizer: optim.Optimizer,
        sync_every: int,
        backup_device: Optional[torch.device] = None,
        pin_memory: bool = True,
        bucket_cap_mb: float = 512.0,
    ) -> None:
        """
        Args:
            sync_every: optimizer steps between synchronisations (>= 1)
            backup_device: where the rollback copy lives (default: with the parameters)
            pin_memory: pin a host-side backup
            bucket_cap_mb: largest single collective, in MiB
        """
        super().__init__()
        assert sync_every >= 1, "sync_every must be greater than or equal to 1"
        self._manager = manager
        self._model = model
        self._local_optimizer = optimizer
        self._local_step = 0
        self._sync_every = sync_every
        self._bucket_cap_bytes = int(bucket_cap_mb * 1024 * 1024)

        self._names: List[str] = [n for n, _ in model.named_parameters()]
        self._params: List[torch.Tensor] = [p for _, p in model.named_parameters()]
        self._backup = _FlatBuckets(self._params, backup_device, pin_memory)
        # name -> view into the flat backup (same keys as model.named_parameters())
        self._backup_parameters: Dict[str, torch.Tensor] = {
            n: v for n, v in zip(self._names, self._backup.views)  # type: ignore[misc]
        }
        # communication buckets on the parameters' own devices
        # communication buckets live in the process group's peer-addressable heap when it has one
        heap = getattr(getattr(manager, "_pg", None), "heap", None)
        self._comm = _FlatBuckets(self._params, None, False, alloc=heap.alloc if heap is not None else None)
        self._hooks: List[RemovableHandle] = []
        self._save_parameters()

    # -- context manager
    def __enter__(self) -> "LocalSGD":
        self._hooks.append(self._local_optimizer.register_step_post_hook(self._step_post_hook))
        return self

    def __exit__(
        self,
        exc_type: Optional[Type[BaseException]],
        exc_value: Optional[BaseException],
        traceback: Optional[TracebackType],
    ) -> bool:
        if exc_type is not None:
            # whatever happened mid-interval, go back to a state all replicas agree on
            self._restore_parameters()
        for hook in self._hooks:
            hook.remove()
        self._hooks.clear()
        return False

    # -- backup
    def _save_parameters(self) -> None:
        self._backup.copy_from_params(non_blocking=True)

    def _restore_parameters(self) -> None:
        self._backup.copy_to_params(non_blocking=False)

    def _step_post_hook(self, _optim: optim.Optimizer, _args: List[object], _kwargs: Dict[str, object]) -> None:
        self._local_step += 1
        if self._local_step >= self._sync_every:
            self.sync()

    def sync(self) -> None:
        """Computes the quorum and synchronises with the other replicas."""
        self._manager.start_quorum()
        self._perform_sync()
        self._local_step = 0

    def _perform_sync(self) -> None:
        self._average()
        if self._manager.should_commit():
            self._save_parameters()
        else:
            self._restore_parameters()

    # -- bucketed collectives
    def _allreduce_flat(self, flat: torch.Tensor) -> List["torch.futures.Future[torch.Tensor]"]:
        cap = max(self._bucket_cap_bytes // flat.element_size(), 1)
        futs = []
        for start in range(0, flat.numel(), cap):
            futs.append(self._manager.allreduce(flat[start : start + cap]))
        return futs

    def _average(self) -> None:
        """Averages all parameters: pack into flat buckets, allreduce, unpack."""
        self._comm.copy_from_params(non_blocking=True)
        futs: List["torch.futures.Future[torch.Tensor]"] = []
        for flat in self._comm.flat.values():
            futs.extend(self._allreduce_flat(flat))
        for f in futs:
            f.wait()
        self._comm.copy_to_params(non_blocking=True)


class DiLoCo(LocalSGD):
    """DiLoCo (https://arxiv.org/abs/2311.08105): averaged pseudo-gradients + outer optimizer.

    Requires a synchronous quorum (``Manager(use_async_quorum=False)``) because a
    recovering replica must hold the global weights before it computes a
    pseudo-gradient.  The pseudo-gradient is ``local - global`` and is handed to the
    outer optimizer as a gradient.
    """

    def __init__(
        self,
        manager: Manager,
        model: nn.Module,
        inner_optimizer: optim.Optimizer,
        outer_optimizer: optim.Optimizer,
        sync_every: int,
        backup_device: Optional[torch.device] = None,
        pin_memory: bool = True,
        bucket_cap_mb: float = 512.0,
        use_fused: Optional[bool] = None,
    ) -> None:
        if manager._use_async_quorum:
            raise ValueError(
                "Using DiLoCo require synchronous quorum to be enabled. "
                "Ensure that the manager is initialized with use_async_quorum=False"
            )
        super().__init__(manager, model, inner_optimizer, sync_every, backup_device, pin_memory, bucket_cap_mb)
        self._outer_optimizer = outer_optimizer
        self._fused = None
        if use_fused is None or use_fused:
            from torchft_b200.ops import outer_step

            self._fused = outer_step.FusedOuterStep.maybe_create(
                params=self._params,
                backup=self._backup,
                comm=self._comm,
                outer_optimizer=outer_optimizer,
            )
            if use_fused and self._fused is None:
                raise RuntimeError("fused DiLoCo outer step requested but not available for this configuration")
            if self._fused is not None:
                pg = getattr(manager, "_pg", None)
                if pg is not None and hasattr(pg, "fused_outer_step") and hasattr(pg, "heap"):
                    # pseudo-gradient, allreduce and Nesterov update become one kernel
                    self._fused.attach_nvlink(pg)

    def _perform_sync(self) -> None:
        if self._fused is not None:
            self._perform_sync_fused()
            return
        # pseudo-gradient straight into the communication buckets
        with torch.no_grad():
            for i, p in enumerate(self._params):
                view = self._comm.views[i]
                torch.sub(p.data, self._backup.views[i].to(p.device, non_blocking=True), out=view)  # type: ignore[union-attr]
                p.grad = view
        self._average_grads()
        # the outer optimizer steps from the GLOBAL weights
        self._restore_parameters()
        if self._manager.should_commit():
            self._outer_optimizer.step()
            self._save_parameters()
        self._outer_optimizer.zero_grad()

    def _average_grads(self) -> None:
        futs: List["torch.futures.Future[torch.Tensor]"] = []
        for flat in self._comm.flat.values():
            futs.extend(self._allreduce_flat(flat))
        for f in futs:
            f.wait()

    def _perform_sync_fused(self) -> None:
        fused = self._fused
        assert fused is not None
        if fused.single_kernel:
            fut = self._manager.run_collective(fused.launch_single_kernel, None)
            fut.wait()
            if self._manager.should_commit():
                fused.commit_single_kernel()
            else:
                self._restore_parameters()
            self._outer_optimizer.zero_grad()
            return
        # kernel 1: comm = local - global (one pass), then averaged across replicas
        fused.compute_pseudogradients()
        self._average_grads()
        if self._manager.should_commit():
            # kernel 2: momentum, global weights, parameters and backup in one pass
            fused.apply_outer_update()
        else:
            self._restore_parameters()
        self._outer_optimizer.zero_grad()
