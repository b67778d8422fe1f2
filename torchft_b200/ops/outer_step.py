"""Fused DiLoCo outer step (``csrc/kernels/outer_step.cu``).

Two kernels replace the reference's per-parameter ATen chain
(``torchft/local_sgd.py:212-225``: sub, allreduce, divide, restore copy, SGD step, save
copy):

* ``pseudograd``: ``comm = local - global`` over the flat buckets in one pass;
* ``nesterov_update``: given the replica-averaged pseudo-gradient ``g``::

      buf    = momentum * buf + g
      step   = g + momentum * buf        (nesterov)   |   buf   (plain momentum)
      global = global - lr * step
      param  = global;  backup = global

  reading g, global and buf once and writing param, backup and buf once.

The update runs only after the group voted to commit, so "no commit => weights
untouched" is preserved.  The momentum buffers are the outer optimizer's own state
tensors (views into one flat buffer), so ``outer_optimizer.state_dict()`` stays valid.
"""

from __future__ import annotations

import ctypes
from typing import TYPE_CHECKING, Dict, List, Optional, Tuple

import torch
from torch import optim

from . import _lib

if TYPE_CHECKING:
    from torchft_b200.local_sgd import _FlatBuckets


class FusedOuterStep:
    def __init__(
        self,
        params: List[torch.Tensor],
        backup: "_FlatBuckets",
        comm: "_FlatBuckets",
        outer_optimizer: optim.SGD,
    ) -> None:
        self._params = params
        self._backup = backup
        self._comm = comm
        self._opt = outer_optimizer
        # flat views of the live parameters: pack/unpack go through these
        self._momentum: Dict[Tuple[torch.dtype, torch.device], torch.Tensor] = {}
        for key, flat in comm.flat.items():
            self._momentum[key] = torch.zeros(flat.numel(), dtype=torch.float32, device=flat.device)
        # expose momentum through the optimizer state (fp32 views shaped like the params)
        for key, idxs in comm.groups.items():
            base = comm.flat[key]
            for i in idxs:
                view = comm.views[i]
                assert view is not None
                off = (view.data_ptr() - base.data_ptr()) // base.element_size()
                buf = self._momentum[key][off : off + view.numel()].view(view.shape)
                outer_optimizer.state[params[i]]["momentum_buffer"] = buf
        self._first = True

    @classmethod
    def maybe_create(
        cls,
        params: List[torch.Tensor],
        backup: "_FlatBuckets",
        comm: "_FlatBuckets",
        outer_optimizer: optim.Optimizer,
    ) -> Optional["FusedOuterStep"]:
        if not _lib.available():
            return None
        if type(outer_optimizer) is not optim.SGD:
            return None
        if any(not p.is_cuda or p.dtype not in (torch.bfloat16, torch.float32) for p in params):
            return None
        if any(b.device.type != "cuda" for b in backup.flat.values()):
            return None
        if len(outer_optimizer.param_groups) != 1:
            return None
        g = outer_optimizer.param_groups[0]
        if g.get("dampening", 0) != 0 or g.get("weight_decay", 0) != 0 or g.get("maximize", False):
            return None
        opt_params = {id(p) for p in g["params"]}
        if opt_params != {id(p) for p in params}:
            return None
        return cls(params, backup, comm, outer_optimizer)  # type: ignore[arg-type]

    def compute_pseudogradients(self) -> None:
        """``comm = local - global`` (params are packed by the same kernel launch sequence)."""
        self._comm.copy_from_params(non_blocking=True)
        lib = _lib.lib()
        for key, flat in self._comm.flat.items():
            g = self._backup.flat[key]
            code = lib.tft_pseudograd(
                _lib.ptr(flat), _lib.ptr(g), ctypes.c_int64(flat.numel()),
                ctypes.c_int(1 if flat.dtype == torch.bfloat16 else 0), _lib.stream_ptr(),
            )
            _lib.check(code, "tft_pseudograd")
            _lib.count_launch()

    def apply_outer_update(self) -> None:
        g = self._opt.param_groups[0]
        lr, mu, nesterov = float(g["lr"]), float(g.get("momentum", 0.0)), bool(g.get("nesterov", False))
        lib = _lib.lib()
        for key, flat in self._comm.flat.items():
            code = lib.tft_nesterov_outer(
                _lib.ptr(flat), _lib.ptr(self._backup.flat[key]), _lib.ptr(self._momentum[key]),
                ctypes.c_int64(flat.numel()), ctypes.c_float(lr), ctypes.c_float(mu),
                ctypes.c_int(1 if nesterov else 0), ctypes.c_int(1 if self._first else 0),
                ctypes.c_int(1 if flat.dtype == torch.bfloat16 else 0), _lib.stream_ptr(),
            )
            _lib.check(code, "tft_nesterov_outer")
            _lib.count_launch()
        self._first = False
        # comm now holds the new global weights; scatter them back into the parameters
        self._comm.copy_to_params(non_blocking=True)
