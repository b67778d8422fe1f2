"""Fused DiLoCo outer step (``csrc/kernels/elementwise.cu``, ``csrc/kernels/p2p_comm.cu``).

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

With the NVLink process group the whole outer step is ONE kernel (``diloco_outer_kernel``):
every replica averages its chunk of the local weights straight out of the peers' memory,
subtracts the global weights, hands the averaged pseudo-gradient chunk to everybody, and after
an in-kernel barrier applies momentum and the update for the whole buffer into spare
``global`` / momentum buffers that are swapped in after the commit vote
(``FusedOuterStep.attach_nvlink``).

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
        self._peer = None  # set by attach_nvlink

    # ------------------------------------------------------------------ single-kernel path over NVLink
    def attach_nvlink(self, pg) -> bool:
        """Switches to the one-kernel outer step when all weights share one dtype and device."""
        if len(self._comm.flat) != 1:
            return False
        key, flat = next(iter(self._comm.flat.items()))
        n = flat.numel()
        if (n * flat.element_size()) % 16:
            return False
        heap = pg.heap
        base = flat.data_ptr()

        def views_of(buf: torch.Tensor) -> List[torch.Tensor]:
            out = []
            for i in self._comm.groups[key]:
                v = self._comm.views[i]
                off = (v.data_ptr() - base) // flat.element_size()
                out.append(buf[off : off + v.numel()].view(v.shape))
            return out

        try:
            local = heap.alloc(n, flat.dtype)
            # the communication bucket doubles as the gradient buffer when it already lives in the heap
            grad = flat if heap.offset_of(flat) is not None else heap.alloc(n, flat.dtype)
        except RuntimeError:
            return False  # heap too small: stay on the two-kernel path
        globals_ = [self._backup.flat[key], torch.empty_like(self._backup.flat[key])]
        moms = [self._momentum[key], torch.zeros_like(self._momentum[key])]
        self._peer = {
            "key": key, "local": local, "grad": grad, "global": globals_, "mom": moms, "cur": 0,
            "local_views": views_of(local),
            "global_views": [views_of(g) for g in globals_],
            "mom_views": [views_of(m) for m in moms],
            "params": [self._params[i] for i in self._comm.groups[key]],
            "idxs": list(self._comm.groups[key]),
        }
        return True

    @property
    def single_kernel(self) -> bool:
        return self._peer is not None

    def launch_single_kernel(self, pg, num_participants: int, contribute: bool):
        """Packs the local weights and starts the fused kernel; returns the work object."""
        st = self._peer
        assert st is not None
        with torch.no_grad():
            torch._foreach_copy_(st["local_views"], [p.data for p in st["params"]])
        g = self._opt.param_groups[0]
        cur = st["cur"]
        return pg.fused_outer_step(
            [st["local"], st["grad"]],
            local=st["local"], grad=st["grad"], global_in=st["global"][cur], mom_in=st["mom"][cur],
            global_out=st["global"][1 - cur], mom_out=st["mom"][1 - cur], inv_n=1.0 / num_participants,
            lr=float(g["lr"]), momentum=float(g.get("momentum", 0.0)), nesterov=bool(g.get("nesterov", False)),
            first=self._first, contribute=contribute,
        )

    def commit_single_kernel(self) -> None:
        """After a successful vote: the spare buffers become the global weights and momentum."""
        st = self._peer
        assert st is not None
        cur = 1 - st["cur"]
        st["cur"] = cur
        key = st["key"]
        self._backup.flat[key] = st["global"][cur]
        self._momentum[key] = st["mom"][cur]
        for j, i in enumerate(st["idxs"]):
            self._backup.views[i] = st["global_views"][cur][j]
            state = self._opt.state[self._params[i]]
            if float(self._opt.param_groups[0].get("momentum", 0.0)) != 0.0:
                state["momentum_buffer"] = st["mom_views"][cur][j]
        with torch.no_grad():
            torch._foreach_copy_([p.data for p in st["params"]], st["global_views"][cur])
        self._first = False

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
