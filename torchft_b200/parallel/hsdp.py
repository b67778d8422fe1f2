"""Hybrid-sharded data parallel training engine (HSDP) with per-step fault tolerance.

Layout
------
Parameters are grouped into *units* (embedding, one per transformer block, head).  All
units live in ONE flat bf16 parameter buffer and ONE flat bf16 gradient buffer; module
parameters are views into the first and carry ``main_grad`` views into the second, so
weight-gradient GEMMs write their result in place and no flatten / unflatten copy exists.

Inside a replica group of ``S`` GPUs every rank owns the ``1/S`` slice of each unit:
fp32 AdamW moments exist only for that slice.  A training step is

1. forward / backward on the full (gathered) parameters, which stay resident in HBM,
2. per unit: reduce-scatter of the gradients over the shard group, then the allreduce of
   the owned slice over the replica groups (through the ``Manager``: averaged over the
   participating replicas, errors recorded instead of raised),
3. ``Manager.should_commit()``; if it passes, fused AdamW on the owned slices, unit by unit in
   forward order on a stream of its own; the updated slices are all-gathered at the start of
   the next step, and the next forward waits unit by unit.  The optimizer is bound by HBM
   bandwidth and the forward pass by the tensor cores, so the two overlap well.

Steps 2 and 3 use the NVLink peer-memory kernels of ``torchft_b200.parallel.nvlink`` when a
shard communicator is given; with a single GPU per replica group they reduce to the
cross-replica allreduce.

The reference composes the same strategy from stock FSDP2 plus its ``ManagedProcessGroup``
(``torchft/process_group.py:1300-1331``, exercised by ``torchft/fsdp_test.py``); that
composition is available here too through ``ft_init_device_mesh``.  This engine is the
B200-first path used by ``bench.py``.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch
from torch import nn

from torchft_b200.ops import functional as F

ALIGN = 128  # elements; keeps every unit and every shard 256-byte aligned


@dataclass
class Unit:
    name: str
    params: List[nn.Parameter]
    offset: int  # start inside the flat buffers (elements)
    numel: int  # padded length (multiple of ALIGN * shard_world)
    fused_gather: bool = False  # its all-gather happens inside the GEMM that first uses it
    fused_rs: bool = False  # its reduce-scatter happens inside the weight-gradient GEMM


class ShardComm:
    """Collectives over the GPUs of one replica group (the shard dimension)."""

    rank: int = 0
    world: int = 1

    def reduce_scatter_(self, full: torch.Tensor, shard_numel: int) -> None:
        """Sums ``full`` over the group; rank r ends up with the sum in its slice r."""

    def all_gather_(self, full: torch.Tensor, shard_numel: int) -> None:
        """Every rank's slice r is copied into slice r of every other rank's ``full``."""

    def status_async(self):
        """``(pinned int32 tensor, event)``: after the event, non-zero means that a collective queued
        before this call gave up waiting for a peer.  ``None``: this backend raises instead."""
        return None

    def renew(self) -> None:
        """Called on every rank of the group after a step that did not commit."""


class HSDPEngine:
    def __init__(
        self,
        model: nn.Module,
        units: List[Tuple[str, List[nn.Parameter]]],
        *,
        manager=None,
        shard_comm: Optional[ShardComm] = None,
        lr: float = 3e-4,
        betas: Tuple[float, float] = (0.9, 0.95),
        eps: float = 1e-8,
        weight_decay: float = 0.1,
        alloc: Optional[Callable[[int, torch.dtype], torch.Tensor]] = None,
        fused_gather_comm=None,
        fused_rs_comm=None,
    ) -> None:
        """
        Args:
            units: ``[(name, params)]`` in forward order (``Llama.units()``)
            manager: ``torchft_b200.Manager`` for the cross-replica dimension (optional)
            shard_comm: collectives of the shard dimension (``None``: one GPU per group)
            alloc: allocator for the flat buffers, ``alloc(numel, dtype) -> tensor``; the
                NVLink backend passes its symmetric-heap allocator so peers can address them
            fused_gather_comm: an ``NVLinkCommunicator`` of the shard group (a channel of its own).
                Units that consist of ONE matrix ``[N, K]`` marked ``linear_weight`` by the model, with ``N % (256 * shard_world) == 0`` and
                ``K % 64 == 0`` (``Llama.units(per_weight=True)``) then skip the all-gather kernel:
                their rows are gathered inside the first GEMM that uses the weight in a step
            fused_rs_comm: an ``NVLinkCommunicator`` of the shard group (again a channel of its own).
                Units that consist of ONE ``linear_weight`` matrix ``[N, K]`` with ``N % (128 * shard_world) == 0``
                and ``K % 256 == 0`` get their gradient reduce-scattered inside the weight-gradient GEMM
                (``NVLinkCommunicator.wgrad_reduce_scatter``); no reduce-scatter kernel runs for them
        """
        self.model = model
        self.manager = manager
        self.comm = shard_comm if shard_comm is not None else ShardComm()
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.opt_step = 0
        first = units[0][1][0]
        self.device = first.device
        S = self.comm.world
        quantum = ALIGN * S

        self.units: List[Unit] = []
        cursor = 0
        for name, params in units:
            n = sum(-(-p.numel() // 8) * 8 for p in params)
            n = -(-n // quantum) * quantum
            self.units.append(Unit(name, list(params), cursor, n))
            cursor += n
        self.total = cursor

        if alloc is None:
            def alloc(numel: int, dtype: torch.dtype) -> torch.Tensor:
                return torch.zeros(numel, dtype=dtype, device=self.device)

        self.flat_param = alloc(self.total, torch.bfloat16)
        self.flat_grad = alloc(self.total, torch.bfloat16)
        # re-point the module parameters into the flat buffers
        with torch.no_grad():
            for u in self.units:
                off = u.offset
                for p in u.params:
                    n = p.numel()
                    view = self.flat_param[off : off + n].view(p.shape)
                    view.copy_(p.data)
                    p.data = view
                    p.main_grad = self.flat_grad[off : off + n].view(p.shape)
                    p.main_grad_initialized = False
                    off += -(-n // 8) * 8
        # optimizer state only for the owned slices, laid out unit after unit
        self.shard_total = self.total // S
        self.exp_avg = alloc(self.shard_total, torch.float32)
        self.exp_avg_sq = alloc(self.shard_total, torch.float32)
        # communication of finished units overlaps the rest of the backward pass on this stream
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        # the optimizer runs here so that the next step's forward can start while it still works
        self.opt_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self._updated: Dict[str, "torch.cuda.Event"] = {}
        self._by_name = {u.name: u for u in self.units}
        # callbacks name a block ("layer3"); its units are "layer3" itself or "layer3/<part>"
        self._by_prefix: Dict[str, List[Unit]] = {}
        for u in self.units:
            self._by_prefix.setdefault(u.name.split("/", 1)[0], []).append(u)
        self._fused_units: List[Unit] = []
        self._fused_comm = fused_gather_comm if S > 1 else None
        if fused_gather_comm is not None and S > 1:
            for u in self.units:
                if len(u.params) != 1 or u.params[0].dim() != 2 or not getattr(u.params[0], "linear_weight", False):
                    continue  # only matrices that the model marks as used through F.linear alone
                n_rows, k = u.params[0].shape
                if n_rows % (256 * S) == 0 and k % 64 == 0 and u.numel == n_rows * k:
                    u.fused_gather = True
                    u.params[0].gather_comm = fused_gather_comm
                    u.params[0].gather_pending = False
                    self._fused_units.append(u)
        self._rs_comm = fused_rs_comm if S > 1 else None
        if self._rs_comm is not None:
            biggest = (0, 0)
            for u in self.units:
                if len(u.params) != 1 or u.params[0].dim() != 2 or not getattr(u.params[0], "linear_weight", False):
                    continue
                n_rows, k = u.params[0].shape
                if self._rs_comm.can_fuse_wgrad(n_rows, k) and u.numel == n_rows * k:
                    u.fused_rs = True
                    u.params[0].rs_comm = self._rs_comm
                    if n_rows * k > biggest[0] * biggest[1]:
                        biggest = (n_rows, k)
            if biggest[0]:
                self._rs_comm.reserve_wgrad_staging(*biggest)
        self._synced: set = set()
        self._futures: list = []
        if hasattr(model, "unit_grad_ready"):
            model.unit_grad_ready = self._unit_grad_ready
        # parameter refresh (all-gather of updated slices) runs unit by unit on the communication
        # stream; forward waits per unit, so only the first unit's exchange is exposed
        self._gathered: Dict[str, "torch.cuda.Event"] = {}
        self._prefetch = hasattr(model, "unit_pre_forward") and self.comm_stream is not None
        if self._prefetch:
            model.unit_pre_forward = self._unit_pre_forward

    # ------------------------------------------------------------------ slices
    def _shard_numel(self, u: Unit) -> int:
        return u.numel // self.comm.world

    def _own(self, flat: torch.Tensor, u: Unit) -> torch.Tensor:
        n = self._shard_numel(u)
        start = u.offset + self.comm.rank * n
        return flat[start : start + n]

    def _state_slice(self, buf: torch.Tensor, u: Unit) -> torch.Tensor:
        start = u.offset // self.comm.world
        return buf[start : start + self._shard_numel(u)]

    # ------------------------------------------------------------------ step pieces
    def zero_grad(self) -> None:
        """Gradients are overwritten by the first backward of a step; nothing is cleared."""
        for u in self.units:
            for p in u.params:
                p.main_grad_initialized = False
                p.grad = None
        self._synced = set()
        self._futures = []

    def _sync_unit(self, u: Unit) -> None:
        """Queues the communication of one unit's gradients on the communication stream."""
        if u.name in self._synced:
            return
        self._synced.add(u.name)
        if self.comm.world == 1 and self.manager is None:
            return
        current = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(current)
        with torch.cuda.stream(self.comm_stream):
            full = self.flat_grad[u.offset : u.offset + u.numel]
            if self.comm.world > 1 and not u.fused_rs:  # fused_rs: the wgrad GEMM already left the sum in the own slice
                self.comm.reduce_scatter_(full, self._shard_numel(u))
            if self.manager is not None:
                self._futures.append(self.manager.allreduce(self._own(self.flat_grad, u)))

    def _unit_grad_ready(self, name: str) -> None:
        """Backward-time callback of the model: the gradients of the named block's units are final."""
        for u in reversed(self._by_prefix.get(name, ())):
            self._sync_unit(u)

    def sync_gradients(self) -> None:
        """Reduce-scatter inside the replica group, then average the owned slices across groups.

        Units whose gradients were announced during backward are already in flight; the rest
        (at least the embedding, whose gradient is complete only when backward returns) go now.
        """
        for u in reversed(self.units):  # backward order: the last units finished first
            self._sync_unit(u)
        # The shard-group kernels report a peer that never showed up through a status word, not an
        # exception: fetch it behind the last collective of each communicator.
        probes = []
        if self.comm.world > 1 and self.comm_stream is not None:
            with torch.cuda.stream(self.comm_stream):
                probes.append(("shard-group collective", self.comm.status_async()))
            if self._fused_comm is not None:
                probes.append(("fused all-gather GEMM", self._fused_comm.status_async()))  # ran on this stream
            if self._rs_comm is not None:
                probes.append(("weight-gradient GEMM fused with reduce-scatter", self._rs_comm.status_async()))
        for f in self._futures:
            f.wait()
        self._futures = []
        for what, probe in probes:
            if probe is None:
                continue
            status, event = probe
            event.synchronize()
            code = int(status.item())
            if code != 0:
                self._shard_failure(TimeoutError(
                    f"{what}: device-side wait gave up (status {code}); gradients or parameters of this step are partial"))
        torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

    def _shard_failure(self, error: Exception) -> None:
        """A collective inside the replica group failed: the step must not commit anywhere in the group."""
        if self.manager is not None:
            self.manager.report_error(error)
        else:
            raise error

    def optimizer_step(self, grad_scale: float = 1.0) -> None:
        """Fused AdamW on the owned slices (the next step starts by all-gathering them).

        With a model that announces its units in forward (``unit_pre_forward``) the kernels go to
        the optimizer stream and every unit gets an event; otherwise they run on the calling stream.
        """
        self.opt_step += 1
        b1, b2 = self.betas
        current = torch.cuda.current_stream(self.device) if self.opt_stream is not None else None
        side = self.opt_stream if self._prefetch else None
        if side is not None:
            side.wait_stream(current)  # gradients are final on the calling stream
        ctx = torch.cuda.stream(side) if side is not None else contextlib.nullcontext()
        with ctx:
            for u in self.units:
                F.adamw_step_(
                    self._own(self.flat_param, u), self._own(self.flat_grad, u),
                    self._state_slice(self.exp_avg, u), self._state_slice(self.exp_avg_sq, u),
                    lr=self.lr, beta1=b1, beta2=b2, eps=self.eps, weight_decay=self.weight_decay,
                    step=self.opt_step, grad_scale=grad_scale,
                )
                if side is not None:
                    ev = torch.cuda.Event()
                    ev.record(side)
                    self._updated[u.name] = ev

    def wait_optimizer(self) -> None:
        """Host-side wait until the optimizer kernels in flight are done (state is final afterwards)."""
        if self.opt_stream is not None:
            self.opt_stream.synchronize()

    def gather_parameters(self, overlap: bool = False) -> None:
        """All-gathers the owned parameter slices of every unit inside the replica group.

        With ``overlap`` the exchange is queued on the communication stream and the model's
        ``unit_pre_forward`` callback makes the compute stream wait unit by unit; otherwise the
        calling stream sees all parameters complete when this returns.
        """
        current = torch.cuda.current_stream(self.device) if self.comm_stream is not None else None
        if not (overlap and self._prefetch):
            if self._updated:  # optimizer work of the previous step may still be in flight on its stream
                current.wait_stream(self.opt_stream)
                self._updated.clear()
            if self.comm.world > 1:
                for u in self.units:
                    self.comm.all_gather_(self.flat_param[u.offset : u.offset + u.numel], self._shard_numel(u))
            return
        if self.comm.world == 1:
            return  # forward waits for the optimizer events directly
        for u in self._fused_units:
            u.params[0].gather_pending = True  # gathered by the GEMM that uses the weight first
        self.comm_stream.wait_stream(current)  # recovery writes of the slices are ordered first
        with torch.cuda.stream(self.comm_stream):
            for u in self.units:
                if u.fused_gather:
                    continue  # its optimizer event stays in _updated: forward waits for it directly
                ev = self._updated.pop(u.name, None)
                if ev is not None:
                    self.comm_stream.wait_event(ev)  # this unit's slice has been updated
                self.comm.all_gather_(self.flat_param[u.offset : u.offset + u.numel], self._shard_numel(u))
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                self._gathered[u.name] = ev

    def _unit_pre_forward(self, name: str) -> None:
        for u in self._by_prefix.get(name, ()):
            for pending in (self._gathered, self._updated):
                ev = pending.pop(u.name, None)
                if ev is not None:
                    torch.cuda.current_stream(self.device).wait_event(ev)

    def _finish_gather(self) -> None:
        """Units whose forward did not run (or ran without the callback) are waited for here."""
        if self._gathered:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
            self._gathered.clear()
        if self._updated:
            torch.cuda.current_stream(self.device).wait_stream(self.opt_stream)
            self._updated.clear()

    # ------------------------------------------------------------------ whole step
    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One fault-tolerant training step; returns the (local) loss tensor."""
        marks = self._timing_marks() if self.timing is not None else None
        if self.manager is not None:
            self.manager.start_quorum()
        # Updated slices are exchanged at the START of a step, on every rank, whether or not it (or a
        # group mate) just recovered: recovery rewrites only the owned slice of a rank, and which
        # ranks of a group recover differs per rank, so a collective inside load_state_dict would
        # not be symmetric.
        self.gather_parameters(overlap=True)
        self.zero_grad()
        loss = self.model(tokens, targets)
        self._finish_gather()
        if marks is not None:
            marks("forward")
        loss.backward()
        if marks is not None:
            marks("backward")
        self.sync_gradients()
        if marks is not None:
            marks("gradient_sync_tail")
        grad_scale = 1.0 / self.comm.world  # reduce-scatter sums over the shard group
        committed = self.manager is None or self.manager.should_commit()
        if marks is not None:
            marks("commit_vote", host=True)
        if committed:
            self.optimizer_step(grad_scale)
            if marks is not None:
                marks("optimizer_queued", final=True)
        elif marks is not None:
            marks("not_committed", final=True)
        if not committed and self.comm.world > 1:
            # The vote is group-wide, so every rank of the group is here: all move to fresh flags and
            # sequence numbers, whichever of them saw the failure (one side may have given up on a
            # collective that the other side completed or never started).
            torch.cuda.synchronize(self.device)
            self.comm.renew()
            for extra in (self._fused_comm, self._rs_comm):
                if extra is not None and getattr(extra, "_bound", None) is not None:
                    extra.renew()
        return loss.detach()

    # ------------------------------------------------------------------ optional per-phase timing
    timing: Optional[List[Dict[str, float]]] = None  # set to [] to collect one dict per step

    def _timing_marks(self):
        """Per-phase timing of one step (``engine.timing = []`` switches it on): device time between
        events on the compute stream for the phases that queue GPU work, host time for the vote."""
        import time as _time

        stream = torch.cuda.current_stream(self.device)
        events = []
        host = [_time.perf_counter()]
        first = torch.cuda.Event(enable_timing=True)
        first.record(stream)
        events.append(("start", first))
        row: Dict[str, float] = {}

        def mark(name: str, host_only: bool = False, final: bool = False, **kw) -> None:
            host_only = host_only or kw.get("host", False)
            now = _time.perf_counter()
            row[f"{name}_host_ms"] = (now - host[0]) * 1e3
            host[0] = now
            if not host_only:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                events.append((name, ev))
            if final:
                events[-1][1].synchronize()
                for (_, a), (n, b) in zip(events, events[1:]):
                    row[f"{n}_device_ms"] = a.elapsed_time(b)
                assert self.timing is not None
                self.timing.append(row)

        return mark

    # ------------------------------------------------------------------ state for live recovery
    def state_dict(self) -> Dict[str, object]:
        """State of THIS rank's slice; rank r of a recovering group pulls it from rank r of a healthy one."""
        # views, not copies: an NVLink transport moves them peer to peer without staging
        self.wait_optimizer()  # whoever reads these views later, on whatever stream, sees final values
        own_params = [self._own(self.flat_param, u) for u in self.units]
        return {"params": own_params, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "opt_step": self.opt_step}

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        params = sd["params"]
        assert isinstance(params, (list, tuple)) and len(params) == len(self.units)
        self.wait_optimizer()  # nothing of an earlier step may still write the state

        def put(dst: torch.Tensor, src: torch.Tensor) -> None:
            # an in-place transport hands back our own tensors: nothing to copy then
            if src.data_ptr() != dst.data_ptr():
                dst.copy_(src.to(dst.device, non_blocking=True))

        with torch.no_grad():
            for u, src in zip(self.units, params):
                put(self._own(self.flat_param, u), src)
            put(self.exp_avg, sd["exp_avg"])  # type: ignore[arg-type]
            put(self.exp_avg_sq, sd["exp_avg_sq"])  # type: ignore[arg-type]
        self.opt_step = int(sd["opt_step"])  # type: ignore[arg-type]
