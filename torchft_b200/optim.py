"""Optimizer wrapper that drives the fault-tolerance protocol.

``zero_grad()`` opens the step (``manager.start_quorum()``) and ``step()`` applies the
update only when the replica group voted to commit, so a step that hit a communication
error leaves the weights untouched.  Same contract as the reference's
``torchft/optim.py:24-63``.

Everything else an optimizer offers (``param_groups``, ``state``, ``state_dict``,
``load_state_dict``, ``add_param_group``, hooks, LR-scheduler access, ...) is forwarded to the
wrapped optimizer, so schedulers and checkpoint code keep working on the wrapper.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Any, Dict, Iterable, Optional, Tuple

import torch
from torch.optim import Optimizer

if TYPE_CHECKING:
    from torchft_b200.manager import Manager

# names that live on the wrapper itself (an LR scheduler re-binds ``step`` on the object it is given);
# all other reads and writes go to the wrapped optimizer
_OWN = frozenset(("optim", "manager", "step", "zero_grad"))


class OptimizerWrapper(Optimizer):
    """``Optimizer`` in the sense of ``isinstance`` (LR schedulers check that), a proxy otherwise."""

    def __init__(self, manager: "Manager", optim: Optimizer) -> None:
        # Optimizer.__init__ is skipped on purpose: there is no state of our own to set up.
        object.__setattr__(self, "optim", optim)
        object.__setattr__(self, "manager", manager)

    # ---- the two calls that carry the protocol
    def zero_grad(self, set_to_none: bool = True) -> None:
        """Start of a step: the quorum is requested before the gradients are cleared."""
        self.manager.start_quorum()
        self.optim.zero_grad(set_to_none)

    def step(self, closure: Optional[object] = None) -> None:
        """End of a step: the update happens only if the replica group votes to commit."""
        if closure is not None:
            raise AssertionError("optimizers that use closures are not supported")
        if not self.manager.should_commit():
            return
        self.optim.step()

    # ---- everything else belongs to the wrapped optimizer
    def __getattribute__(self, name: str) -> Any:
        if name in _OWN or (name.startswith("__") and name.endswith("__")):
            return object.__getattribute__(self, name)
        return getattr(object.__getattribute__(self, "optim"), name)

    def __setattr__(self, name: str, value: Any) -> None:
        if name in _OWN:
            object.__setattr__(self, name, value)
        else:
            setattr(self.optim, name, value)

    def __repr__(self) -> str:
        return f"OptimizerWrapper({self.optim!r})"


class FusedAdamW(Optimizer):
    """AdamW for bf16 parameters with fp32 moments, one fused kernel launch per parameter.

    For a model that is trained through the stock interfaces (``DistributedDataParallel`` +
    ``OptimizerWrapper``) rather than through ``HSDPEngine``, which carries the same update for its
    flat buffers.  ``torch.optim.AdamW`` keeps the moments in the parameters' dtype; here they stay
    fp32 next to bf16 parameters.  Differences that matter for fault tolerance:

    * the moments are allocated in the constructor (under whatever allocator is current, e.g.
      ``SymmetricHeap.allocating``), so a process that joins has live tensors for a checkpoint
      transport to write into before its first step;
    * ``state_dict`` hands out those tensors themselves and ``load_state_dict`` copies into them in
      place, keeping their dtype and storage (the base class would cast the moments to bf16 and
      replace the tensors).

    Parameters that are not bf16 CUDA tensors take the same update in plain PyTorch arithmetic.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 1e-2) -> None:
        if lr < 0 or eps < 0 or weight_decay < 0 or not (0 <= betas[0] < 1 and 0 <= betas[1] < 1):
            raise ValueError(f"invalid hyper-parameters: lr={lr} betas={betas} eps={eps} weight_decay={weight_decay}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        for group in self.param_groups:
            self._prepare(group)

    def _prepare(self, group: Dict[str, Any]) -> None:
        group.setdefault("step", 0)
        for p in group["params"]:
            if p not in self.state:
                self.state[p] = {
                    "exp_avg": torch.zeros(p.shape, dtype=torch.float32, device=p.device),
                    "exp_avg_sq": torch.zeros(p.shape, dtype=torch.float32, device=p.device),
                }

    def add_param_group(self, param_group: Dict[str, Any]) -> None:
        super().add_param_group(param_group)
        if hasattr(self, "state"):  # the base constructor adds the initial groups before `state` is usable here
            self._prepare(self.param_groups[-1])

    @torch.no_grad()
    def step(self, closure: Optional[object] = None) -> None:  # type: ignore[override]
        if closure is not None:
            raise AssertionError("closures are not supported")
        from torchft_b200.ops import functional as F

        for group in self.param_groups:
            group["step"] += 1
            t, lr, (b1, b2), eps, wd = group["step"], group["lr"], group["betas"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                g = p.grad
                if g is None:
                    continue
                m, v = self.state[p]["exp_avg"], self.state[p]["exp_avg_sq"]
                if p.is_cuda and p.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and p.is_contiguous() and g.is_contiguous():
                    F.adamw_step_(p, g, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd, step=t)
                    continue
                gf = g.float()
                m.mul_(b1).add_(gf, alpha=1 - b1)
                v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
                update = (m / (1 - b1**t)) / ((v / (1 - b2**t)).sqrt() + eps)
                p.copy_((p.float() * (1 - lr * wd) - lr * update).to(p.dtype))

    def state_dict(self) -> Dict[str, Any]:  # type: ignore[override]
        """The live moment tensors (in parameter order) and the hyper-parameters of every group."""
        return {
            "groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups],
            "exp_avg": [[self.state[p]["exp_avg"] for p in g["params"]] for g in self.param_groups],
            "exp_avg_sq": [[self.state[p]["exp_avg_sq"] for p in g["params"]] for g in self.param_groups],
        }

    @torch.no_grad()
    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:  # type: ignore[override]
        if len(state_dict["groups"]) != len(self.param_groups):
            raise ValueError("the state has a different number of parameter groups")
        for group, saved, ms, vs in zip(self.param_groups, state_dict["groups"], state_dict["exp_avg"], state_dict["exp_avg_sq"]):
            if len(ms) != len(group["params"]) or len(vs) != len(group["params"]):
                raise ValueError("the state has a different number of parameters")
            group.update({k: (tuple(v) if k == "betas" else v) for k, v in saved.items()})
            for p, m, v in zip(group["params"], ms, vs):
                for mine, theirs in ((self.state[p]["exp_avg"], m), (self.state[p]["exp_avg_sq"], v)):
                    if mine.data_ptr() != theirs.data_ptr():  # a transport may have written in place already
                        mine.copy_(theirs)
