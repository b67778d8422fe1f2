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

from typing import TYPE_CHECKING, Any, Optional

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
