"""Optimizer wrapper that drives the fault-tolerance protocol.

``zero_grad()`` opens the step (``manager.start_quorum()``) and ``step()`` applies the
update only when the replica group voted to commit, so a step that hit a communication
error leaves the weights untouched.  Same contract as the reference's
``torchft/optim.py:24-63``.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Any, Dict, List, Mapping, Optional

import torch
from torch.optim import Optimizer

if TYPE_CHECKING:
    from torchft_b200.manager import Manager


class OptimizerWrapper(Optimizer):
    def __init__(self, manager: "Manager", optim: Optimizer) -> None:
        # Optimizer.__init__ is skipped on purpose: every attribute proxies ``optim``.
        self.optim = optim
        self.manager = manager

    def add_param_group(self, param_group: Dict[str, Any]) -> None:
        self.optim.add_param_group(param_group)

    def load_state_dict(self, state_dict: Mapping[str, Any]) -> None:
        self.optim.load_state_dict(state_dict)  # type: ignore[arg-type]

    def state_dict(self) -> Dict[str, Any]:
        return self.optim.state_dict()

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.manager.start_quorum()
        self.optim.zero_grad(set_to_none)

    def step(self, closure: Optional[object] = None) -> None:
        assert closure is None, "optimizers that use closures are not supported"
        if self.manager.should_commit():
            self.optim.step()

    @property
    def param_groups(self) -> List[Dict[str, Any]]:  # type: ignore[override]
        return self.optim.param_groups

    @property
    def state(self) -> Mapping[torch.Tensor, Any]:  # type: ignore[override]
        return self.optim.state
