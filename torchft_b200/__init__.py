"""torchft_b200: per-step fault-tolerant training, built for NVIDIA B200.

Public API (same names as ``torchft``): ``Manager``, ``Optimizer``,
``DistributedDataParallel``, ``DistributedSampler``, ``ProcessGroupGloo``,
``ProcessGroupBabyNCCL`` plus the B200-native ``ProcessGroupNVLink``.
"""

from torchft_b200.data import DistributedSampler
from torchft_b200.ddp import DistributedDataParallel
from torchft_b200.manager import Manager
from torchft_b200.optim import OptimizerWrapper as Optimizer
from torchft_b200.process_group import ProcessGroupBabyNCCL, ProcessGroupGloo

__all__ = (
    "DistributedDataParallel",
    "DistributedSampler",
    "Manager",
    "Optimizer",
    "ProcessGroupBabyNCCL",
    "ProcessGroupGloo",
)


def __getattr__(name: str):
    # resolved on first use: the NVLink backend pulls in the CUDA kernel library
    if name == "ProcessGroupNVLink":
        from torchft_b200.parallel.nvlink import ProcessGroupNVLink

        return ProcessGroupNVLink
    raise AttributeError(f"module 'torchft_b200' has no attribute {name!r}")
