"""torchft_b200: per-step fault-tolerant training, built for NVIDIA B200.

Public API (same names as ``torchft``): ``Manager``, ``Optimizer``,
``DistributedDataParallel``, ``DistributedSampler``, ``ProcessGroupGloo``,
``ProcessGroupBabyNCCL`` plus the B200-native ``ProcessGroupNVLink``.

Names are resolved on first use, so that ``torchft_b200.utils.build`` can be imported (and the
native parts built) in a fresh checkout where the compiled control plane does not exist yet.
"""

import importlib

_EXPORTS = {
    "DistributedSampler": ("torchft_b200.data", "DistributedSampler"),
    "DistributedDataParallel": ("torchft_b200.ddp", "DistributedDataParallel"),
    "Manager": ("torchft_b200.manager", "Manager"),
    "Optimizer": ("torchft_b200.optim", "OptimizerWrapper"),
    "FusedAdamW": ("torchft_b200.optim", "FusedAdamW"),
    "ProcessGroupBabyNCCL": ("torchft_b200.process_group", "ProcessGroupBabyNCCL"),
    "ProcessGroupGloo": ("torchft_b200.process_group", "ProcessGroupGloo"),
    # the NVLink backend pulls in the CUDA kernel library
    "ProcessGroupNVLink": ("torchft_b200.parallel.nvlink", "ProcessGroupNVLink"),
}

__all__ = tuple(sorted(k for k in _EXPORTS if k != "ProcessGroupNVLink"))


def __getattr__(name: str):
    target = _EXPORTS.get(name)
    if target is None:
        # submodules (torchft_b200._control, torchft_b200.manager, ...) still import the usual way
        try:
            return importlib.import_module(f"{__name__}.{name}")
        except ModuleNotFoundError:
            raise AttributeError(f"module 'torchft_b200' has no attribute {name!r}") from None
    value = getattr(importlib.import_module(target[0]), target[1])
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_EXPORTS))
