"""ctypes loader for ``libtft_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`torchft_b200.utils.build`.  There is no silent
fallback: on a machine with a GPU a missing library raises, so a test can never pass
on an eager PyTorch path by accident.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from torchft_b200.utils import build as _build

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    """A kernel launch was rejected or a device-side wait gave up."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.kernels_lib_path()
            if not path.exists():
                raise KernelError(
                    f"{path} is missing: run `python -m torchft_b200.utils.build` (or __graft_entry__.build())"
                )
            _lib = ctypes.CDLL(str(path))
    return _lib


def available() -> bool:
    return torch.cuda.is_available() and _build.kernels_lib_path().exists()


def stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> ctypes.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what} failed with CUDA error code {code}")


# Number of kernels of this library launched by this process (used by bench.py to
# report how many of the framework's own kernels ran inside a timed region).
_launches = 0


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launches() -> int:
    return _launches
