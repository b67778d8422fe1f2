"""ctypes loader for ``libtft_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`torchft_b200.utils.build`.  There is no silent
fallback: on a machine with a GPU a missing library raises, so a test can never pass
on an eager PyTorch path by accident.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from torchft_b200.utils import build as _build

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None

P, I, L, F = c_void_p, c_int, c_int64, c_float

# name -> argument types (return type is always int: a cudaError_t, 0 on success)
_PROTOTYPES = {
    "tft_gemm_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, I, P, P],
    "tft_gemm2_bf16": [P, P, P, I, I, I, I, I, I, I, I, I, I, P, P],
    "tft_rmsnorm_bwd_parts": [I],
    "tft_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "tft_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, P],
    "tft_rope_table": [P, I, I, F, P],
    "tft_rope": [P, P, P, I, I, I, I, I, I, P],
    "tft_swiglu_fwd": [P, P, L, I, P],
    "tft_swiglu_bwd": [P, P, P, L, I, P],
    "tft_xent": [P, P, P, I, I, I, F, L, P],
    "tft_embedding_fwd": [P, P, P, L, I, P],
    "tft_embedding_bwd": [P, P, P, L, I, P],
    "tft_adamw": [P, P, P, P, L, F, F, F, F, F, I, F, P],
    "tft_pseudograd": [P, P, L, I, P],
    "tft_nesterov_outer": [P, P, P, L, F, F, I, I, I, P],
    "tft_attn_fwd": [P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P],
    "tft_attn_fwd_pair": [P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P],
    "tft_attn_bwd": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "tft_attn_bwd_parts": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P, I],
    "tft_attn_dq_tmem": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P, P],
    "tft_attn_bwd_tmem": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P, I],
}


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
            handle = ctypes.CDLL(str(path))
            for name, argtypes in _PROTOTYPES.items():
                fn = getattr(handle, name, None)
                if fn is not None:
                    fn.argtypes = argtypes
                    fn.restype = c_int
            _lib = handle
    return _lib


def available() -> bool:
    return torch.cuda.is_available() and _build.kernels_lib_path().exists()


def stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what} failed with CUDA error code {code}")


# Number of kernels of this library launched by this process (bench.py reports how many
# of the framework's own kernels ran inside the timed region).
_launches = 0


def count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def launches() -> int:
    return _launches


_status: dict = {}


def status_word(device: Optional[torch.device] = None) -> torch.Tensor:
    """A per-device int32 that kernels set when a device-side wait gave up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    key = (dev.type, dev.index)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status[key]


def check_status(what: str = "kernel") -> None:
    """Synchronising check of the status word; raises if a kernel reported a time-out."""
    s = status_word()
    v = int(s.item())
    if v != 0:
        s.zero_()
        raise KernelError(f"{what}: device-side wait gave up (status {v})")
