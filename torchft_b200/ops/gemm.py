"""bf16 GEMM on the 5th-generation tensor cores.

Two kernels with one contract: ``csrc/kernels/gemm_tcgen05_2cta.cu`` computes 256 x 256 tiles on
pairs of CTAs (``tcgen05.mma.cta_group::2``) and ``csrc/kernels/gemm_tcgen05.cu`` computes
128 x 256 tiles on single CTAs.  ``TFT_GEMM=single`` or ``TFT_GEMM=pair`` in the environment picks
one for the whole process; ``impl=`` picks one per call.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib

DEFAULT_IMPL = os.environ.get("TFT_GEMM", "pair")
assert DEFAULT_IMPL in ("single", "pair"), f"TFT_GEMM must be 'single' or 'pair', not {DEFAULT_IMPL!r}"


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    out: Optional[torch.Tensor] = None,
    *,
    a_kmajor: bool = True,
    b_kmajor: bool = True,
    accumulate: bool = False,
    out_dtype: torch.dtype = torch.bfloat16,
    status: Optional[torch.Tensor] = None,
    impl: Optional[str] = None,
) -> torch.Tensor:
    """``out (+)= op(a) @ op(b)`` with fp32 accumulation.

    ``a_kmajor``: ``a`` is stored ``[M, K]``; otherwise ``[K, M]`` (used as ``a.T``).
    ``b_kmajor``: ``b`` is stored ``[N, K]`` (used as ``b.T``, the ``nn.Linear`` weight
    layout); otherwise ``[K, N]``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_kmajor:
        M, K = a.shape
    else:
        K, M = a.shape
    if b_kmajor:
        N, Kb = b.shape
    else:
        Kb, N = b.shape
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if status is None:
        status = _lib.status_word(a.device)
    fn = _lib.lib().tft_gemm2_bf16 if (impl or DEFAULT_IMPL) == "pair" else _lib.lib().tft_gemm_bf16
    code = fn(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        0 if a_kmajor else 1, 0 if b_kmajor else 1, 1 if out.dtype == torch.float32 else 0,
        1 if accumulate else 0, _lib.ptr(status), _lib.stream_ptr(),
    )
    _lib.check(code, "tft_gemm_bf16")
    _lib.count_launch()
    return out
