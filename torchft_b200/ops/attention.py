"""Causal grouped-query flash attention on tcgen05 tensor cores
(``csrc/kernels/attention_fwd_pair.cu``, ``attention_fwd.cu`` and ``attention_bwd.cu``).

Two forward kernels with one contract: ``pair`` runs two query tiles per CTA in ping-pong, keeps P in
tensor memory and accumulates the output there; ``single`` runs one tile per CTA with P through shared
memory.  ``TFT_ATTN_FWD`` in the environment picks one for the process, ``impl=`` per call.
"""

from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import _lib


def _token_stride(t: torch.Tensor) -> int:
    # [B, S, H, D] view, possibly into a wider fused row
    assert t.stride(-1) == 1 and t.stride(-2) == t.shape[-1], "heads must be packed inside a token row"
    assert t.stride(0) == t.stride(1) * t.shape[1], "batch must be contiguous over the sequence"
    return t.stride(1)


FWD_IMPL = os.environ.get("TFT_ATTN_FWD", "pair")
assert FWD_IMPL in ("single", "pair"), f"TFT_ATTN_FWD must be 'single' or 'pair', not {FWD_IMPL!r}"


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                  impl: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q [B,S,Hq,D]``, ``k/v [B,S,Hkv,D]`` (bf16) -> ``(o [B,S,Hq,D], lse [B,Hq,S])``."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    o = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    fn = _lib.lib().tft_attn_fwd_pair if (impl or FWD_IMPL) == "pair" else _lib.lib().tft_attn_fwd
    code = fn(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), B, S, Hq, Hkv, D,
        _token_stride(q), _token_stride(k), _token_stride(v), scale, _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr(),
    )
    _lib.check(code, "tft_attn_fwd")
    _lib.count_launch()
    return o, lse


BWD_IMPL = os.environ.get("TFT_ATTN_BWD", "split")
assert BWD_IMPL in ("smem", "tmem", "tmem-dq", "split"), f"TFT_ATTN_BWD must be 'smem', 'tmem', 'tmem-dq' or 'split', not {BWD_IMPL!r}"


def attention_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                  scale: Optional[float] = None,
                  out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                  impl: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients ``(dq, dk, dv)``; ``out`` may name preallocated (possibly strided) destinations.

    ``impl="smem"``: P and dS go through shared memory (``attention_bwd.cu``); ``"tmem"``: they stay in
    tensor memory as MMA operands (``attention_bwd_tmem.cu``); ``"tmem-dq"``: the dQ kernel of the latter behind
    the dK/dV kernel of the former; ``"split"``: the same with the dK/dV kernel whose S and dP products run as
    separate pipelines.  Default from ``TFT_ATTN_BWD``."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if out is None:
        dq = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device=q.device)
        dk = torch.empty(B, S, Hkv, D, dtype=torch.bfloat16, device=q.device)
        dv = torch.empty(B, S, Hkv, D, dtype=torch.bfloat16, device=q.device)
    else:
        dq, dk, dv = out
    delta = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    do = do if do.is_contiguous() else do.contiguous()
    status = _lib.ptr(_lib.status_word(q.device))
    common = (_lib.ptr(do), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(delta),
              _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), B, S, Hq, Hkv, D,
              _token_stride(q), _token_stride(k), _token_stride(v), _token_stride(dq), _token_stride(dk), _token_stride(dv),
              scale, status, _lib.stream_ptr())
    which = impl or BWD_IMPL
    if which == "tmem":
        _lib.check(_lib.lib().tft_attn_bwd_tmem(*common, 7), "tft_attn_bwd_tmem")
    elif which in ("tmem-dq", "split"):  # dQ from tensor memory behind a shared-memory dK/dV kernel
        # "split": the dK/dV kernel whose S and dP products run as separate pipelines
        _lib.check(_lib.lib().tft_attn_bwd_parts(*common, 11 if which == "split" else 3), "tft_attn_bwd_parts")
        _lib.check(_lib.lib().tft_attn_bwd_tmem(*common, 4), "tft_attn_bwd_tmem")
    else:
        _lib.check(_lib.lib().tft_attn_bwd(*common), "tft_attn_bwd")
    _lib.count_launch(3)
    return dq, dk, dv


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):  # type: ignore[override]
        o, lse = attention_fwd(q, k, v, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attention_bwd(do, q, k, v, o, lse, ctx.scale)
        return dq, dk, dv, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention with grouped KV heads; differentiable."""
    return _Attention.apply(q, k, v, scale)
