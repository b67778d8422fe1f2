"""Autograd-aware wrappers of the sm_100a kernels (bf16 activations, fp32 statistics).

Every function here runs the hand-written kernel from ``libtft_kernels.so``; there is no
PyTorch fallback.  The numerics tests compare each of them with a plain fp32 PyTorch
implementation of the same operation.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .gemm import gemm


def _check_bf16(*tensors: torch.Tensor) -> None:
    for t in tensors:
        assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous(), "expected contiguous CUDA bf16 tensors"


# ------------------------------------------------------------------ linear
class _Linear(torch.autograd.Function):
    """``y = x @ w.T`` with all three products on the tcgen05 GEMM.

    If the weight has a ``main_grad`` attribute (a preallocated bf16 buffer, for
    example a slice of a flat gradient bucket), the weight gradient is written or
    accumulated there directly and autograd sees ``None`` for it; the flag
    ``main_grad_initialized`` tells whether to overwrite or accumulate.

    If the weight carries ``gather_comm`` (an ``NVLinkCommunicator``) and ``gather_pending`` is
    set, the forward product runs through the all-gather fused GEMM, which also completes the
    local copy of the weight for the backward products.

    If the weight carries ``rs_comm`` (an ``NVLinkCommunicator``), its rows are sharded over that
    group and the weight-gradient product runs through the GEMM fused with the reduce-scatter:
    only this rank's rows of ``main_grad`` receive the gradient, already summed over the group.
    """

    @staticmethod
    def forward(ctx, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        comm = getattr(w, "gather_comm", None)
        if comm is not None and getattr(w, "gather_pending", False):
            # the weight is sharded by rows over the GPUs of the group and only this rank's rows are
            # current: ONE kernel pulls the peers' rows into place and multiplies as they arrive
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            y = comm.all_gather_linear(x2, w)
            w.gather_pending = False
        else:
            y = gemm(x2, w)
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        ctx.weight = w
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy: torch.Tensor):  # type: ignore[override]
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_kmajor=False).view(ctx.x_shape)  # dY [M,N] @ W [N,K]
        dw = None
        if ctx.needs_input_grad[1]:
            weight = ctx.weight
            main_grad = getattr(weight, "main_grad", None)
            rs_comm = getattr(weight, "rs_comm", None)
            if main_grad is not None and rs_comm is not None:
                # rows of the weight are sharded over the GPUs of the group: the GEMM's epilogue sends
                # every tile to its owner, and only this rank's rows of the summed gradient are written
                acc = bool(getattr(weight, "main_grad_initialized", False))
                rows = weight.shape[0] // rs_comm.world
                own = main_grad[rs_comm.rank * rows : (rs_comm.rank + 1) * rows]
                rs_comm.wgrad_reduce_scatter(dy2, x2, own, accumulate=acc)
                weight.main_grad_initialized = True
            elif main_grad is not None:
                acc = bool(getattr(weight, "main_grad_initialized", False))
                gemm(dy2, x2, main_grad, a_kmajor=False, b_kmajor=False, accumulate=acc)  # dY^T @ X
                weight.main_grad_initialized = True
            else:
                dw = gemm(dy2, x2, a_kmajor=False, b_kmajor=False)
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _Linear.apply(x, w)


# ------------------------------------------------------------------ RMSNorm
_scratch: dict = {}


def _norm_scratch(rows: int, dim: int, device: torch.device) -> torch.Tensor:
    parts = _lib.lib().tft_rmsnorm_bwd_parts(rows)
    # one buffer per stream: two streams may run this backward at the same time
    key = (device.index, parts * dim, _lib.stream_ptr())
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.empty(parts * dim, dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, res: Optional[torch.Tensor] = None):
    """Returns ``(y, h, rstd)``: ``h = x + res`` (``x`` itself without residual), ``y = rmsnorm(h) * w``."""
    dim = x.shape[-1]
    rows = x.numel() // dim
    y = torch.empty_like(x)
    h = torch.empty_like(x) if res is not None else x
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    code = _lib.lib().tft_rmsnorm_fwd(
        _lib.ptr(x), _lib.ptr(res), _lib.ptr(w), _lib.ptr(y), _lib.ptr(h if res is not None else None),
        _lib.ptr(rstd), rows, dim, eps, _lib.stream_ptr(),
    )
    _lib.check(code, "tft_rmsnorm_fwd")
    _lib.count_launch()
    return y, h, rstd


def rmsnorm_bwd(dy, h, w, rstd, dres: Optional[torch.Tensor], dw_out: Optional[torch.Tensor] = None, accumulate: bool = False):
    """Returns ``(dh, dw)``; ``dres`` is the gradient arriving on the residual path (added to ``dh``)."""
    dim = h.shape[-1]
    rows = h.numel() // dim
    dx = torch.empty_like(h)
    dw = dw_out if dw_out is not None else torch.empty_like(w)
    code = _lib.lib().tft_rmsnorm_bwd(
        _lib.ptr(dy), _lib.ptr(h), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(dw),
        _lib.ptr(_norm_scratch(rows, dim, h.device)), rows, dim, 1 if accumulate else 0, _lib.stream_ptr(),
    )
    _lib.check(code, "tft_rmsnorm_bwd")
    _lib.count_launch(2)
    return dx, dw


def _main_grad_target(weight: torch.Tensor):
    """``(buffer, accumulate)`` when the parameter carries a preallocated ``main_grad``."""
    main_grad = getattr(weight, "main_grad", None)
    if main_grad is None:
        return None, False
    acc = bool(getattr(weight, "main_grad_initialized", False))
    weight.main_grad_initialized = True
    return main_grad, acc


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):  # type: ignore[override]
        _check_bf16(x, w)
        y, _, rstd = rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        ctx.weight = w
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, w, rstd = ctx.saved_tensors
        dw_out, acc = _main_grad_target(ctx.weight)
        dx, dw = rmsnorm_bwd(dy.contiguous(), x, w, rstd, None, dw_out, acc)
        return dx, (None if dw_out is not None else dw), None


class _AddRMSNorm(torch.autograd.Function):
    """``h = x + res;  y = rmsnorm(h) * w``; returns ``(y, h)`` from one kernel."""

    @staticmethod
    def forward(ctx, x, res, w, eps):  # type: ignore[override]
        _check_bf16(x, res, w)
        y, h, rstd = rmsnorm_fwd(x, w, eps, res)
        ctx.save_for_backward(h, w, rstd)
        ctx.weight = w
        return y, h

    @staticmethod
    def backward(ctx, dy, dh):  # type: ignore[override]
        h, w, rstd = ctx.saved_tensors
        dres = dh.contiguous() if dh is not None else None
        dw_out, acc = _main_grad_target(ctx.weight)
        dx, dw = rmsnorm_bwd(dy.contiguous(), h, w, rstd, dres, dw_out, acc)
        return dx, dx, (None if dw_out is not None else dw), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return _RMSNorm.apply(x, w, eps)


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
    return _AddRMSNorm.apply(x, res, w, eps)


# ------------------------------------------------------------------ RoPE
def rope_table(max_pos: int, head_dim: int, theta: float, device: torch.device) -> torch.Tensor:
    """``[max_pos, head_dim/2, 2]`` fp32 table of (cos, sin)."""
    cs = torch.empty(max_pos, head_dim // 2, 2, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.check(_lib.lib().tft_rope_table(_lib.ptr(cs), max_pos, head_dim, theta, _lib.stream_ptr()), "tft_rope_table")
    _lib.count_launch()
    return cs


def rope_(x: torch.Tensor, cs: torch.Tensor, heads: int, head_dim: int, inverse: bool = False,
          positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotates ``x[..., heads*head_dim]`` (a view into a wider row is fine) in place.

    Without ``positions`` (int32, one per token) a 3-D input ``[B, S, ...]`` uses the
    position inside its sequence and a 2-D input the row index.
    """
    assert x.dtype == torch.bfloat16 and x.stride(-1) == 1
    tokens = x.numel() // (heads * head_dim)
    row_stride = x.stride(-2) if x.dim() >= 2 else heads * head_dim
    seq_len = x.shape[-2] if x.dim() >= 3 else 0
    code = _lib.lib().tft_rope(_lib.ptr(x), _lib.ptr(cs), _lib.ptr(positions), tokens, heads, head_dim, row_stride,
                               1 if inverse else 0, seq_len, _lib.stream_ptr())
    _lib.check(code, "tft_rope")
    _lib.count_launch()
    return x


# ------------------------------------------------------------------ SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):  # type: ignore[override]
        _check_bf16(gu)
        F = gu.shape[-1] // 2
        rows = gu.numel() // (2 * F)
        out = torch.empty(*gu.shape[:-1], F, dtype=gu.dtype, device=gu.device)
        _lib.check(_lib.lib().tft_swiglu_fwd(_lib.ptr(gu), _lib.ptr(out), rows, F, _lib.stream_ptr()), "tft_swiglu_fwd")
        _lib.count_launch()
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        (gu,) = ctx.saved_tensors
        F = gu.shape[-1] // 2
        rows = gu.numel() // (2 * F)
        dgu = torch.empty_like(gu)
        _lib.check(
            _lib.lib().tft_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dout.contiguous()), _lib.ptr(dgu), rows, F, _lib.stream_ptr()),
            "tft_swiglu_bwd",
        )
        _lib.count_launch()
        return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up[..., :F] = gate`` and ``gate_up[..., F:] = up``."""
    return _SwiGLU.apply(gate_up)


# ------------------------------------------------------------------ cross entropy
class _CrossEntropy(torch.autograd.Function):
    """Mean token cross entropy; the logits buffer is overwritten with its own gradient."""

    @staticmethod
    def forward(ctx, logits, targets, ignore_index):  # type: ignore[override]
        _check_bf16(logits)
        V = logits.shape[-1]
        rows = logits.numel() // V
        targets = targets.reshape(-1).to(torch.int64)
        n_valid = int(rows) if ignore_index is None else None
        if n_valid is None:
            n_valid_t = (targets != ignore_index).sum().clamp(min=1)
            scale = 1.0 / float(n_valid_t.item())
        else:
            scale = 1.0 / rows
        loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
        code = _lib.lib().tft_xent(_lib.ptr(logits), _lib.ptr(targets), _lib.ptr(loss_rows), rows, V, V, scale,
                                   -100 if ignore_index is None else ignore_index, _lib.stream_ptr())
        _lib.check(code, "tft_xent")
        _lib.count_launch()
        ctx.save_for_backward(logits)  # now holds d loss / d logits
        return loss_rows.sum() * scale

    @staticmethod
    def backward(ctx, dloss):  # type: ignore[override]
        (grad,) = ctx.saved_tensors
        # dloss is 1.0 in the usual loss.backward(); avoid a full pass in that case
        return grad, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: Optional[int] = None) -> torch.Tensor:
    """Mean cross entropy.  ``logits`` is consumed: after the call it holds the gradient
    (valid for ``loss.backward()`` with unit upstream gradient)."""
    return _CrossEntropy.apply(logits, targets, ignore_index)


# ------------------------------------------------------------------ embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, table):  # type: ignore[override]
        _check_bf16(table)
        tokens = tokens.to(torch.int64).contiguous()
        dim = table.shape[1]
        out = torch.empty(*tokens.shape, dim, dtype=table.dtype, device=table.device)
        _lib.check(
            _lib.lib().tft_embedding_fwd(_lib.ptr(tokens), _lib.ptr(table), _lib.ptr(out), tokens.numel(), dim, _lib.stream_ptr()),
            "tft_embedding_fwd",
        )
        _lib.count_launch()
        ctx.save_for_backward(tokens)
        ctx.table = table
        return out

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        (tokens,) = ctx.saved_tensors
        table = ctx.table
        dim = table.shape[1]
        main_grad = getattr(table, "main_grad", None)
        if main_grad is not None:
            if not getattr(table, "main_grad_initialized", False):
                main_grad.zero_()
            target, ret = main_grad, None
            table.main_grad_initialized = True
        else:
            target = torch.zeros_like(table)
            ret = target
        _lib.check(
            _lib.lib().tft_embedding_bwd(_lib.ptr(tokens), _lib.ptr(dout.contiguous()), _lib.ptr(target), tokens.numel(), dim,
                                         _lib.stream_ptr()),
            "tft_embedding_bwd",
        )
        _lib.count_launch()
        return None, ret


def embedding(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return _Embedding.apply(tokens, table)


# ------------------------------------------------------------------ AdamW
def adamw_step_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float,
                beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0) -> None:
    """One fused AdamW update of a flat bf16 parameter buffer with fp32 moments."""
    assert p.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and m.dtype == torch.float32 and v.dtype == torch.float32
    assert p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()
    n = p.numel()
    assert g.numel() == n and m.numel() == n and v.numel() == n
    code = _lib.lib().tft_adamw(_lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), n, lr, beta1, beta2, eps,
                                weight_decay, step, grad_scale, _lib.stream_ptr())
    _lib.check(code, "tft_adamw")
    _lib.count_launch()
