"""Llama-style decoder built on the sm_100a kernels of ``torchft_b200.ops``.

Every matrix product runs on the tcgen05 GEMM, attention on the tcgen05 flash-attention
kernels, and the normalisation / rotary / activation / loss / embedding work on the
fused bandwidth kernels.  Projections are stored fused (``wqkv``: q, k, v rows;
``w13``: gate rows then up rows) so each block issues four GEMMs forward.

The reference ships no transformer (its only model is the LeNet of ``train_ddp.py``);
this model exists because the benchmark configurations name Llama-3-8B and 1B shapes.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
from torch import nn

from torchft_b200.ops import functional as F
from torchft_b200.ops.attention import attention_bwd, attention_fwd


@dataclass
class LlamaConfig:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    vocab_size: int = 128256
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq_len: int = 4096
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @classmethod
    def llama3_8b(cls, **kw) -> "LlamaConfig":
        return cls(**kw)

    @classmethod
    def llama_1b(cls, **kw) -> "LlamaConfig":
        base = dict(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn_dim=8192, max_seq_len=2048)
        base.update(kw)
        return cls(**base)

    @classmethod
    def tiny(cls, **kw) -> "LlamaConfig":
        base = dict(dim=256, n_layers=2, n_heads=2, n_kv_heads=1, ffn_dim=512, vocab_size=1024, max_seq_len=256)
        base.update(kw)
        return cls(**base)

    def num_params(self) -> int:
        hd = self.head_dim
        per_layer = (self.n_heads + 2 * self.n_kv_heads) * hd * self.dim + self.dim * self.n_heads * hd
        per_layer += 3 * self.ffn_dim * self.dim + 2 * self.dim
        return self.n_layers * per_layer + 2 * self.vocab_size * self.dim + self.dim

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token: 6 x matmul parameters plus causal attention."""
        matmul_params = self.num_params() - self.vocab_size * self.dim - (2 * self.n_layers + 1) * self.dim
        attn = 6 * self.n_layers * self.n_heads * self.head_dim * seq_len  # 12 * L * d * S / 2 (causal)
        return 6.0 * matmul_params + attn


class _RopeAttention(torch.autograd.Function):
    """Rotary embedding + causal attention on a fused ``qkv`` activation.

    ``qkv`` (the output of the fused projection, ``[B, S, (Hq + 2 Hkv) * hd]``) is rotated
    in place and handed to the attention kernel as three strided views; the backward pass
    writes dq / dk / dv straight into one fused gradient buffer and un-rotates dq and dk
    in place, so no split, concatenation or transposition pass ever runs.
    """

    @staticmethod
    def forward(ctx, qkv, cs, n_heads, n_kv_heads, head_dim):  # type: ignore[override]
        B, S, _ = qkv.shape
        q, k, v = _split_qkv(qkv, n_heads, n_kv_heads, head_dim)
        F.rope_(qkv[..., : (n_heads + n_kv_heads) * head_dim], cs, n_heads + n_kv_heads, head_dim, positions=None)
        o, lse = attention_fwd(q, k, v)
        ctx.save_for_backward(qkv, o, lse, cs)
        ctx.dims = (n_heads, n_kv_heads, head_dim)
        return o.view(B, S, n_heads * head_dim)

    @staticmethod
    def backward(ctx, do):  # type: ignore[override]
        qkv, o, lse, cs = ctx.saved_tensors
        n_heads, n_kv_heads, head_dim = ctx.dims
        B, S, _ = qkv.shape
        q, k, v = _split_qkv(qkv, n_heads, n_kv_heads, head_dim)
        dqkv = torch.empty_like(qkv)
        outs = _split_qkv(dqkv, n_heads, n_kv_heads, head_dim)
        attention_bwd(do.reshape(B, S, n_heads, head_dim), q, k, v, o, lse, out=outs)
        F.rope_(dqkv[..., : (n_heads + n_kv_heads) * head_dim], cs, n_heads + n_kv_heads, head_dim, inverse=True)
        return dqkv, None, None, None, None


def _split_qkv(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, hd: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    B, S, _ = qkv.shape
    nq, nk = n_heads * hd, n_kv_heads * hd
    q = qkv[..., :nq].view(B, S, n_heads, hd)
    k = qkv[..., nq : nq + nk].view(B, S, n_kv_heads, hd)
    v = qkv[..., nq + nk :].view(B, S, n_kv_heads, hd)
    return q, k, v


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None) -> None:
        super().__init__()
        hd = cfg.head_dim
        kw = dict(dtype=torch.bfloat16, device=device)
        self.cfg = cfg
        self.attn_norm = nn.Parameter(torch.ones(cfg.dim, **kw))
        self.wqkv = nn.Parameter(torch.empty((cfg.n_heads + 2 * cfg.n_kv_heads) * hd, cfg.dim, **kw))
        self.wo = nn.Parameter(torch.empty(cfg.dim, cfg.n_heads * hd, **kw))
        self.ffn_norm = nn.Parameter(torch.ones(cfg.dim, **kw))
        self.w13 = nn.Parameter(torch.empty(2 * cfg.ffn_dim, cfg.dim, **kw))
        self.w2 = nn.Parameter(torch.empty(cfg.dim, cfg.ffn_dim, **kw))
        for w in (self.wqkv, self.wo, self.w13, self.w2):
            w.linear_weight = True  # used only through F.linear: eligible for the all-gather fused GEMM

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor], cs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Takes the previous block's MLP output ``x`` and residual stream; returns the same pair."""
        cfg = self.cfg
        if residual is None:
            h = x
            xn = F.rmsnorm(x, self.attn_norm, cfg.norm_eps)
        else:
            xn, h = F.add_rmsnorm(x, residual, self.attn_norm, cfg.norm_eps)
        qkv = F.linear(xn, self.wqkv)
        a = _RopeAttention.apply(qkv, cs, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
        a = F.linear(a, self.wo)
        xn2, h2 = F.add_rmsnorm(a, h, self.ffn_norm, cfg.norm_eps)
        gu = F.linear(xn2, self.w13)
        act = F.swiglu(gu)
        return F.linear(act, self.w2), h2


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None) -> None:
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=torch.bfloat16, device=device)
        self.tok_embeddings = nn.Parameter(torch.empty(cfg.vocab_size, cfg.dim, **kw))
        self.layers = nn.ModuleList([LlamaBlock(cfg, device=device) for _ in range(cfg.n_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.dim, **kw))
        self.output = nn.Parameter(torch.empty(cfg.vocab_size, cfg.dim, **kw))
        self._cs: Optional[torch.Tensor] = None
        # Called during backward with a unit name ("layer7", "head") as soon as all weight
        # gradients of that unit are final; an engine uses it to start communicating them
        # while the rest of the backward pass still runs.
        self.unit_grad_ready = None
        # Called in forward with a unit name right before the first kernel that reads that
        # unit's parameters; an engine that refreshes parameters on another stream makes the
        # current stream wait for the unit's refresh here.
        self.unit_pre_forward = None

    @torch.no_grad()
    def init_weights(self, seed: int = 0) -> None:
        gen = torch.Generator(device=self.tok_embeddings.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("norm"):
                p.fill_(1.0)
            else:
                # normal_ on bf16 directly; chunked so no fp32 temporary of a whole matrix lives
                p.normal_(mean=0.0, std=self.cfg.init_std, generator=gen)

    def rope_cache(self, device: torch.device) -> torch.Tensor:
        if self._cs is None or self._cs.device != device:
            self._cs = F.rope_table(self.cfg.max_seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._cs

    def units(self, per_weight: bool = False) -> List[Tuple[str, List[nn.Parameter]]]:
        """Parameters grouped the way they are sharded and communicated: the embedding, one
        group per block, and the head (final norm + output projection).

        With ``per_weight`` every projection matrix of a block is a unit of its own, named
        ``layer<i>/<weight>`` (the norms of the block share ``layer<i>/norms``); an engine that
        shards by unit then shards each matrix by rows, which is what the all-gather fused into
        the GEMM needs.  Callbacks keep using the block name ``layer<i>`` as a prefix.
        """
        groups: List[Tuple[str, List[nn.Parameter]]] = [("embed", [self.tok_embeddings])]
        for i, layer in enumerate(self.layers):
            if per_weight:
                for wname in ("wqkv", "wo", "w13", "w2"):
                    groups.append((f"layer{i}/{wname}", [getattr(layer, wname)]))
                groups.append((f"layer{i}/norms", [layer.attn_norm, layer.ffn_norm]))
            else:
                groups.append((f"layer{i}", list(layer.parameters())))
        groups.append(("head", [self.norm, self.output]))
        return groups

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``tokens [B, S]`` -> mean cross entropy against ``targets`` (or bf16 logits without targets)."""
        cs = self.rope_cache(tokens.device)
        pre = self.unit_pre_forward
        if pre is not None:
            pre("embed")
        x = F.embedding(tokens, self.tok_embeddings)
        residual = None
        hook = self.unit_grad_ready if torch.is_grad_enabled() else None
        for i, layer in enumerate(self.layers):
            if pre is not None:
                pre(f"layer{i}")
            if hook is not None and x.requires_grad:
                # the gradient w.r.t. a block's input is the last thing its backward produces,
                # so when it arrives every weight gradient of that block is complete
                x.register_hook(lambda g, name=f"layer{i}": hook(name))
            x, residual = layer(x, residual, cs)
        if hook is not None and x.requires_grad:
            x.register_hook(lambda g: hook("head"))
        if pre is not None:
            pre("head")
        xn, _ = F.add_rmsnorm(x, residual, self.norm, self.cfg.norm_eps)
        logits = F.linear(xn, self.output)
        if targets is None:
            return logits
        return F.cross_entropy(logits.view(-1, self.cfg.vocab_size), targets.reshape(-1))
