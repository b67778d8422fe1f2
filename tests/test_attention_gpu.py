"""Flash-attention kernels (tcgen05) against an fp32 PyTorch reference."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def reference(q, k, v, do):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    qh = qf.permute(0, 2, 1, 3)
    kh = kf.permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    vh = vf.permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    s = qh @ kh.transpose(-1, -2) / math.sqrt(D)
    mask = torch.ones(S, S, device=q.device, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    o = (s.softmax(-1) @ vh).permute(0, 2, 1, 3)
    o.backward(do.float())
    return o.detach(), torch.logsumexp(s, -1).detach(), qf.grad, kf.grad, vf.grad


def rel(a, b):
    return ((a.float() - b).abs().max() / b.abs().max()).item()


def norm_rel(a, b):
    """Frobenius norm of the error over that of the reference (about 2e-3 for a correct bf16 result)."""
    return ((a.float() - b).norm() / b.norm()).item()


@pytest.mark.parametrize("shape", [(1, 128, 1, 1, 128), (2, 512, 4, 2, 128), (1, 384, 4, 1, 64), (1, 200, 2, 2, 128), (1, 1024, 8, 2, 128)])
def test_attention_fwd_bwd(shape):
    from torchft_b200.ops import _lib
    from torchft_b200.ops.attention import attention

    B, S, Hq, Hkv, D = shape
    torch.manual_seed(1)
    q, k, v = (torch.randn(B, S, h, D, device="cuda").to(torch.bfloat16).requires_grad_() for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
    o = attention(q, k, v)
    o.backward(do)
    ro, _, rq, rk, rv = reference(q.detach(), k.detach(), v.detach(), do)
    assert rel(o, ro) < 2e-2 and norm_rel(o, ro) < 6e-3
    assert rel(q.grad, rq) < 2e-2 and rel(k.grad, rk) < 2e-2 and rel(v.grad, rv) < 2e-2
    assert norm_rel(q.grad, rq) < 8e-3 and norm_rel(k.grad, rk) < 8e-3 and norm_rel(v.grad, rv) < 8e-3
    _lib.check_status("attention")


def test_attention_at_the_benchmark_shape():
    """One sequence of 4096 tokens, 32 query heads over 8 key/value heads, head dimension 128."""
    from torchft_b200.ops import _lib
    from torchft_b200.ops.attention import attention

    B, S, Hq, Hkv, D = 1, 4096, 32, 8, 128
    torch.manual_seed(2)
    q, k, v = (torch.randn(B, S, h, D, device="cuda").to(torch.bfloat16).requires_grad_() for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
    o = attention(q, k, v)
    o.backward(do)
    ro, _, rq, rk, rv = reference(q.detach(), k.detach(), v.detach(), do)
    assert rel(o, ro) < 2e-2 and norm_rel(o, ro) < 6e-3
    assert rel(q.grad, rq) < 2e-2 and rel(k.grad, rk) < 2e-2 and rel(v.grad, rv) < 2e-2
    assert norm_rel(q.grad, rq) < 8e-3 and norm_rel(k.grad, rk) < 8e-3 and norm_rel(v.grad, rv) < 8e-3
    _lib.check_status("attention")


@pytest.mark.parametrize("shape", [(1, 128, 1, 1, 128), (1, 256, 2, 1, 128), (2, 512, 4, 2, 128), (1, 384, 4, 1, 64),
                                   (1, 200, 2, 2, 128), (1, 1024, 8, 2, 128), (1, 4096, 8, 2, 128)])
def test_forward_kernels_agree_with_fp32(shape):
    """Both forward kernels (one tile per CTA; two tiles per CTA with P and O in tensor memory) against
    fp32 PyTorch: output and log-sum-exp.  Odd tile counts, a ragged last tile and head dimension 64 included."""
    from torchft_b200.ops import _lib
    from torchft_b200.ops.attention import attention_fwd

    B, S, Hq, Hkv, D = shape
    torch.manual_seed(3)
    q, k, v = (torch.randn(B, S, h, D, device="cuda").to(torch.bfloat16) for h in (Hq, Hkv, Hkv))
    # a few large scores make the running maximum jump late in a row (exercises the rescale of O)
    # (late keys: the last, masked tile; keys at a quarter of the sequence: a tile in the middle of the rows below)
    q[:, S // 2 :, :, 0] *= 8
    k[:, S - 64 :, :, 0] *= 8
    k[:, S // 4 : S // 4 + 32, :, 0] *= 8
    qf, kf, vf = q.float(), k.float(), v.float()
    qh = qf.permute(0, 2, 1, 3)
    kh = kf.permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    vh = vf.permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    s = qh @ kh.transpose(-1, -2) / math.sqrt(D)
    s = s.masked_fill(~torch.ones(S, S, device="cuda", dtype=torch.bool).tril(), float("-inf"))
    ro = (s.softmax(-1) @ vh).permute(0, 2, 1, 3)
    rl = torch.logsumexp(s, -1)
    for impl in ("single", "pair"):
        o, lse = attention_fwd(q, k, v, impl=impl)
        assert rel(o, ro) < 2e-2 and norm_rel(o, ro) < 6e-3, (impl, rel(o, ro), norm_rel(o, ro))
        assert (lse * math.log(2) - rl).abs().max().item() < 2e-3, impl
        _lib.check_status("attention")


@pytest.mark.parametrize("shape", [(1, 128, 1, 1, 128), (1, 256, 2, 1, 128), (2, 512, 4, 2, 128), (1, 384, 4, 1, 64),
                                   (1, 200, 2, 2, 128), (1, 1024, 8, 2, 128), (1, 4096, 8, 2, 128)])
def test_backward_kernels_agree_with_fp32(shape):
    """Both backward paths (P and dS through shared memory; through tensor memory) against fp32 autograd."""
    from torchft_b200.ops import _lib
    from torchft_b200.ops.attention import attention_bwd, attention_fwd

    B, S, Hq, Hkv, D = shape
    torch.manual_seed(4)
    q, k, v = (torch.randn(B, S, h, D, device="cuda").to(torch.bfloat16) for h in (Hq, Hkv, Hkv))
    do = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
    o, lse = attention_fwd(q, k, v)
    _, _, rq, rk, rv = reference(q, k, v, do)
    for impl in ("smem", "tmem-dq", "split", "tmem"):
        dq, dk, dv = attention_bwd(do, q, k, v, o, lse, impl=impl)
        for name, got, want in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
            assert rel(got, want) < 2e-2 and norm_rel(got, want) < 8e-3, (impl, name, rel(got, want), norm_rel(got, want))
        _lib.check_status("attention")


def test_attention_on_fused_qkv_views():
    from torchft_b200.ops.attention import attention_bwd, attention_fwd

    B, S, Hq, Hkv, D = 1, 512, 8, 2, 128
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    q = qkv[..., : Hq * D].view(B, S, Hq, D)
    k = qkv[..., Hq * D : (Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qkv[..., (Hq + Hkv) * D :].view(B, S, Hkv, D)
    do = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16)
    o, lse = attention_fwd(q, k, v)
    dqkv = torch.zeros_like(qkv)
    outs = (
        dqkv[..., : Hq * D].view(B, S, Hq, D),
        dqkv[..., Hq * D : (Hq + Hkv) * D].view(B, S, Hkv, D),
        dqkv[..., (Hq + Hkv) * D :].view(B, S, Hkv, D),
    )
    attention_bwd(do, q, k, v, o, lse, out=outs)
    ro, rl, rq, rk, rv = reference(q, k, v, do)
    assert rel(o, ro) < 2e-2
    assert (lse * math.log(2) - rl).abs().max().item() < 1e-3
    assert rel(outs[0], rq) < 2e-2 and rel(outs[1], rk) < 2e-2 and rel(outs[2], rv) < 2e-2
