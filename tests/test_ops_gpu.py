"""Numerics of the sm_100a kernels against plain fp32 PyTorch references of the same ops."""


import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def bf16(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def rel_err(a, b):
    """Largest element error relative to the largest reference element (catches a single bad tile)."""
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


def norm_err(a, b):
    """Frobenius norm of the error over the Frobenius norm of the reference.  Rounding a correct
    fp32 result to bf16 gives about 2e-3 here; an element-wise bug in a few percent of the entries,
    which the max-based measure above lets through, does not."""
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("impl", ["single", "pair"])
@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, False), (False, True)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (384, 520, 328), (1024, 1024, 512), (2304, 19200, 192)])
def test_gemm_all_layouts(a_k, b_k, shape, impl):
    """(2304, 19200, 192): 9 x 75 tiles of 256 x 256 = 675 = 9 waves of 74 pairs + 9, so the pair
    kernel's split tail (halves of the last tiles) is exercised; 520 and 328 are ragged edges."""
    import functools

    from torchft_b200.ops import _lib
    from torchft_b200.ops.gemm import gemm as _gemm

    gemm = functools.partial(_gemm, impl=impl)

    M, N, K = shape
    a = bf16(M, K) if a_k else bf16(K, M)
    b = bf16(N, K) if b_k else bf16(K, N)
    A = a.float() if a_k else a.float().t()
    B = b.float().t() if b_k else b.float()
    ref = A @ B
    out = gemm(a, b, a_kmajor=a_k, b_kmajor=b_k)
    assert rel_err(out, ref) < 1e-2 and norm_err(out, ref) < 4e-3
    out32 = gemm(a, b, a_kmajor=a_k, b_kmajor=b_k, out_dtype=torch.float32)
    assert rel_err(out32, ref) < 1e-4 and norm_err(out32, ref) < 1e-5
    acc = bf16(M, N)
    ref2 = ref + acc.float()
    gemm(a, b, acc, a_kmajor=a_k, b_kmajor=b_k, accumulate=True)
    assert rel_err(acc, ref2) < 1e-2 and norm_err(acc, ref2) < 4e-3
    _lib.check_status("gemm")


# The products of one Llama-3-8B layer and of the head at the benchmark's 4096 tokens:
# (name, layout, M, N, K) with layout = (A is K-major, B is K-major).
LLAMA_GEMMS = [
    ("wqkv forward", (True, True), 4096, 6144, 4096),
    ("w13 forward", (True, True), 4096, 28672, 4096),
    ("w2 forward", (True, True), 4096, 4096, 14336),
    ("head forward", (True, True), 4096, 128256, 4096),
    ("w13 input gradient", (True, False), 4096, 4096, 28672),
    ("w13 weight gradient", (False, False), 28672, 4096, 4096),
    ("w2 weight gradient", (False, False), 4096, 14336, 4096),
]


@pytest.mark.parametrize("name,layout,M,N,K", LLAMA_GEMMS, ids=[g[0].replace(" ", "_") for g in LLAMA_GEMMS])
def test_gemm_at_benchmark_shapes(name, layout, M, N, K):
    from torchft_b200.ops import _lib
    from torchft_b200.ops.gemm import gemm

    a_k, b_k = layout
    torch.manual_seed(M + N + K)
    a = bf16(M, K, scale=0.5) if a_k else bf16(K, M, scale=0.5)
    b = bf16(N, K, scale=0.05) if b_k else bf16(K, N, scale=0.05)
    ref = (a.float() if a_k else a.float().t()) @ (b.float().t() if b_k else b.float())  # fp32, no TF32
    for impl in ("single", "pair"):
        out = gemm(a, b, a_kmajor=a_k, b_kmajor=b_k, impl=impl)
        assert rel_err(out, ref) < 1e-2 and norm_err(out, ref) < 4e-3, (name, impl)
        del out
    out32 = gemm(a, b, a_kmajor=a_k, b_kmajor=b_k, out_dtype=torch.float32, impl="pair")
    # fp32 output: what is left is the order of the fp32 summation over K (up to 28672 terms here)
    assert norm_err(out32, ref) < 1e-4, name
    _lib.check_status("gemm")


def test_linear_autograd_and_main_grad():
    from torchft_b200.ops.functional import linear

    x = bf16(4, 96, 256, scale=0.5).requires_grad_()
    w = bf16(512, 256, scale=0.05).requires_grad_()
    y = linear(x, w)
    dy = bf16(4, 96, 512)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = xf @ wf.t()
    yf.backward(dy.float())
    assert rel_err(y, yf) < 1e-2 and norm_err(y, yf) < 4e-3
    assert rel_err(x.grad, xf.grad) < 1e-2 and norm_err(x.grad, xf.grad) < 4e-3
    assert rel_err(w.grad, wf.grad) < 1e-2 and norm_err(w.grad, wf.grad) < 4e-3

    # gradient accumulation straight into a preallocated buffer
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.empty_like(w2)
    for _ in range(2):
        linear(x.detach(), w2).backward(dy)
    assert w2.grad is None
    assert rel_err(w2.main_grad, 2 * wf.grad) < 1e-2


@pytest.mark.parametrize("dim", [2048, 4096, 768])
def test_rmsnorm_fwd_bwd(dim):
    from torchft_b200.ops.functional import add_rmsnorm, rmsnorm

    rows = 300
    x = bf16(rows, dim).requires_grad_()
    w = (1 + 0.1 * torch.randn(dim, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = rmsnorm(x, w, 1e-5)
    dy = bf16(rows, dim)
    y.backward(dy)

    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    yf.backward(dy.float())
    assert rel_err(y, yf) < 1e-2 and norm_err(y, yf) < 4e-3
    assert rel_err(x.grad, xf.grad) < 2e-2 and norm_err(x.grad, xf.grad) < 5e-3
    assert rel_err(w.grad, wf.grad) < 2e-2 and norm_err(w.grad, wf.grad) < 5e-3

    # fused residual add
    a, r = bf16(rows, dim).requires_grad_(), bf16(rows, dim).requires_grad_()
    w2 = w.detach().clone().requires_grad_()
    y2, h2 = add_rmsnorm(a, r, w2, 1e-5)
    dh = bf16(rows, dim)
    (y2.float() * dy.float()).sum().add((h2.float() * dh.float()).sum()).backward()
    af, rf, w2f = a.detach().float().requires_grad_(), r.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    hf = (af + rf).to(torch.bfloat16).float() + 0 * (af + rf)  # forward value rounded like the kernel
    hf = (af + rf)
    yf2 = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * w2f
    ((yf2 * dy.float()).sum() + (hf * dh.float()).sum()).backward()
    assert rel_err(h2, hf) < 1e-2 and rel_err(y2, yf2) < 2e-2
    assert rel_err(a.grad, af.grad) < 2e-2 and torch.equal(a.grad, r.grad)
    assert rel_err(w2.grad, w2f.grad) < 2e-2


@pytest.mark.parametrize("hd", [64, 128])
def test_rope_matches_reference_and_inverts(hd):
    from torchft_b200.ops.functional import rope_, rope_table

    T, H = 200, 6
    theta = 500000.0
    cs = rope_table(256, hd, theta, torch.device(DEV))
    x = bf16(T, H * hd)
    ref = x.float().view(T, H, hd)
    pos = torch.arange(T, device=DEV, dtype=torch.float32)
    inv = theta ** (-torch.arange(hd // 2, device=DEV, dtype=torch.float32) / (hd // 2))
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = ref[..., : hd // 2], ref[..., hd // 2 :]
    expect = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).view(T, H * hd)
    y = x.clone()
    rope_(y, cs, H, hd)
    assert rel_err(y, expect) < 1e-2
    rope_(y, cs, H, hd, inverse=True)
    assert rel_err(y, x) < 2e-2
    # view into a wider fused buffer
    wide = bf16(T, 3 * H * hd)
    q = wide[:, : H * hd]
    keep = wide[:, H * hd :].clone()
    expect_q = wide[:, : H * hd].clone()
    rope_(expect_q.contiguous(), cs, H, hd)
    e2 = wide[:, : H * hd].contiguous()
    rope_(e2, cs, H, hd)
    rope_(q, cs, H, hd)
    assert torch.equal(wide[:, : H * hd], e2) and torch.equal(wide[:, H * hd :], keep)


def test_swiglu():
    from torchft_b200.ops.functional import swiglu

    gu = bf16(130, 2 * 1024).requires_grad_()
    out = swiglu(gu)
    d = bf16(130, 1024)
    out.backward(d)
    gf = gu.detach().float().requires_grad_()
    g, u = gf[:, :1024], gf[:, 1024:]
    of = torch.nn.functional.silu(g) * u
    of.backward(d.float())
    assert rel_err(out, of) < 1e-2 and norm_err(out, of) < 4e-3
    assert rel_err(gu.grad, gf.grad) < 2e-2 and norm_err(gu.grad, gf.grad) < 5e-3


@pytest.mark.parametrize("rows", [64, 4096])  # 4096 x 128256 is the benchmark's logits matrix
def test_cross_entropy_loss_and_grad(rows):
    from torchft_b200.ops.functional import cross_entropy

    V = 128256
    logits = bf16(rows, V, scale=2.0)
    targets = torch.randint(V, (rows,), device=DEV)
    lf = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lf, targets)
    ref.backward()
    work = logits.clone().requires_grad_()
    loss = cross_entropy(work, targets)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    assert (work.grad.float() - lf.grad).abs().max().item() < 2e-2 * lf.grad.abs().max().item() + 1e-6
    assert norm_err(work.grad, lf.grad) < 5e-3

    # ignore_index
    targets2 = targets.clone()
    targets2[::3] = -100
    lf2 = logits.float().requires_grad_()
    ref2 = torch.nn.functional.cross_entropy(lf2, targets2, ignore_index=-100)
    work2 = logits.clone().requires_grad_()
    loss2 = cross_entropy(work2, targets2, ignore_index=-100)
    assert abs(loss2.item() - ref2.item()) < 2e-3 * abs(ref2.item())


def test_embedding_fwd_bwd():
    from torchft_b200.ops.functional import embedding

    V, D = 1000, 256
    table = bf16(V, D).requires_grad_()
    tokens = torch.randint(V, (4, 50), device=DEV)
    tokens[0, :10] = 7  # repeated rows exercise the atomics
    out = embedding(tokens, table)
    assert torch.equal(out, table.detach()[tokens])
    d = bf16(4, 50, D)
    out.backward(d)
    ref = torch.zeros(V, D, device=DEV)
    ref.index_add_(0, tokens.reshape(-1), d.float().view(-1, D))
    assert rel_err(table.grad, ref) < 3e-2


def test_adamw_matches_torch():
    from torchft_b200.ops.functional import adamw_step_

    n = 8 * 1000 + 5
    p = bf16(n)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    ref_p = p.float().clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = bf16(n)
        ref_p.grad = g.float()
        opt.step()
        adamw_step_(p, g, m, v, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        # the kernel rounds the parameter to bf16 each step; keep the reference in lockstep
        assert (p.float() - ref_p.detach()).abs().max().item() < 1e-2 * ref_p.detach().abs().max().item()
        ref_p.data.copy_(p.float())
    st = opt.state[ref_p]
    assert rel_err(m, st["exp_avg"]) < 1e-4 and rel_err(v, st["exp_avg_sq"]) < 1e-4


def test_fused_adamw_optimizer_on_bf16_parameters():
    """``FusedAdamW`` (one kernel per bf16 parameter, fp32 moments) against ``torch.optim.AdamW`` on fp32 copies."""
    from torchft_b200.optim import FusedAdamW

    params = [torch.nn.Parameter(bf16(257, 33)), torch.nn.Parameter(bf16(1000))]
    refs = [torch.nn.Parameter(p.detach().float().clone()) for p in params]
    kw = dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ours, theirs = FusedAdamW(params, **kw), torch.optim.AdamW(refs, **kw)
    for _ in range(3):
        for p, q in zip(params, refs):
            g = bf16(*p.shape)
            p.grad, q.grad = g, g.float()
        ours.step()
        theirs.step()
        for p, q in zip(params, refs):
            assert (p.float() - q.detach()).abs().max().item() < 1e-2 * q.detach().abs().max().item()
            q.data.copy_(p.float())  # the kernel rounds the parameter to bf16 each step
    for p, q in zip(params, refs):
        assert ours.state[p]["exp_avg"].dtype == torch.float32
        assert rel_err(ours.state[p]["exp_avg"], theirs.state[q]["exp_avg"]) < 1e-4
        assert rel_err(ours.state[p]["exp_avg_sq"], theirs.state[q]["exp_avg_sq"]) < 1e-4


def test_diloco_fused_outer_step_matches_sgd():
    from torchft_b200.local_sgd import _FlatBuckets
    from torchft_b200.ops.outer_step import FusedOuterStep

    torch.manual_seed(0)
    params = [torch.nn.Parameter(bf16(33, 7)), torch.nn.Parameter(bf16(129))]
    ref_params = [torch.nn.Parameter(p.detach().float().clone()) for p in params]
    outer = torch.optim.SGD(params, lr=0.7, momentum=0.9, nesterov=True)
    ref_outer = torch.optim.SGD(ref_params, lr=0.7, momentum=0.9, nesterov=True)
    backup = _FlatBuckets(params, None, False)
    backup.copy_from_params()
    comm = _FlatBuckets(params, None, False)
    fused = FusedOuterStep.maybe_create(params, backup, comm, outer)
    assert fused is not None
    for _ in range(3):
        global_ref = [p.detach().clone() for p in ref_params]
        deltas = [torch.randn_like(p).mul(0.01).to(torch.bfloat16) for p in params]
        with torch.no_grad():
            for p, d in zip(params, deltas):
                p.add_(d)
        fused.compute_pseudogradients()
        fused.apply_outer_update()
        for rp, gp, p, d in zip(ref_params, global_ref, params, deltas):
            rp.data.copy_(gp)
            rp.grad = (p.detach().float() * 0 + d.float())
        ref_outer.step()
        for p, rp, i in zip(params, ref_params, range(2)):
            assert (p.detach().float() - rp.detach()).abs().max().item() < 3e-2 * rp.detach().abs().max().item()
            assert torch.equal(backup.views[i], p.detach())
            rp.data.copy_(p.detach().float())
            ref_outer.state[rp]["momentum_buffer"].copy_(outer.state[p]["momentum_buffer"])
