"""Llama model on the sm_100a kernels against a plain fp32 PyTorch implementation."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def reference_loss(model, tokens, targets):
    """The same architecture in fp32 eager PyTorch, differentiable w.r.t. cloned weights."""
    cfg = model.cfg
    P = {n: p.detach().float().requires_grad_() for n, p in model.named_parameters()}
    hd, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    B, S = tokens.shape

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w

    pos = torch.arange(S, device=tokens.device, dtype=torch.float32)
    inv = cfg.rope_theta ** (-torch.arange(hd // 2, device=tokens.device, dtype=torch.float32) / (hd // 2))
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(x):
        a, b = x[..., : hd // 2], x[..., hd // 2 :]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    h = P["tok_embeddings"][tokens]
    mask = torch.ones(S, S, device=tokens.device, dtype=torch.bool).tril()
    for i in range(cfg.n_layers):
        pre = f"layers.{i}."
        xn = norm(h, P[pre + "attn_norm"])
        qkv = xn @ P[pre + "wqkv"].t()
        q = rope(qkv[..., : Hq * hd].view(B, S, Hq, hd))
        k = rope(qkv[..., Hq * hd : (Hq + Hkv) * hd].view(B, S, Hkv, hd))
        v = qkv[..., (Hq + Hkv) * hd :].view(B, S, Hkv, hd)
        qh = q.permute(0, 2, 1, 3)
        kh = k.permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
        vh = v.permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
        s = (qh @ kh.transpose(-1, -2) / math.sqrt(hd)).masked_fill(~mask, float("-inf"))
        a = (s.softmax(-1) @ vh).permute(0, 2, 1, 3).reshape(B, S, Hq * hd)
        h = h + a @ P[pre + "wo"].t()
        xn2 = norm(h, P[pre + "ffn_norm"])
        gu = xn2 @ P[pre + "w13"].t()
        act = torch.nn.functional.silu(gu[..., : cfg.ffn_dim]) * gu[..., cfg.ffn_dim :]
        h = h + act @ P[pre + "w2"].t()
    logits = norm(h, P["norm"]) @ P["output"].t()
    loss = torch.nn.functional.cross_entropy(logits.view(-1, cfg.vocab_size), targets.reshape(-1))
    loss.backward()
    return loss.item(), {n: p.grad for n, p in P.items()}


def test_llama_loss_and_gradients_match_fp32_reference():
    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.ops import _lib

    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(init_std=0.05)
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=1)
    tokens = torch.randint(cfg.vocab_size, (2, 256), device="cuda")
    targets = torch.randint(cfg.vocab_size, (2, 256), device="cuda")
    ref_loss, ref_grads = reference_loss(model, tokens, targets)
    loss = model(tokens, targets)
    loss.backward()
    _lib.check_status("llama")
    assert abs(loss.item() - ref_loss) < 2e-2 * abs(ref_loss)
    for n, p in model.named_parameters():
        g, r = p.grad.float(), ref_grads[n]
        err = (g - r).norm() / (r.norm() + 1e-12)
        assert err < 5e-2, f"{n}: relative gradient error {err.item():.4f}"


def test_engine_trains_and_state_round_trips():
    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.parallel.hsdp import HSDPEngine

    cfg = LlamaConfig.tiny()
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=0)
    engine = HSDPEngine(model, model.units(), lr=1e-3)
    tokens = torch.randint(cfg.vocab_size, (2, 256), device="cuda")
    targets = torch.randint(cfg.vocab_size, (2, 256), device="cuda")
    losses = [float(engine.train_step(tokens, targets)) for _ in range(5)]
    assert losses[-1] < losses[0]
    for p in model.parameters():
        assert p.grad is None and p.data.untyped_storage().data_ptr() == engine.flat_param.untyped_storage().data_ptr()

    sd = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in engine.state_dict().items()}
    model2 = Llama(cfg, device="cuda")
    model2.init_weights(seed=5)
    engine2 = HSDPEngine(model2, model2.units(), lr=1e-3)
    engine2.load_state_dict(sd)
    a = float(engine.train_step(tokens, targets))
    b = float(engine2.train_step(tokens, targets))
    assert abs(a - b) < 1e-3 * abs(a)
    # the embedding gradient uses atomics, so the two runs agree to rounding, not bit for bit
    torch.testing.assert_close(engine.flat_param.float(), engine2.flat_param.float(), rtol=2e-2, atol=2e-3)


def test_forward_backward_is_cuda_graph_capturable():
    """The kernels make no call that is illegal during stream capture: a whole forward + backward
    of the model replays from a CUDA graph with the gradients of the eager run."""
    from torchft_b200.models.llama import Llama, LlamaConfig

    cfg = LlamaConfig.tiny()
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=2)
    gen = torch.Generator().manual_seed(0)
    tokens = torch.randint(cfg.vocab_size, (2, 128), generator=gen).cuda()
    targets = torch.randint(cfg.vocab_size, (2, 128), generator=gen).cuda()
    # everything on a side stream from the start: gradient accumulation nodes created on the
    # default stream would break the capture (a PyTorch rule, not one of these kernels)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            model.zero_grad(set_to_none=True)
            loss = model(tokens, targets)
            loss.backward()
        eager_loss = float(loss)
        eager_grads = [p.grad.detach().clone() for p in model.parameters()]
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    model.zero_grad(set_to_none=True)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_loss = model(tokens, targets)
        static_loss.backward()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    assert abs(float(static_loss) - eager_loss) < 1e-3
    for p, ref in zip(model.parameters(), eager_grads):
        # the embedding gradient is accumulated with atomics: compare with a tolerance
        torch.testing.assert_close(p.grad.float(), ref.float(), atol=2e-2, rtol=2e-2)
