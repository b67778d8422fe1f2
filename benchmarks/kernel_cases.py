"""Small, self-contained cases of the hot kernels, for timing and for Nsight Compute.

    python benchmarks/kernel_cases.py gemm            # 8192^3 bf16 GEMM, all three layouts
    python benchmarks/kernel_cases.py attention       # S=4096, 32/8 heads, hd 128: fwd + bwd
    python benchmarks/kernel_cases.py adamw           # 256 Mi parameters
    python benchmarks/kernel_cases.py norm            # RMSNorm fwd/bwd, [16384, 4096]
    python benchmarks/kernel_cases.py xent            # cross entropy, [4096, 128256]

Each case holds a few GB at most, uses inputs larger than the 126 MB L2 where bandwidth
matters, launches each kernel a handful of times and prints CUDA-event timings with the
achieved fraction of the measured peaks (``MEASURED_PEAKS.json`` if present).  Profile one
kernel of a case with, for example:

    ncu --set full --clock-control none -k regex:gemm2_kernel -s 2 -c 1 -o prof \
        python benchmarks/kernel_cases.py gemm
"""

import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
try:
    with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
        PEAKS.update(json.load(f))
        PEAKS["source"] = "measured"
except OSError:
    pass


def timeit(fn, iters=20, warmup=10):
    """Mean CUDA-event time of ``iters`` launches after ``warmup`` (enough of both for the clocks to have
    left their idle state: a handful of sub-millisecond launches is over before the GPU has ramped up)."""
    for _ in range(warmup):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def bf16(*shape):
    return torch.randn(*shape, device="cuda").to(torch.bfloat16)


def report(name, ms, flops=None, bytes_=None):
    out = {"kernel": name, "ms": round(ms, 4)}
    if flops:
        tf = flops / ms / 1e9
        out.update({"tflops": round(tf, 1), f"frac_of_{PEAKS['source']}_bf16_peak": round(tf / PEAKS["bf16_tflops"], 3)})
    if bytes_:
        gbs = bytes_ / ms / 1e6
        out.update({"GBps": round(gbs, 1), f"frac_of_{PEAKS['source']}_hbm_peak": round(gbs / PEAKS["hbm_gbs"], 3)})
    print(json.dumps(out), flush=True)


def case_gemm():
    from torchft_b200.ops.gemm import gemm

    M = N = K = 8192
    a, b, c = bf16(M, K), bf16(N, K), torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * M * N * K
    for impl, kernel in (("pair", "gemm2_kernel"), ("single", "gemm_kernel")):
        report(f"{kernel}<K-major A, K-major B> (forward)", timeit(lambda: gemm(a, b, c, impl=impl)), flops=fl)
        report(f"{kernel}<K-major A, MN-major B> (dgrad)", timeit(lambda: gemm(a, b, c, b_kmajor=False, impl=impl)), flops=fl)
        report(f"{kernel}<MN-major A, MN-major B> (wgrad)",
               timeit(lambda: gemm(a, b, c, a_kmajor=False, b_kmajor=False, impl=impl)), flops=fl)
    report("cublas bf16 (torch.matmul)", timeit(lambda: torch.matmul(a, b.t(), out=c)), flops=fl)


def case_attention():
    from torchft_b200.ops.attention import attention_bwd, attention_fwd

    B, S, Hq, Hkv, D = 1, 4096, 32, 8, 128
    q, k, v, do = bf16(B, S, Hq, D), bf16(B, S, Hkv, D), bf16(B, S, Hkv, D), bf16(B, S, Hq, D)
    o, lse = attention_fwd(q, k, v)
    fl = 4.0 * S * S * D * Hq / 2
    report("attn_fwd_kernel<128> (causal, one query tile per CTA)", timeit(lambda: attention_fwd(q, k, v, impl="single")), flops=fl)
    report("attn_fwd_pair_kernel<128> (causal, two query tiles per CTA)", timeit(lambda: attention_fwd(q, k, v, impl="pair")), flops=fl)
    report("attention backward (delta + dkdv + dq), P and dS through shared memory",
           timeit(lambda: attention_bwd(do, q, k, v, o, lse, impl="smem")), flops=2.5 * fl)
    report("attention backward, dQ kernel with dS in tensor memory, dK/dV through shared memory",
           timeit(lambda: attention_bwd(do, q, k, v, o, lse, impl="tmem-dq")), flops=2.5 * fl)
    report("attention backward, dQ kernel with dS in tensor memory, dK/dV with separate S and dP pipelines",
           timeit(lambda: attention_bwd(do, q, k, v, o, lse, impl="split")), flops=2.5 * fl)
    report("attention backward (delta + dkdv + dq), P and dS in tensor memory",
           timeit(lambda: attention_bwd(do, q, k, v, o, lse, impl="tmem")), flops=2.5 * fl)
    # The library kernel the reference arm of bench.py runs: F.scaled_dot_product_attention (whatever
    # backend torch picks on this GPU), same shapes, heads-first layout as it wants them.
    import torch.nn.functional as F

    qh, kh, vh = (t.transpose(1, 2).contiguous().requires_grad_() for t in (q, k, v))
    doh = do.transpose(1, 2).contiguous()
    sdpa = lambda: F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True)  # noqa: E731
    with torch.no_grad():
        report("F.scaled_dot_product_attention forward", timeit(sdpa), flops=fl)
    out = sdpa()
    report("F.scaled_dot_product_attention backward", timeit(lambda: torch.autograd.grad(out, (qh, kh, vh), doh, retain_graph=True)),
           flops=2.5 * fl)


def case_attention_default():
    """Only the default forward and backward kernels, a few launches each: the case for a profiler capture."""
    from torchft_b200.ops.attention import attention_bwd, attention_fwd

    B, S, Hq, Hkv, D = 1, 4096, 32, 8, 128
    q, k, v, do = bf16(B, S, Hq, D), bf16(B, S, Hkv, D), bf16(B, S, Hkv, D), bf16(B, S, Hq, D)
    fl = 4.0 * S * S * D * Hq / 2
    o, lse = attention_fwd(q, k, v)
    report("attention forward (default kernel)", timeit(lambda: attention_fwd(q, k, v), iters=3, warmup=2), flops=fl)
    report("attention backward (default kernels)", timeit(lambda: attention_bwd(do, q, k, v, o, lse), iters=3, warmup=2),
           flops=2.5 * fl)


def case_adamw():
    from torchft_b200.ops.functional import adamw_step_

    n = 256 << 20
    p, g = bf16(n), bf16(n)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    ms = timeit(lambda: adamw_step_(p, g, m, v, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3))
    report("adamw_kernel", ms, bytes_=n * (2 + 2 + 2 + 4 * 4))


def case_norm():
    from torchft_b200.ops.functional import rmsnorm_bwd, rmsnorm_fwd

    rows, dim = 16384, 4096
    x, r, w, dy = bf16(rows, dim), bf16(rows, dim), bf16(dim), bf16(rows, dim)
    _, h, rstd = rmsnorm_fwd(x, w, 1e-5, r)
    report("rmsnorm_fwd_kernel (+residual)", timeit(lambda: rmsnorm_fwd(x, w, 1e-5, r)), bytes_=rows * dim * 2 * 4)
    report("rmsnorm_bwd_kernel (+residual grad)", timeit(lambda: rmsnorm_bwd(dy, h, w, rstd, dy)), bytes_=rows * dim * 2 * 4)


def case_xent():
    from torchft_b200.ops import _lib

    rows, V = 4096, 128256
    logits = bf16(rows, V)
    targets = torch.randint(V, (rows,), device="cuda")
    loss = torch.empty(rows, device="cuda")

    def run():
        _lib.check(_lib.lib().tft_xent(logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), rows, V, V, 1.0 / rows, -100,
                                       _lib.stream_ptr()), "tft_xent")

    report("xent_kernel", timeit(run), bytes_=rows * V * 2 * 3)


if __name__ == "__main__":
    cases = {"gemm": case_gemm, "attention": case_attention, "attention_default": case_attention_default, "adamw": case_adamw, "norm": case_norm, "xent": case_xent}
    which = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    print(json.dumps({"peaks": PEAKS["source"], "hbm_gbs": PEAKS["hbm_gbs"], "bf16_tflops": PEAKS["bf16_tflops"]}))
    cases[which]()
