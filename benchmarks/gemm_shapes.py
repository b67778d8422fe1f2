"""bf16 GEMM table: the two tcgen05 kernels of this repository against cuBLAS (torch.matmul).

    python benchmarks/gemm_shapes.py [--iters 20] [--shapes square,wqkv,wo,w13,w2,head]

For the 8192^3 square case and for every projection of a Llama-3-8B layer at 4096 tokens, the three
products of a linear layer are timed -- forward ``X W^T``, input gradient ``dY W`` and weight
gradient ``dY^T X`` -- each with the single-CTA kernel (128 x 256 tiles), the CTA-pair kernel
(256 x 256 tiles, split tail) and cuBLAS.  Operands rotate through enough copies that consecutive
launches never find their inputs in the 126 MB L2, and the three candidates take turns in short
bursts so that all see the same clocks.  CUDA-event time per launch after warm-up; the
fraction is of the measured cuBLAS burst figure in ``MEASURED_PEAKS.json`` when that file exists.
One JSON line per (shape, product).
"""

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

PEAK = {"tflops": 1590.0, "source": "fallback"}
try:
    with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
        PEAK = {"tflops": float(json.load(f)["bf16_tflops"]), "source": "measured"}
except (OSError, KeyError, ValueError):
    pass

TOKENS = 4096
LAYERS = {  # name: (out features, in features)
    "wqkv": (6144, 4096),
    "wo": (4096, 4096),
    "w13": (28672, 4096),
    "w2": (4096, 14336),
    "head": (128256, 4096),
}


def time_interleaved(fns, sets, iters, rounds=5):
    """Mean time per launch of every ``fn`` in ``fns``.

    The candidates take turns in short bursts (``rounds`` bursts of ``iters / rounds`` launches each)
    instead of running one after the other: the GPU sits at its power limit during these kernels, and
    whoever ran last in a long sequence would be measured at the lowest clock.
    """
    for fn in fns:
        for s in sets:
            fn(*s)
    torch.cuda.synchronize()
    per_burst = max(1, iters // rounds)
    totals = [0.0] * len(fns)
    k = 0
    for _ in range(rounds):
        for i, fn in enumerate(fns):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(per_burst):
                fn(*sets[k % len(sets)])
                k += 1
            end.record()
            end.synchronize()
            totals[i] += start.elapsed_time(end)
    return [t / (rounds * per_burst) for t in totals]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--shapes", default="square,wqkv,wo,w13,w2,head")
    args = ap.parse_args()
    from torchft_b200.ops.gemm import gemm

    def bf16(*shape):
        return torch.randn(*shape, device="cuda").to(torch.bfloat16)

    for name in args.shapes.split(","):
        tokens, (n_out, n_in) = (8192, (8192, 8192)) if name == "square" else (TOKENS, LAYERS[name])
        per_set = 2 * (tokens * n_in + n_out * n_in + tokens * n_out)
        copies = max(2, -(-300_000_000 // per_set))  # > 2 x L2 in rotation
        xs = [bf16(tokens, n_in) for _ in range(copies)]
        ws = [bf16(n_out, n_in) for _ in range(copies)]
        dys = [bf16(tokens, n_out) for _ in range(copies)]
        y = torch.empty(tokens, n_out, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(tokens, n_in, device="cuda", dtype=torch.bfloat16)
        dw = torch.empty(n_out, n_in, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * tokens * n_out * n_in
        products = {
            "forward": (list(zip(xs, ws)),
                        lambda impl: (lambda x, w: gemm(x, w, y, impl=impl)),
                        lambda x, w: torch.matmul(x, w.t(), out=y), (tokens, n_out, n_in)),
            "input_gradient": (list(zip(dys, ws)),
                               lambda impl: (lambda d, w: gemm(d, w, dx, b_kmajor=False, impl=impl)),
                               lambda d, w: torch.matmul(d, w, out=dx), (tokens, n_in, n_out)),
            "weight_gradient": (list(zip(dys, xs)),
                                lambda impl: (lambda d, x: gemm(d, x, dw, a_kmajor=False, b_kmajor=False, impl=impl)),
                                lambda d, x: torch.matmul(d.t(), x, out=dw), (n_out, n_in, tokens)),
        }
        for product, (sets, ours, cublas, mnk) in products.items():
            row = {"shape": name, "product": product, "M": mnk[0], "N": mnk[1], "K": mnk[2]}
            labels = ("single_cta", "cta_pair", "cublas")
            times = time_interleaved([ours("single"), ours("pair"), cublas], sets, args.iters)
            for label, ms in zip(labels, times):
                tf = flops / ms / 1e9
                row[f"{label}_ms"] = round(ms, 4)
                row[f"{label}_tflops"] = round(tf, 1)
                row[f"{label}_frac_of_{PEAK['source']}_peak"] = round(tf / PEAK["tflops"], 3)
            row["pair_over_cublas"] = round(row["cublas_ms"] / row["cta_pair_ms"], 3)
            row["single_over_cublas"] = round(row["cublas_ms"] / row["single_cta_ms"], 3)
            print(json.dumps(row), flush=True)
        del xs, ws, dys, y, dx, dw
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
