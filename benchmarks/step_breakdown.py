"""Per-kernel device time of one Llama-3-8B training step on one GPU (torch profiler, CUDA activity only).

    python benchmarks/step_breakdown.py [--model llama3_8b] [--steps 2]

Runs the HSDP engine without a manager (no quorum), two warm-up steps, then profiles ``--steps`` steps and
prints the kernels sorted by total device time.  Kernels of different streams overlap, so the column
sums to more than the wall time of the step.
"""

from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
from torch.profiler import ProfilerActivity, profile


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "llama_1b", "tiny"])
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args()
    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.parallel.hsdp import HSDPEngine

    cfg = {"llama3_8b": LlamaConfig.llama3_8b, "llama_1b": LlamaConfig.llama_1b, "tiny": LlamaConfig.tiny}[args.model]()
    model = Llama(cfg, device="cuda")
    model.init_weights(0)
    engine = HSDPEngine(model, model.units())
    tokens = torch.randint(cfg.vocab_size, (1, cfg.max_seq_len), device="cuda")
    targets = torch.randint(cfg.vocab_size, (1, cfg.max_seq_len), device="cuda")
    for _ in range(2):
        engine.train_step(tokens, targets)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            engine.train_step(tokens, targets)
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=70))


if __name__ == "__main__":
    main()
