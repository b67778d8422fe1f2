"""Runs the reference's own training path on the benchmark's metric and config.

What runs: the reference's ``torchft.Manager`` + ``torchft.DistributedDataParallel`` (bucketed
comm hook -> ``Manager.allreduce`` -> ``ProcessGroupNCCL`` allreduce + divide) +
``torchft.Optimizer`` around ``torch.optim.AdamW``, per-step quorum against a lighthouse, on a
plain PyTorch Llama-3-8B-shape model (``nn.Linear`` / cuBLAS, ``scaled_dot_product_attention``,
``F.rms_norm``, ``F.cross_entropy``).  None of this repository's kernels, models or engine is
on that path.  The control-plane extension is this repository's C++ build under the
reference's module name, because the Rust original cannot be built offline (see
``baseline/make_ref.py``).

Scope: replica groups of ONE GPU at every N (N replica groups, fault-tolerant DDP across them).
The reference's HSDP glue (``ft_init_device_mesh`` / ``ManagedDeviceMesh``) assigns ``self.mesh``
in its constructor, which torch 2.11 rejects (``DeviceMesh.mesh`` is a read-only property), so
the sharded layout cannot run unmodified; the reference's DDP path can, and Llama-3-8B with
replicated AdamW state (about 100 GB) fits one 180 GB GPU.  The JSON line names the layout.
"""

from __future__ import annotations

import json
import os
import socket
import sys
import time
from datetime import timedelta

HERE = os.path.dirname(os.path.abspath(__file__))


def _say(obj) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(obj), flush=True)


def run(args) -> None:
    """Runs the arm and keeps every rank's traceback: a failing rank prints it with its rank number
    before the launcher tears the other ranks down, so the cause of a non-zero exit is on record."""
    try:
        _run(args)
    except BaseException:
        import traceback

        sys.stderr.write(f"[reference arm] rank {os.environ.get('RANK', '0')} failed:\n{traceback.format_exc()}\n")
        sys.stderr.flush()
        raise


def _one_gpu_per_process() -> int:
    """Shows this process only its own GPU, as ``cuda:0``.

    This is how the reference is launched (its README starts every replica group with its own
    ``CUDA_VISIBLE_DEVICES``), and its recovery path depends on it: ``CheckpointServer`` sends
    ``torch.save`` of CUDA tensors and the receiver calls ``torch.load`` without ``map_location``
    (torchft/checkpointing.py:187-203), which rebuilds every tensor on the device index it was
    saved from.  With all GPUs visible, every healing replica therefore first materialises the whole
    state on the sender's GPU 0 and keeps it there until its first ``should_commit``; with seven
    healers that is 7 x 16 GB on the GPU that also holds replica 0's parameters, gradients and
    cached activation memory, and a healer runs out of memory.  Must run before CUDA is initialised.
    """
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    visible = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
    chosen = visible[local_rank] if visible else str(local_rank)
    os.environ["CUDA_VISIBLE_DEVICES"] = chosen
    return int(chosen) if chosen.isdigit() else local_rank


def _run(args) -> None:
    if args.gpus not in (1, 2, 4, 8):
        _say({"impl": "reference", "unavailable": f"unsupported GPU count {args.gpus}"})
        return
    physical_gpu = _one_gpu_per_process()  # index for nvidia-smi, which ignores the visible-device list
    # The reference advertises socket.gethostname() in URLs; inside a container that name may
    # not resolve, so make the lookup succeed without touching the reference's files.
    try:
        socket.getaddrinfo(socket.gethostname(), None)
    except OSError:
        socket.gethostname = lambda: "127.0.0.1"  # type: ignore[assignment]
    sys.path.insert(0, os.path.join(HERE, "_ref"))

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch import nn

    import torchft
    from torchft.torchft import Lighthouse

    sys.path.insert(0, os.path.dirname(HERE))
    from bench import ClockSampler  # clock sampling only

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    assert world == args.gpus
    assert torch.cuda.device_count() == 1, "CUDA was initialised before the visible-device list was narrowed"
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    if world > 1:
        # plumbing only (barriers, the lighthouse address, max over ranks); the data plane is the
        # reference's own ProcessGroupNCCL across the replica groups
        dist.init_process_group("gloo")

    def bcast(obj, src=0):
        if world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=src)
        return box[0]

    shapes = {
        "llama3_8b": dict(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn=14336, vocab=128256, seq=4096),
        "llama_1b": dict(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn=8192, vocab=128256, seq=2048),
        "tiny": dict(dim=256, n_layers=2, n_heads=2, n_kv_heads=1, ffn=512, vocab=1024, seq=256),
    }[args.model]
    seq = args.seq or shapes["seq"]
    hd = shapes["dim"] // shapes["n_heads"]

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            d, hq, hkv, f = shapes["dim"], shapes["n_heads"], shapes["n_kv_heads"], shapes["ffn"]
            self.attn_norm = nn.Parameter(torch.ones(d))
            self.ffn_norm = nn.Parameter(torch.ones(d))
            self.wq = nn.Linear(d, hq * hd, bias=False)
            self.wk = nn.Linear(d, hkv * hd, bias=False)
            self.wv = nn.Linear(d, hkv * hd, bias=False)
            self.wo = nn.Linear(hq * hd, d, bias=False)
            self.w1 = nn.Linear(d, f, bias=False)
            self.w3 = nn.Linear(d, f, bias=False)
            self.w2 = nn.Linear(f, d, bias=False)

        def forward(self, x, cos, sin):
            B, S, _ = x.shape
            h = F.rms_norm(x, (x.shape[-1],), self.attn_norm, 1e-5)
            q = self.wq(h).view(B, S, shapes["n_heads"], hd).transpose(1, 2)
            k = self.wk(h).view(B, S, shapes["n_kv_heads"], hd).transpose(1, 2)
            v = self.wv(h).view(B, S, shapes["n_kv_heads"], hd).transpose(1, 2)

            def rope(t):
                a, b = t[..., : hd // 2], t[..., hd // 2 :]
                return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

            a = F.scaled_dot_product_attention(rope(q), rope(k), v, is_causal=True, enable_gqa=True)
            x = x + self.wo(a.transpose(1, 2).reshape(B, S, -1))
            h = F.rms_norm(x, (x.shape[-1],), self.ffn_norm, 1e-5)
            return x + self.w2(F.silu(self.w1(h)) * self.w3(h))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(shapes["vocab"], shapes["dim"])
            self.layers = nn.ModuleList([Block() for _ in range(shapes["n_layers"])])
            self.norm = nn.Parameter(torch.ones(shapes["dim"]))
            self.out = nn.Linear(shapes["dim"], shapes["vocab"], bias=False)
            pos = torch.arange(seq, dtype=torch.float32)
            inv = 500000.0 ** (-torch.arange(hd // 2, dtype=torch.float32) / (hd // 2))
            ang = pos[:, None] * inv[None, :]
            self.register_buffer("cos", ang.cos().to(torch.bfloat16), persistent=False)
            self.register_buffer("sin", ang.sin().to(torch.bfloat16), persistent=False)

        def forward(self, tokens, targets):
            x = self.emb(tokens)
            for layer in self.layers:
                x = layer(x, self.cos, self.sin)
            logits = self.out(F.rms_norm(x, (x.shape[-1],), self.norm, 1e-5))
            return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1))

    torch.manual_seed(1234)
    with torch.device(device):
        model = Model().to(torch.bfloat16)
    for p in model.parameters():
        if p.dim() > 1:
            nn.init.normal_(p, std=0.02)

    lighthouse = None
    if rank == 0:
        lighthouse = Lighthouse(bind="[::]:0", min_replicas=world, join_timeout_ms=60000, quorum_tick_ms=10)
    lighthouse_addr = bcast(lighthouse.address() if lighthouse else None)
    store = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)

    optimizer_box = {}
    init_mode = getattr(args, "ref_init", "resume")
    # With "heal" the replicas that are not the primary fetch the whole state over HTTP at step 0, one
    # after the other under the server's lock (torchft/checkpointing.py:139-170): budget for world - 1
    # serial transfers of 16 GB each.
    budget = timedelta(seconds=300 if init_mode == "resume" else 1800)
    pg = torchft.process_group.ProcessGroupNCCL()
    manager = torchft.Manager(
        pg=pg,
        load_state_dict=lambda sd: (model.load_state_dict(sd["model"]), optimizer_box["o"].load_state_dict(sd["optim"])),
        state_dict=lambda: {"model": model.state_dict(), "optim": optimizer_box["o"].state_dict()},
        min_replica_size=world,
        timeout=budget,
        quorum_timeout=budget,
        connect_timeout=timedelta(seconds=120),
        rank=0,
        world_size=1,
        store_addr="127.0.0.1",
        store_port=store.port,
        lighthouse_addr=lighthouse_addr,
        replica_id=f"ref_{rank}_",
    )
    ddp = torchft.DistributedDataParallel(manager, model, gradient_as_bucket_view=True)
    inner = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    optimizer = torchft.Optimizer(manager, inner)
    optimizer_box["o"] = inner
    if init_mode == "resume":
        # Every replica group built the same weights from the same seed above, i.e. each has "loaded the
        # same checkpoint".  Restoring the manager's own state_dict with it, as the reference asks of
        # anyone who resumes from a periodic checkpoint (torchft/manager.py:83-84), puts all groups at
        # the same step > 0, so the first quorum finds nobody behind and no replica heals at step 0.
        manager.load_state_dict({"step": 1, "batches_committed": world})

    total = args.warmup + 2 * args.steps
    gen = torch.Generator().manual_seed(1000 + rank)
    host_tokens = torch.randint(shapes["vocab"], (total, 1, seq), generator=gen).pin_memory()
    host_targets = torch.randint(shapes["vocab"], (total, 1, seq), generator=gen).pin_memory()
    idx = [0]

    def one_step(read_loss):
        i = idx[0]
        idx[0] += 1
        tokens = host_tokens[i].to(device, non_blocking=True)
        targets = host_targets[i].to(device, non_blocking=True)
        optimizer.zero_grad()
        loss = ddp(tokens, targets)
        loss.backward()
        optimizer.step()
        return float(loss.item()) if read_loss else loss

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_step(True)
    sync_all()
    sampler = ClockSampler(physical_gpu)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    start.record()
    for _ in range(args.steps):
        one_step(False)
    end.record()
    sync_all()
    device_ms = start.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else {}
    sync_all()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        final_loss = one_step(True)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([device_ms, e2e_s], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        device_ms, e2e_s = float(t[0]), float(t[1])
    tokens_per_step = world * seq
    ms = device_ms / args.steps
    _say({
        "metric": "tokens_per_s_llama3_8b_hsdp_per_step_quorum" if args.model == "llama3_8b" else f"tokens_per_s_{args.model}",
        "value": round(tokens_per_step / (ms / 1e3), 1),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms, 3),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic uniform token ids, random-init weights (std 0.02)",
        "impl": "reference",
        "config": {
            "model": args.model,
            "global_batch": world,
            "seq_len": seq,
            "parallelism": f"torchft DDP {world}x1 (replica groups x 1 GPU), ProcessGroupNCCL; the reference's "
                           "HSDP mesh glue does not run on torch 2.11, so no sharding inside a group",
            "optimizer": "torch.optim.AdamW(fused=True), bf16 parameters and bf16 moments",
            "init": ("same seed on every replica group + Manager.load_state_dict(step=1): the reference's resume path, "
                     "no step-0 heal" if init_mode == "resume" else
                     "step-0 heal: every other replica group fetches the state from group 0 over the reference's HTTP transport"),
            "devices": "one visible GPU per process (CUDA_VISIBLE_DEVICES), as the reference's README launches it",
            "note": "reference Python sources unmodified; control-plane extension is a C++ stand-in for the "
                    "unbuildable Rust one; model is plain PyTorch (cuBLAS, SDPA)",
        },
        "clocks": clocks,
        "gpu_launches": 0,
        "committed_steps": manager.current_step(),
        "final_loss": round(final_loss, 4),
        "e2e": {"value": round(tokens_per_step * args.steps / e2e_s, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 2 * seq * 8, "d2h_bytes_per_step": 4},
    })
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
