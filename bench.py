"""Headline benchmark: training throughput (tokens/s) of a Llama-3-8B-shape decoder under
per-step quorum, HSDP over the GPUs of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Topology: N = 1 -> 1 replica group x 1 GPU; N = 2 -> 2 x 1; N = 4 -> 2 x 2; N = 8 -> 2 x 4
(replica groups x shard GPUs).  Micro-batch 1 x seq 4096 per GPU (weak scaling), bf16
parameters and gradients, fp32 AdamW moments, synthetic uniform token ids, random-init
weights.  Every step runs the full protocol: lighthouse quorum, forward, backward,
gradient reduce-scatter inside the group, cross-replica allreduce through the Manager,
should_commit, fused AdamW, parameter all-gather.

Rank 0 prints one JSON line.  ``value`` is timed on the device with CUDA events (max over
ranks); ``e2e`` is a second measurement by wall clock through the public API that also
copies every step's inputs from pinned host memory and reads the loss back.

``--impl reference`` runs the reference's own code path instead (see ``baseline/``).
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import subprocess
import sys
import tempfile
import time
from datetime import timedelta

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOPOLOGY = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (2, 4)}


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "llama_1b", "tiny"])
    ap.add_argument("--seq", type=int, default=0, help="sequence length (default: the model's)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end phase")
    ap.add_argument("--topology", default="", help="override the layout, '<replica groups>x<shard GPUs>' (default: 1x1, 2x1, 2x2, 2x4)")
    ap.add_argument("--ddp", action="store_true",
                    help="the reference arm's layout through the stock interfaces: N replica groups of one GPU, torch "
                         "DistributedDataParallel (buckets in the symmetric heap) + OptimizerWrapper + FusedAdamW around "
                         "the same model, kernels and NVLink process group, instead of HSDPEngine")
    ap.add_argument("--fused-gather", action="store_true",
                    help="shard every projection matrix by rows and gather it inside its first GEMM of the step "
                         "(all-gather fused GEMM) instead of with separate all-gather kernels")
    ap.add_argument("--fused-rs", action="store_true",
                    help="shard every projection matrix by rows and reduce-scatter its gradient inside the "
                         "weight-gradient GEMM (no reduce-scatter kernel for those matrices)")
    ap.add_argument("--gather-engine", default="copy", choices=["sm", "copy", "copy-push"],
                    help="parameter all-gather inside a replica group: one SM kernel per unit, or the copy engines "
                         "(pull / push) between two barrier kernels")
    ap.add_argument("--reduce-engine", default="copy", choices=["sm", "copy"],
                    help="gradient reduce-scatter inside a replica group: one SM kernel per unit that loads over NVLink, "
                         "or copy-engine pulls into local staging plus a local sum kernel")
    ap.add_argument("--allreduce-engine", default="copy", choices=["sm", "copy"],
                    help="cross-replica gradient allreduce of buffers >= 8 MiB: the fused peer-load kernel, or the copy "
                         "engines plus a local sum kernel")
    ap.add_argument("--ref-init", default="resume", choices=["resume", "heal"],
                    help="reference arm only: 'resume' starts every replica group from the same seed and the same "
                         "manager step (no step-0 heal); 'heal' lets group 0 serve its state over HTTP at step 0")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(prefix="tft_clocks_", suffix=".csv")
            os.close(fd)
            out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)],
                stdout=out, stderr=subprocess.DEVNULL,
            )
        except Exception:  # noqa: BLE001 - sampling is best effort
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:  # noqa: BLE001
            pass
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class DDPArm:
    """Trains the model the way a user of the stock interfaces would: ``DistributedDataParallel(manager, model)``
    whose buckets go through ``Manager.allreduce``, ``OptimizerWrapper`` around ``FusedAdamW``.  Parameters,
    gradient buckets and moments are allocated under the heap's memory pool, so buckets are reduced in place and
    a joining replica receives its state straight into the live tensors.  Same ``train_step`` / ``state_dict``
    surface as ``HSDPEngine``."""

    def __init__(self, make_model, manager, heap, pool_bytes: int, lr: float, betas, eps: float, weight_decay: float,
                 bucket_cap_mb: int) -> None:
        from torchft_b200.ddp import DistributedDataParallel
        from torchft_b200.optim import FusedAdamW, OptimizerWrapper

        with heap.allocating(pool_bytes):
            self.model = make_model()
            self.ddp = DistributedDataParallel(manager, self.model, gradient_as_bucket_view=True, bucket_cap_mb=bucket_cap_mb)
            self.adamw = FusedAdamW(self.model.parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.optimizer = OptimizerWrapper(manager, self.adamw)
        self.timing = None

    def train_step(self, tokens, targets):
        self.optimizer.zero_grad()  # quorum for this step
        loss = self.ddp(tokens, targets)
        loss.backward()  # buckets are averaged over the replica groups as they fill
        self.optimizer.step()  # commit vote, then the update
        return loss.detach()

    def state_dict(self):
        return {"model": self.model.state_dict(), "optim": self.adamw.state_dict()}

    def load_state_dict(self, sd) -> None:
        import torch

        with torch.no_grad():
            mine = self.model.state_dict()
            for k, v in sd["model"].items():
                if mine[k].data_ptr() != v.data_ptr():
                    mine[k].copy_(v)
        self.adamw.load_state_dict(sd["optim"])


def run_ours(args: argparse.Namespace) -> None:
    import torch
    import torch.distributed as dist

    from torchft_b200 import _control
    from torchft_b200.manager import Manager
    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.ops import _lib
    from torchft_b200.parallel.hsdp import HSDPEngine
    from torchft_b200.parallel.nvlink import NVLinkCommunicator, NVLinkShardComm, ProcessGroupNVLink, SymmetricHeap
    from torchft_b200.parallel.nvlink_heal import NVLinkCheckpointTransport
    from torch.distributed import TCPStore

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    if args.gpus not in TOPOLOGY:
        raise SystemExit(f"--gpus must be one of {sorted(TOPOLOGY)}")
    n_groups, shard_world = TOPOLOGY[args.gpus]
    if args.topology:
        # experiments only: "<replica groups>x<shard GPUs>", e.g. 1x2 to study sharding without replication
        n_groups, shard_world = (int(v) for v in args.topology.lower().split("x"))
        if n_groups * shard_world != args.gpus:
            raise SystemExit(f"--topology {args.topology} does not multiply to --gpus {args.gpus}")
    if args.ddp:
        n_groups, shard_world = args.gpus, 1
    group, shard_rank = divmod(rank, shard_world)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _control.set_log_enabled(False)

    if world > 1:
        dist.init_process_group("nccl", device_id=device)  # plumbing only: barriers and the max over ranks

    def bcast(obj, src):
        if world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=src)
        return box[0]

    # ---- control plane: one lighthouse for the job, one store + manager server per replica group
    lighthouse = None
    if rank == 0:
        lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=n_groups, join_timeout_ms=60000, quorum_tick_ms=10)
    lighthouse_addr = bcast(lighthouse.address() if lighthouse else None, 0)
    group_store = None
    ports = [None] * n_groups
    if shard_rank == 0:
        group_store = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
    for g in range(n_groups):
        ports[g] = bcast(group_store.port if (group == g and shard_rank == 0) else None, g * shard_world)
    store_port = ports[group]

    cfg = {"llama3_8b": LlamaConfig.llama3_8b, "llama_1b": LlamaConfig.llama_1b, "tiny": LlamaConfig.tiny}[args.model]()
    seq = args.seq or cfg.max_seq_len
    cfg.max_seq_len = max(cfg.max_seq_len, seq)
    batch = 1

    # ---- memory: flat parameters and gradients live in the NVLink-visible heap
    n_params = cfg.num_params()
    padded = n_params + 64 * 1024 * (cfg.n_layers + 2)
    # bf16 parameters + bf16 gradients (full) and the fp32 AdamW moments of the owned slices
    heap_bytes = 2 * 2 * padded + 2 * 4 * (padded // shard_world + 1024) + (1 << 30)
    if args.ddp:
        heap_bytes += 4 << 30  # allocator granularity of ~300 separate tensors and the staging area
    heap = SymmetricHeap.get(heap_bytes, device)
    shard = NVLinkCommunicator(heap, timeout=timedelta(seconds=60))
    client_store = TCPStore("127.0.0.1", store_port, is_master=False, wait_for_workers=False)
    shard.bind(client_store, shard_rank, shard_world, "shard")  # fixed membership; renewed after a failed step

    def make_model():
        m = Llama(cfg, device=device)
        m.init_weights(seed=1234)  # identical on every rank, as after the step-0 heal
        return m

    model = None if args.ddp else make_model()
    pg = ProcessGroupNVLink(timeout=timedelta(seconds=60), heap=heap, staging_bytes=64 << 20,
                            copy_engine_min_bytes=(8 << 20) if args.allreduce_engine == "copy" else None)
    engine_box = {}
    manager = Manager(
        pg=pg,
        load_state_dict=lambda sd: engine_box["engine"].load_state_dict(sd),
        state_dict=lambda: engine_box["engine"].state_dict(),
        min_replica_size=n_groups,
        use_async_quorum=True,
        timeout=timedelta(seconds=120),
        quorum_timeout=timedelta(seconds=120),
        rank=shard_rank,
        world_size=shard_world,
        store_addr="127.0.0.1",
        store_port=store_port,
        lighthouse_addr=lighthouse_addr,
        replica_id=f"bench_{group}_",
        hostname="127.0.0.1",
        # step-0 weight sync and any later recovery move GPU to GPU over NVLink
        checkpoint_transport=NVLinkCheckpointTransport(heap, timeout=timedelta(seconds=120)),
    )
    fused = None
    if args.ddp:
        engine = DDPArm(make_model, manager, heap, pool_bytes=2 * 2 * padded + 2 * 4 * padded + (3 << 30), lr=3e-4,
                        betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, bucket_cap_mb=512)
        engine_box["engine"] = engine
    if args.fused_gather and shard_world > 1:
        fused = NVLinkCommunicator(heap, timeout=timedelta(seconds=60))
        fused.bind(client_store, shard_rank, shard_world, "fused")
    fused_rs = None
    if args.fused_rs and shard_world > 1:
        fused_rs = NVLinkCommunicator(heap, timeout=timedelta(seconds=60))
        fused_rs.bind(client_store, shard_rank, shard_world, "fused_rs")
    if not args.ddp:
        engine = HSDPEngine(
            model, model.units(per_weight=fused is not None or fused_rs is not None), fused_rs_comm=fused_rs, manager=manager, shard_comm=NVLinkShardComm(shard, gather_engine=args.gather_engine, reduce_engine=args.reduce_engine),
            lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, alloc=heap.alloc, fused_gather_comm=fused,
        )
        engine_box["engine"] = engine

    # ---- data: synthetic token ids in pinned host memory, a fresh batch every step
    total_steps = args.warmup + 2 * args.steps + 8  # a few spare batches for the optional timing pass
    gen = torch.Generator().manual_seed(1000 + rank)
    host_tokens = torch.randint(cfg.vocab_size, (total_steps, batch, seq), generator=gen).pin_memory()
    host_targets = torch.randint(cfg.vocab_size, (total_steps, batch, seq), generator=gen).pin_memory()
    h2d_bytes = 2 * batch * seq * 8
    step_idx = [0]

    def one_step(read_loss: bool):
        i = step_idx[0]
        step_idx[0] += 1
        tokens = host_tokens[i].to(device, non_blocking=True)
        targets = host_targets[i].to(device, non_blocking=True)
        loss = engine.train_step(tokens, targets)
        return float(loss.item()) if read_loss else loss

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_step(True)
    sync_all()

    # ---- phase A: device-timed
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launches()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    start.record()
    last = None
    for _ in range(args.steps):
        last = one_step(False)
    end.record()
    sync_all()
    device_ms = start.elapsed_time(end)
    launches = _lib.launches() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    final_loss = float(last.item())
    committed = manager.current_step()

    # ---- phase B: end to end by wall clock, inputs from pinned host memory, loss read back every step
    e2e_s = None
    if not args.no_e2e:
        sync_all()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            final_loss = one_step(True)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0

    if world > 1:
        t = torch.tensor([device_ms, e2e_s or 0.0], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        device_ms, e2e_max = float(t[0]), float(t[1])
        e2e_s = e2e_max if e2e_s is not None else None

    if os.environ.get("TFT_ENGINE_TIMING"):
        # optional diagnosis, after everything that is reported has been measured
        engine.timing = []
        for _ in range(5):
            one_step(True)
        if rank == 0:
            keys = sorted({k for row in engine.timing for k in row})
            print(json.dumps({"engine_timing_ms": {k: round(statistics.median(r.get(k, 0.0) for r in engine.timing), 3)
                                                   for k in keys}}), file=sys.stderr, flush=True)
        engine.timing = None
    _lib.check_status("bench")
    tokens_per_step = args.gpus * batch * seq
    ms_per_step = device_ms / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    if rank == 0:
        out = {
            "metric": "tokens_per_s_llama3_8b_hsdp_per_step_quorum" if args.model == "llama3_8b" else f"tokens_per_s_{args.model}",
            "value": round(value, 1),
            "unit": "tokens/s",
            "n_gpus": args.gpus,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 3),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights (std 0.02)",
            "impl": "ours",
            "config": {
                "model": {"llama3_8b": "Llama-3-8B shape (32L, d4096, 32/8 heads, ffn 14336, vocab 128256)",
                          "llama_1b": "Llama 1B shape (16L, d2048, 32/8 heads, ffn 8192, vocab 128256)",
                          "tiny": "tiny test model"}[args.model],
                "global_batch": args.gpus * batch,
                "seq_len": seq,
                "parallelism": (f"ddp{n_groups}x1 (torch DistributedDataParallel over replica groups of one GPU, 512 MiB buckets in the symmetric heap)"
                                if args.ddp else f"hsdp{n_groups}x{shard_world} (replica groups x shard GPUs)"),
                "optimizer": "fused AdamW lr 3e-4 betas (0.9, 0.95) wd 0.1, fp32 moments",
                "quorum": "lighthouse quorum + should_commit every step",
                "engine": "DistributedDataParallel + OptimizerWrapper + FusedAdamW" if args.ddp else "HSDPEngine",
                "parameter_gather": ("inside the first GEMM of each projection (all-gather fused GEMM)" if fused is not None
                                     else f"per-unit all-gather ({args.gather_engine}) overlapped with forward"),
                "gradient_reduce_scatter": ("inside the weight-gradient GEMM of every projection matrix" if fused_rs is not None
                                            else f"per unit after its backward ({args.reduce_engine})"),
                "cross_replica_allreduce": ("copy engines + local sum kernel for buffers >= 8 MiB" if args.allreduce_engine == "copy"
                                            else "fused peer-memory kernel (sum, 1/n, broadcast in one pass)"),
                "l2_policy": "no flush needed: weights, gradients and activations streamed per step exceed 100 GB (L2 is 126 MB)",
            },
            "clocks": clocks,
            "gpu_launches": launches,
            "model_tflops_per_gpu": round(cfg.flops_per_token(seq) * batch * seq / (ms_per_step / 1e3) / 1e12, 1),
            "committed_steps": committed,
            "final_loss": round(final_loss, 4),
        }
        if e2e_s is not None:
            out["e2e"] = {
                "value": round(tokens_per_step * args.steps / e2e_s, 1),
                "unit": "tokens/s",
                "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": 4,
            }
        print(json.dumps(out), flush=True)

    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        from baseline.reference_bench import run_reference

        run_reference(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
