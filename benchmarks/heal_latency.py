"""Fault-injection benchmark: live-recovery (heal) latency, lost steps and steady throughput.

    python benchmarks/heal_latency.py --transport nvlink --model llama_1b --steps 600 --kill-at 40
    python benchmarks/heal_latency.py --transport http   --model llama_1b --steps 600 --kill-at 40
    python benchmarks/heal_latency.py --transport nvlink --model llama_1b --steps 1000 --kill-at 200 --kills 4

Two replica groups of one GPU each train a Llama-shape model under per-step quorum.  After
``--kill-at`` committed steps replica 1 leaves (its process exits between two steps, with
nothing in flight) and the parent starts a fresh process in its place.  The newcomer joins
the quorum, pulls parameters and AdamW state from the survivor and resumes.  Reported:

* ``heal_s``: time the newcomer spent fetching the checkpoint (metadata + transfer),
  ``heal_bytes`` and the resulting GB/s;
* ``rejoin_s``: from the newcomer's ``Manager`` being up to its first committed step;
* on the survivor: steps that did not commit and the median step time before / after.

With ``--kills N`` the replica leaves N times, every ``--kill-at`` steps, and each newcomer heals from
the survivor; the summary then carries the median and the worst heal and rejoin times.

``--transport http`` uses the serialising HTTP transport (the reference's method,
``torchft/checkpointing.py``), ``nvlink`` the peer-memory transport.  The failure is injected
on the host; no GPU is faulted or hung.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from datetime import timedelta

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def worker(args: argparse.Namespace) -> None:
    import torch
    from torch.distributed import TCPStore

    from torchft_b200 import _control
    from torchft_b200.checkpointing import CheckpointServer
    from torchft_b200.manager import Manager
    from torchft_b200.models.llama import Llama, LlamaConfig
    from torchft_b200.ops._lib import KernelError
    from torchft_b200.parallel.hsdp import HSDPEngine
    from torchft_b200.parallel.nvlink import ProcessGroupNVLink, SymmetricHeap
    from torchft_b200.parallel.nvlink_heal import NVLinkCheckpointTransport
    from torchft_b200.utils import tracing

    _control.set_log_enabled(False)
    torch.cuda.set_device(args.rank)
    cfg = {"llama3_8b": LlamaConfig.llama3_8b, "llama_1b": LlamaConfig.llama_1b, "tiny": LlamaConfig.tiny}[args.model]()
    seq = args.seq or cfg.max_seq_len
    n = cfg.num_params() + 64 * 1024 * (cfg.n_layers + 2)
    heap_bytes = 2 * 2 * n + 2 * 4 * (n + 1024) + (1 << 30)
    for attempt in range(60):
        # The memory of the process this one replaces is released once the survivors have moved to
        # a membership without it (they unmap its heap then); until that quorum, allocation can fail.
        try:
            heap = SymmetricHeap.get(heap_bytes)
            break
        except KernelError:
            if not args.restarted or attempt == 59:
                raise
            time.sleep(0.5)
    group_store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    model = Llama(cfg, device="cuda")
    model.init_weights(seed=7 + args.rank + (100 if args.restarted else 0))
    timeout = timedelta(seconds=args.timeout)
    if args.transport == "nvlink":
        transport = NVLinkCheckpointTransport(heap, timeout=timeout)
    else:
        transport = CheckpointServer(timeout=timeout)
    box = {}
    t_up = time.perf_counter()
    manager = Manager(
        pg=ProcessGroupNVLink(timeout=timedelta(seconds=args.device_timeout), heap=heap, staging_bytes=16 << 20),
        load_state_dict=lambda sd: box["e"].load_state_dict(sd),
        state_dict=lambda: box["e"].state_dict(),
        min_replica_size=1,
        timeout=timeout,
        quorum_timeout=timeout,
        rank=0,
        world_size=1,
        store_addr="127.0.0.1",
        store_port=group_store.port,
        lighthouse_addr=args.lighthouse,
        replica_id=f"heal_{args.rank}_",
        hostname="127.0.0.1",
        checkpoint_transport=transport,
    )
    engine = HSDPEngine(model, model.units(), manager=manager, alloc=heap.alloc)
    box["e"] = engine
    gen = torch.Generator().manual_seed(args.rank)
    tokens = torch.randint(cfg.vocab_size, (1, seq), generator=gen).cuda()
    targets = torch.randint(cfg.vocab_size, (1, seq), generator=gen).cuda()

    step_times, uncommitted, first_commit_s = [], 0, None
    while manager.current_step() < args.steps:
        before = manager.current_step()
        t0 = time.perf_counter()
        loss = engine.train_step(tokens, targets)
        loss.item()
        dt = time.perf_counter() - t0
        committed = manager.current_step() > before
        step_times.append((manager.current_step(), dt, manager.num_participants(), committed))
        if committed and first_commit_s is None:
            first_commit_s = time.perf_counter() - t_up
        if not committed:
            uncommitted += 1
        if args.rank == 1 and args.kill_at > 0 and manager.current_step() >= args.kill_at:
            # leave between steps: nothing of ours is in flight on the GPU
            torch.cuda.synchronize()
            heal = tracing.summary().get("tft.heal_recv", {"calls": 0, "total_s": 0.0})
            print(json.dumps({"event": "replica_left", "step": manager.current_step(), "restarted": args.restarted,
                              "heal_calls": heal["calls"], "heal_s": round(heal["total_s"], 4),
                              "rejoin_s": round(first_commit_s, 3) if first_commit_s is not None else None}), flush=True)
            os._exit(0)
    torch.cuda.synchronize()
    heal = tracing.summary().get("tft.heal_recv", {"calls": 0, "total_s": 0.0})
    state_bytes = sum(t.numel() * t.element_size() for t in (engine.flat_param, engine.exp_avg, engine.exp_avg_sq))
    alone = [dt for _, dt, n, c in step_times if n == 1 and c]
    together = [dt for _, dt, n, c in step_times if n == 2 and c]
    print(json.dumps({
        "event": "result", "rank": args.rank, "restarted": args.restarted, "transport": args.transport,
        "model": args.model, "heal_calls": heal["calls"], "heal_s": round(heal["total_s"], 4),
        "heal_bytes": state_bytes if heal["calls"] else 0,
        "heal_GBps": round(state_bytes / heal["total_s"] / 1e9, 2) if heal["calls"] and heal["total_s"] > 0 else None,
        "rejoin_s": round(first_commit_s, 3) if first_commit_s is not None else None,
        "uncommitted_steps": uncommitted,
        "median_step_s_two_replicas": round(statistics.median(together), 4) if together else None,
        "median_step_s_alone": round(statistics.median(alone), 4) if alone else None,
        "tokens_per_s_two_replicas": round(2 * seq / statistics.median(together), 1) if together else None,
        "final_step": manager.current_step(),
    }), flush=True)
    manager.shutdown(wait=False)


def parent(args: argparse.Namespace) -> None:
    from torchft_b200 import _control

    _control.set_log_enabled(False)
    lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=args.join_timeout_ms, quorum_tick_ms=10,
                                     heartbeat_timeout_ms=args.heartbeat_timeout_ms)
    base = [sys.executable, os.path.abspath(__file__), "--worker", "--lighthouse", lighthouse.address(), "--transport",
            args.transport, "--model", args.model, "--steps", str(args.steps), "--kill-at", str(args.kill_at),
            "--timeout", str(args.timeout), "--device-timeout", str(args.device_timeout), "--seq", str(args.seq)]

    def start(rank: int, kill_at: int, restarted: bool) -> subprocess.Popen:
        cmd = [a for a in base]
        cmd[cmd.index("--kill-at") + 1] = str(kill_at)
        cmd += ["--rank", str(rank)] + (["--restarted"] if restarted else [])
        return subprocess.Popen(cmd, stdout=subprocess.PIPE, text=True)

    results = []

    def collect(out: str) -> None:
        for line in out.strip().splitlines():
            if line.startswith("{"):
                results.append(json.loads(line))
                print(line)

    survivor = start(0, 0, False)
    replica = start(1, args.kill_at, False)
    for k in range(args.kills):
        out, _ = replica.communicate(timeout=1800)
        collect(out)
        # a supervisor (torchrun, a scheduler) would restart the group; do the same
        next_kill = args.kill_at * (k + 2) if k + 1 < args.kills else 0
        replica = start(1, next_kill, True)
    for proc in (replica, survivor):
        out, _ = proc.communicate(timeout=3600)
        collect(out)
    lighthouse.shutdown()
    heals = [x for x in results if x.get("restarted") and x.get("heal_calls")]
    survivor_result = next((x for x in results if x.get("event") == "result" and x.get("rank") == 0), None)
    last = next((x for x in results if x.get("event") == "result" and x.get("restarted")), None)
    if heals and survivor_result:
        heal_s = [x["heal_s"] for x in heals]
        rejoin_s = [x["rejoin_s"] for x in heals if x.get("rejoin_s") is not None]
        print(json.dumps({
            "summary": "heal", "transport": args.transport, "model": args.model, "kills": args.kills,
            "heal_s": round(statistics.median(heal_s), 4), "heal_s_max": max(heal_s),
            "heal_GBps": last["heal_GBps"] if last else None, "heal_bytes": last["heal_bytes"] if last else None,
            "rejoin_s": round(statistics.median(rejoin_s), 3) if rejoin_s else None,
            "rejoin_s_max": max(rejoin_s) if rejoin_s else None,
            "survivor_uncommitted_steps": survivor_result["uncommitted_steps"],
            "tokens_per_s_two_replicas": survivor_result["tokens_per_s_two_replicas"],
        }))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--worker", action="store_true")
    ap.add_argument("--restarted", action="store_true")
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--lighthouse", default="")
    ap.add_argument("--transport", default="nvlink", choices=["nvlink", "http"])
    ap.add_argument("--model", default="llama_1b", choices=["llama3_8b", "llama_1b", "tiny"])
    ap.add_argument("--seq", type=int, default=0, help="tokens per step and replica (0: the model's maximum)")
    ap.add_argument("--steps", type=int, default=600)
    ap.add_argument("--kill-at", type=int, default=40, help="replica 1 leaves after this many committed steps (0: never)")
    ap.add_argument("--kills", type=int, default=1, help="how many times the replica leaves (every --kill-at steps)")
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("--device-timeout", type=float, default=30.0)
    ap.add_argument("--join-timeout-ms", type=int, default=200)
    ap.add_argument("--heartbeat-timeout-ms", type=int, default=1000)
    args = ap.parse_args()
    if args.worker:
        worker(args)
    else:
        parent(args)


if __name__ == "__main__":
    main()
