"""Per-step cost of the control plane: quorum + should_commit round trips, no GPU involved.

    python benchmarks/control_plane_latency.py [--groups 2] [--ranks 1] [--steps 300] [--protocol framed|grpc|both]

One lighthouse, ``--groups`` manager servers, one client thread per (group, local rank); every
thread runs ``quorum`` then ``should_commit`` per step, as ``Manager.start_quorum`` /
``Manager.should_commit`` do.  Membership is stable after the first step, so the lighthouse
answers from its fast path (all members of the previous quorum are back) without waiting for a
tick.  Reported per protocol: median / p99 microseconds of the quorum call, of the commit call,
and of a whole step, taken on the slowest thread.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from datetime import timedelta

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run(protocol: str, groups: int, ranks: int, steps: int) -> dict:
    from torchft_b200 import _control as C

    C.set_log_enabled(False)
    C.set_rpc_protocol(protocol)
    lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=groups, join_timeout_ms=1000, quorum_tick_ms=100)
    managers = [
        C.Manager(replica_id=f"g{g}", lighthouse_addr=lighthouse.address(), hostname="127.0.0.1", bind="[::]:0",
                  store_addr=f"store{g}", world_size=ranks, heartbeat_interval=timedelta(milliseconds=100),
                  connect_timeout=timedelta(seconds=5))
        for g in range(groups)
    ]
    results = {}
    barrier = threading.Barrier(groups * ranks)

    def worker(g: int, r: int) -> None:
        client = C.ManagerClient(managers[g].address(), connect_timeout=timedelta(seconds=5))
        tq, tc, ts = [], [], []
        for step in range(steps + 5):
            barrier.wait()
            t0 = time.perf_counter()
            client.quorum(r, step, "meta", False, timeout=timedelta(seconds=30))
            t1 = time.perf_counter()
            client.should_commit(r, step, True, timeout=timedelta(seconds=30))
            t2 = time.perf_counter()
            if step >= 5:  # the first steps form the quorum and warm the connections
                tq.append((t1 - t0) * 1e6)
                tc.append((t2 - t1) * 1e6)
                ts.append((t2 - t0) * 1e6)
        results[(g, r)] = (tq, tc, ts)

    threads = [threading.Thread(target=worker, args=(g, r)) for g in range(groups) for r in range(ranks)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for m in managers:
        m.shutdown()
    lighthouse.shutdown()

    def stat(idx: int) -> dict:
        med = max(statistics.median(v[idx]) for v in results.values())
        p99 = max(sorted(v[idx])[int(0.99 * (len(v[idx]) - 1))] for v in results.values())
        return {"median_us": round(med, 1), "p99_us": round(p99, 1)}

    return {"protocol": protocol, "groups": groups, "ranks_per_group": ranks, "steps": steps, "quorum": stat(0),
            "should_commit": stat(1), "step": stat(2)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--groups", type=int, default=2)
    ap.add_argument("--ranks", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--protocol", default="both", choices=["framed", "grpc", "both"])
    ap.add_argument("--child", action="store_true")
    args = ap.parse_args()
    if args.protocol != "both":
        print(json.dumps(run(args.protocol, args.groups, args.ranks, args.steps)), flush=True)
        return
    # the protocol is a per-process setting of the clients: one child per protocol
    for protocol in ("framed", "grpc"):
        subprocess.run([sys.executable, os.path.abspath(__file__), "--protocol", protocol, "--groups", str(args.groups),
                        "--ranks", str(args.ranks), "--steps", str(args.steps)], check=True)


if __name__ == "__main__":
    main()
