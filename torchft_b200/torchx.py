"""Job description for a fault-tolerant HSDP run: one role per replica group, plus a local launcher.

``hsdp(...)`` has the call signature of the reference's TorchX component
(``torchft/torchx.py:11-76``): ``replicas`` replica groups, each a ``torchrun`` of
``workers_per_replica`` processes with its own rendezvous port and restart budget, all pointed
at one lighthouse through ``TORCHFT_LIGHTHOUSE``.  When the ``torchx`` package is importable the
function returns a ``torchx.specs.AppDef`` and can be named in a ``.torchxconfig``; without it
the same description is returned in the small dataclasses below, which ``run_local`` can execute
directly (every role becomes a child process group on this host; GPUs are dealt out in order).

Differences from the reference's component, on purpose:

* every role gets ``REPLICA_GROUP_ID`` and ``NUM_REPLICA_GROUPS`` (the reference's example trainer
  reads them but its component never sets them);
* ``CUDA_VISIBLE_DEVICES`` is only blanked when ``gpu == 0``; with ``gpu > 0`` ``run_local`` assigns
  ``gpu`` devices per worker to each role.
"""

from __future__ import annotations

import os
import shutil
import signal
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

try:  # pragma: no cover - torchx is optional
    import torchx.specs as _specs
except Exception:  # noqa: BLE001
    _specs = None

BASE_MASTER_PORT = 29600
DEFAULT_LIGHTHOUSE = "http://localhost:29510"


@dataclass
class Resource:
    cpu: int = 2
    gpu: int = 0
    memMB: int = 1024
    h: Optional[str] = None


@dataclass
class Role:
    name: str
    entrypoint: str
    args: List[str]
    env: Dict[str, str]
    image: str = ""
    num_replicas: int = 1
    min_replicas: Optional[int] = None
    max_retries: int = 0
    resource: Resource = field(default_factory=Resource)


@dataclass
class AppDef:
    name: str
    roles: List[Role]


def _role_env(user_env: Optional[Dict[str, str]], group: int, groups: int, gpu: int) -> Dict[str, str]:
    env = dict(user_env or {})
    env.setdefault("TORCH_CPP_LOG_LEVEL", "INFO")
    env.setdefault("LOGLEVEL", "INFO")
    env.setdefault("CLICOLOR_FORCE", "1")
    env.setdefault("TORCHFT_LIGHTHOUSE", os.environ.get("TORCHFT_LIGHTHOUSE", DEFAULT_LIGHTHOUSE))
    if gpu == 0:
        env.setdefault("CUDA_VISIBLE_DEVICES", "")
    env["REPLICA_GROUP_ID"] = str(group)
    env["NUM_REPLICA_GROUPS"] = str(groups)
    return env


def hsdp(
    *script_args: str,
    replicas: int = 2,
    workers_per_replica: int = 1,
    max_restarts: int = 10,
    script: str = "train_ddp.py",
    env: Optional[Dict[str, str]] = None,
    image: str = "",
    h: Optional[str] = None,
    cpu: int = 2,
    gpu: int = 0,
    memMB: int = 1024,
):
    """Describes ``replicas`` replica groups of ``workers_per_replica`` workers each."""
    if replicas <= 0:
        raise ValueError("replicas must be > 0")
    if workers_per_replica <= 0:
        raise ValueError("workers_per_replica must be > 0")
    roles = []
    for group in range(replicas):
        args = [
            f"--master_port={BASE_MASTER_PORT + group}",
            "--master_addr=127.0.0.1",
            "--nnodes=1",
            f"--nproc_per_node={workers_per_replica}",
            f"--max_restarts={max_restarts}",
        ]
        if script:
            args.append(script)
        args.extend(script_args)
        role_env = _role_env(env, group, replicas, gpu)
        if _specs is not None:  # pragma: no cover - torchx is optional
            roles.append(_specs.Role(
                name=f"replica_{group}", image=image, min_replicas=workers_per_replica,
                num_replicas=workers_per_replica, resource=_specs.resource(cpu=cpu, gpu=gpu, memMB=memMB, h=h),
                max_retries=0, env=role_env, entrypoint="torchrun", args=args,
            ))
        else:
            roles.append(Role(
                name=f"replica_{group}", entrypoint="torchrun", args=args, env=role_env, image=image,
                num_replicas=workers_per_replica, min_replicas=workers_per_replica, max_retries=0,
                resource=Resource(cpu=cpu, gpu=gpu, memMB=memMB, h=h),
            ))
    if _specs is not None:  # pragma: no cover
        return _specs.AppDef(name="torchft", roles=roles)
    return AppDef(name="torchft", roles=roles)


def _entrypoint_argv(entrypoint: str) -> List[str]:
    if entrypoint == "torchrun" and shutil.which("torchrun") is None:
        return [sys.executable, "-m", "torch.distributed.run"]
    return [entrypoint]


class LocalRun:
    """Handle on the child processes started by ``run_local``."""

    def __init__(self, procs: Dict[str, subprocess.Popen]) -> None:
        self.procs = procs

    def wait(self, timeout: Optional[float] = None) -> Dict[str, int]:
        deadline = None if timeout is None else time.monotonic() + timeout
        codes: Dict[str, int] = {}
        for name, proc in self.procs.items():
            left = None if deadline is None else max(0.0, deadline - time.monotonic())
            codes[name] = proc.wait(timeout=left)
        return codes

    def kill(self, role: str, sig: int = signal.SIGKILL) -> None:
        """Ends ONE role's process group: a fault injected at the job level."""
        proc = self.procs[role]
        try:
            os.killpg(proc.pid, sig)
        except ProcessLookupError:
            pass

    def stop(self) -> None:
        for name in list(self.procs):
            if self.procs[name].poll() is None:
                self.kill(name, signal.SIGTERM)
        for proc in self.procs.values():
            try:
                proc.wait(timeout=10)
            except subprocess.TimeoutExpired:
                os.killpg(proc.pid, signal.SIGKILL)


def run_local(app, cwd: Optional[str] = None, log_dir: Optional[str] = None,
              roles: Optional[Sequence[str]] = None) -> LocalRun:
    """Starts every role of ``app`` on this host; each gets its own process group and log file."""
    procs: Dict[str, subprocess.Popen] = {}
    next_gpu = 0
    for role in app.roles:
        gpus_per_worker = int(getattr(role.resource, "gpu", 0) or 0)
        env = dict(os.environ)
        env.update(role.env)
        want = gpus_per_worker * int(role.num_replicas)
        if want > 0 and "CUDA_VISIBLE_DEVICES" not in role.env:
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(next_gpu + i) for i in range(want))
            next_gpu += want
        if roles is not None and role.name not in roles:
            continue
        out = None
        if log_dir is not None:
            os.makedirs(log_dir, exist_ok=True)
            out = open(os.path.join(log_dir, f"{role.name}.log"), "ab")
        procs[role.name] = subprocess.Popen(
            _entrypoint_argv(role.entrypoint) + list(role.args), env=env, cwd=cwd,
            stdout=out, stderr=subprocess.STDOUT if out is not None else None, start_new_session=True,
        )
    return LocalRun(procs)


def main(argv: Optional[Sequence[str]] = None) -> int:
    """``python -m torchft_b200.torchx --replicas 2 --workers-per-replica 1 [--lighthouse] -- script args``"""
    import argparse

    ap = argparse.ArgumentParser(description="run replica groups of a fault-tolerant job on this host")
    ap.add_argument("--replicas", type=int, default=2)
    ap.add_argument("--workers-per-replica", type=int, default=1)
    ap.add_argument("--max-restarts", type=int, default=10)
    ap.add_argument("--gpu", type=int, default=0, help="GPUs per worker")
    ap.add_argument("--script", default="train_ddp.py")
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--lighthouse", action="store_true", help="also start a lighthouse for the job")
    ap.add_argument("script_args", nargs="*")
    args = ap.parse_args(argv)

    lighthouse = None
    env: Dict[str, str] = {}
    if args.lighthouse:
        from torchft_b200 import _control

        lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=1)
        env["TORCHFT_LIGHTHOUSE"] = lighthouse.address()
    app = hsdp(*args.script_args, replicas=args.replicas, workers_per_replica=args.workers_per_replica,
               max_restarts=args.max_restarts, script=args.script, env=env, gpu=args.gpu)
    run = run_local(app, log_dir=args.log_dir)
    try:
        codes = run.wait()
    except KeyboardInterrupt:
        run.stop()
        codes = {"interrupted": 130}
    finally:
        if lighthouse is not None:
            lighthouse.shutdown()
    return max(codes.values()) if codes else 0


if __name__ == "__main__":
    sys.exit(main())
