"""The example trainer and the lighthouse CLI, end to end on CPU (three real processes)."""

import os
import socket
import subprocess
import sys
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_train_ddp_example_two_replica_groups(tmp_path):
    lh_port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", TORCHFT_B200_LOG="", CHECKPOINT_DIR=str(tmp_path),
               CHECKPOINT_EVERY="2")
    lighthouse = subprocess.Popen(
        [sys.executable, "-m", "torchft_b200.lighthouse", "--min_replicas", "2", "--bind", f"[::]:{lh_port}",
         "--join_timeout_ms", "20000"],
        env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL,
    )
    workers = []
    try:
        for _ in range(100):
            try:
                urllib.request.urlopen(f"http://127.0.0.1:{lh_port}/status", timeout=1).read()
                break
            except Exception:
                time.sleep(0.1)
        for g in range(2):
            wenv = dict(env, REPLICA_GROUP_ID=str(g), NUM_REPLICA_GROUPS="2", TOTAL_STEPS="5", RANK="0", WORLD_SIZE="1",
                        MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()),
                        TORCHFT_LIGHTHOUSE=f"http://127.0.0.1:{lh_port}")
            # each replica group has its own store; here the worker hosts it itself
            code = (
                "import os, torch.distributed as dist\n"
                "store = dist.TCPStore('127.0.0.1', int(os.environ['MASTER_PORT']), is_master=True, wait_for_workers=False)\n"
                "import runpy; runpy.run_path(os.path.join(%r, 'train_ddp.py'), run_name='__main__')\n" % ROOT
            )
            workers.append(subprocess.Popen([sys.executable, "-c", code], env=wenv, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
        for w in workers:
            out, _ = w.communicate(timeout=240)
            assert w.returncode == 0, out.decode()[-3000:]
        status = urllib.request.urlopen(f"http://127.0.0.1:{lh_port}/status", timeout=5).read().decode()
        assert "train_ddp_0" in status and "train_ddp_1" in status
        # replica group 0 left durable checkpoints behind (manager state included)
        from torchft_b200.utils.durable import latest_step

        assert latest_step(str(tmp_path)) is not None and latest_step(str(tmp_path)) >= 2
    finally:
        for w in workers:
            if w.poll() is None:
                w.kill()
        lighthouse.kill()
        lighthouse.wait()


def test_standalone_lighthouse_binary_usage():
    from torchft_b200.utils import build

    exe = build.lighthouse_bin_path()
    if not exe.exists():
        build.build_control()
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=30)
    assert res.returncode == 2 and "min_replicas is required" in res.stderr


def test_job_description_roles():
    from torchft_b200 import torchx as tx

    app = tx.hsdp("--flag", replicas=3, workers_per_replica=2, max_restarts=4, env={"FOO": "1"})
    assert app.name == "torchft" and [r.name for r in app.roles] == ["replica_0", "replica_1", "replica_2"]
    for g, role in enumerate(app.roles):
        assert role.entrypoint == "torchrun" and role.num_replicas == 2
        assert f"--master_port={29600 + g}" in role.args and "--nproc_per_node=2" in role.args
        assert "--max_restarts=4" in role.args and role.args[-2:] == ["train_ddp.py", "--flag"]
        assert role.env["REPLICA_GROUP_ID"] == str(g) and role.env["NUM_REPLICA_GROUPS"] == "3"
        assert role.env["FOO"] == "1" and role.env["CUDA_VISIBLE_DEVICES"] == ""
        assert role.env["TORCHFT_LIGHTHOUSE"].startswith("http://")
    import pytest

    with pytest.raises(ValueError):
        tx.hsdp(replicas=0)


def test_local_launcher_runs_two_replica_groups(tmp_path):
    """torchrun per replica group, started from the job description; the groups find each other through the lighthouse."""
    from torchft_b200 import _control
    from torchft_b200 import torchx as tx

    lighthouse = _control.Lighthouse(bind="[::]:0", min_replicas=2, join_timeout_ms=20000)
    try:
        port = lighthouse.address().rsplit(":", 1)[1]
        app = tx.hsdp(replicas=2, workers_per_replica=1, max_restarts=0, script=os.path.join(ROOT, "train_ddp.py"),
                      env={"TORCHFT_LIGHTHOUSE": f"http://127.0.0.1:{port}", "TOTAL_STEPS": "4", "PYTHONPATH": ROOT,
                           "TORCHFT_B200_LOG": "", "LOGLEVEL": "WARNING", "TORCH_CPP_LOG_LEVEL": "WARNING"})
        for role in app.roles:  # the default ports may be taken on a shared host
            role.args[0] = f"--master_port={_free_port()}"
        run = tx.run_local(app, log_dir=str(tmp_path))
        try:
            codes = run.wait(timeout=300)
        finally:
            run.stop()
        logs = "\n".join(open(os.path.join(tmp_path, f)).read()[-2000:] for f in os.listdir(tmp_path))
        assert codes == {"replica_0": 0, "replica_1": 0}, logs
    finally:
        lighthouse.shutdown()
