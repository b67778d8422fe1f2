"""Race and memory-error detection for the C++ control plane.

The lighthouse, the manager servers and their clients are compiled together with a native
stress harness (``csrc/control/stress_main.cc``) under ThreadSanitizer, AddressSanitizer and
UndefinedBehaviorSanitizer and run in one process: decoder fuzzing, quorum and should_commit rounds
from many threads, dashboard polling, garbage HTTP/2 clients, and a replica group that goes away
half way through.
"""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "torchft_b200", "csrc", "control")
SOURCES = ["wire.cc", "net.cc", "h2.cc", "quorum.cc", "lighthouse.cc", "manager.cc", "cli.cc", "stress_main.cc"]


def _compiler():
    cxx = os.environ.get("TFT_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++"))
    if cxx is None:
        pytest.skip("no C++ compiler")
    return cxx


@pytest.mark.parametrize("sanitizer,marker", [("thread", "ThreadSanitizer"), ("address", "AddressSanitizer"),
                                              ("undefined", "runtime error:")])
def test_control_plane_under_sanitizer(tmp_path, sanitizer, marker):
    cxx = _compiler()
    exe = tmp_path / f"stress_{sanitizer}"
    build = subprocess.run(
        [cxx, "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-pthread", "-I", SRC,
         *[os.path.join(SRC, s) for s in SOURCES], "-o", str(exe)],
        capture_output=True, text=True, timeout=600,
    )
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip(f"-fsanitize={sanitizer} runtime not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 second_deadlock_stack=1", ASAN_OPTIONS="detect_leaks=1")
    for protocol in ("framed", "grpc"):  # the length-prefixed transport and gRPC over HTTP/2
        run = subprocess.run([str(exe), "4", "3", "40", protocol], capture_output=True, text=True, timeout=300, env=env)
        assert marker not in run.stderr, protocol + "\n" + run.stderr[-6000:]
        assert "LeakSanitizer" not in run.stderr, protocol + "\n" + run.stderr[-6000:]
        assert run.returncode == 0, protocol + "\n" + run.stderr[-3000:]
        assert "stress: 0 failure(s)" in run.stderr
