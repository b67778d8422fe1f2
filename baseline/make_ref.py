"""Prepares ``baseline/_ref`` for the reference arm of ``bench.py``.

The reference cannot be pip-installed offline (its build backend, maturin, and the Rust
toolchain are missing).  Its Python sources are pure Python, though; the only compiled
piece is the control-plane extension ``torchft.torchft`` (Manager server, ManagerClient,
Lighthouse, QuorumResult).  This script

1. copies the reference's own, unmodified ``torchft/*.py`` into ``baseline/_ref/torchft``;
2. builds this repository's C++ control plane under the module name ``torchft`` and places
   it there as ``torchft/torchft.<abi>.so`` -- a drop-in for the Rust extension with the
   interface of ``torchft/torchft.pyi``.

Everything the benchmark measures (NCCL allreduce + divide, DDP bucketing, the Manager state
machine, HTTP checkpoint transport) then runs from the reference's Python.

    python baseline/make_ref.py [path/to/reference/checkout]

Without an argument the checkout is looked for in ``$TORCHFT_REFERENCE_DIR`` and then in a
directory called ``reference`` next to this repository.
"""

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

def _reference_checkout() -> Path:
    if len(sys.argv) > 1:
        return Path(sys.argv[1])
    if os.environ.get("TORCHFT_REFERENCE_DIR"):
        return Path(os.environ["TORCHFT_REFERENCE_DIR"])
    return ROOT.parent / "reference"


REF_SRC = _reference_checkout() / "torchft"
DEST = ROOT / "baseline" / "_ref" / "torchft"


def main() -> None:
    import pybind11

    if not REF_SRC.is_dir():
        raise SystemExit(f"{REF_SRC} is not available here")
    DEST.mkdir(parents=True, exist_ok=True)
    for src in sorted(REF_SRC.glob("*.py")):
        if src.name.endswith("_test.py"):
            continue
        shutil.copy2(src, DEST / src.name)
    shutil.copy2(REF_SRC / "torchft.pyi", DEST / "torchft.pyi")
    control = ROOT / "torchft_b200" / "csrc" / "control"
    sources = [str(p) for p in sorted(control.glob("*.cc")) if p.name not in ("lighthouse_main.cc", "stress_main.cc")]
    out = DEST / ("torchft" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
    cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-pthread", "-shared", "-fvisibility=hidden", "-Wl,-Bsymbolic",
           "-DTFT_MODULE_NAME=torchft", "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           "-I", str(control), *sources, "-o", str(out)]
    subprocess.run(cmd, check=True)
    print(f"reference sources + control-plane stand-in ready under {DEST}")


if __name__ == "__main__":
    main()
