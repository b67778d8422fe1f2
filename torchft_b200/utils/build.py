"""In-tree native builds.

Two artefacts are produced next to the Python sources:

* ``torchft_b200/lib/libtft_kernels.so`` -- every ``.cu`` file under ``csrc/kernels``
  compiled with nvcc for ``sm_100a`` and exported through a plain C ABI (loaded with
  ctypes, no link-time dependency on torch or libcuda).
* ``torchft_b200/_control.*.so`` -- the C++ control plane (lighthouse, manager server and
  client) as a pybind11 extension module, plus the ``tft_lighthouse`` executable.

Objects are rebuilt only when a source or header is newer than the object.
"""

from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List

PKG = Path(__file__).resolve().parent.parent
KERNEL_SRC = PKG / "csrc" / "kernels"
CONTROL_SRC = PKG / "csrc" / "control"
LIB_DIR = PKG / "lib"
OBJ_DIR = PKG / "lib" / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _newest(paths: List[Path]) -> float:
    return max((p.stat().st_mtime for p in paths if p.exists()), default=0.0)


def kernels_lib_path() -> Path:
    return LIB_DIR / "libtft_kernels.so"


def control_module_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / f"_control{suffix}"


def lighthouse_bin_path() -> Path:
    return LIB_DIR / "tft_lighthouse"


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compiles all CUDA sources for sm_100a and links ``libtft_kernels.so``."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(KERNEL_SRC.glob("*.cu"))
    headers = sorted(KERNEL_SRC.glob("*.cuh")) + sorted(KERNEL_SRC.glob("*.h"))
    hdr_time = _newest(headers)
    objs: List[Path] = []
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(KERNEL_SRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd: List[str]) -> None:
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    out = kernels_lib_path()
    if force or jobs or not out.exists():
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-cudart", "shared"]
        run(cmd)
    return out


def build_control(force: bool = False) -> Path:
    """Builds the pybind11 control-plane module and the standalone lighthouse binary."""
    import pybind11

    LIB_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(p for p in CONTROL_SRC.glob("*.cc") if p.name not in ("lighthouse_main.cc", "stress_main.cc"))
    headers = sorted(CONTROL_SRC.glob("*.h"))
    out = control_module_path()
    newest = max(_newest(sources), _newest(headers))
    # Prefer the distribution compiler: it links libstdc++ dynamically, so the module
    # shares one C++ runtime with torch.  -Bsymbolic keeps a statically linked runtime
    # (other toolchains) from being half-interposed by the process-wide one.
    cxx = os.environ.get("TFT_CXX") or ("/usr/bin/g++" if Path("/usr/bin/g++").exists() else os.environ.get("CXX", "g++"))
    common = ["-O2", "-std=c++17", "-fPIC", "-pthread", "-Wall", "-Wno-unused-function", "-Wl,-Bsymbolic"]
    if force or not out.exists() or out.stat().st_mtime < newest:
        py_inc = sysconfig.get_paths()["include"]
        cmd = [cxx, *common, "-shared", "-fvisibility=hidden", "-I", pybind11.get_include(), "-I", py_inc,
               "-I", str(CONTROL_SRC), *map(str, sources), "-o", str(out)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"control build failed:\n{res.stdout}\n{res.stderr}")
    main_src = CONTROL_SRC / "lighthouse_main.cc"
    exe = lighthouse_bin_path()
    if main_src.exists() and (force or not exe.exists() or exe.stat().st_mtime < max(newest, main_src.stat().st_mtime)):
        lib_sources = [str(p) for p in sources if p.name != "bindings.cc"]
        cmd = [cxx, *common, "-I", str(CONTROL_SRC), str(main_src), *lib_sources, "-o", str(exe)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"lighthouse binary build failed:\n{res.stdout}\n{res.stderr}")
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_control(force=force)
    build_kernels(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", kernels_lib_path(), control_module_path())
