import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")

# Property tests draw the same examples on every run unless asked to explore
# (HYPOTHESIS_PROFILE=explore, or --hypothesis-seed=N on the command line).
try:
    from hypothesis import settings as _hypothesis_settings

    _hypothesis_settings.register_profile("repeatable", derandomize=True, database=None)
    _hypothesis_settings.register_profile("explore", derandomize=False)
    _hypothesis_settings.load_profile(os.environ.get("HYPOTHESIS_PROFILE", "repeatable"))
except ImportError:  # the property tests skip themselves without hypothesis
    pass


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")
    # Native code is built in-tree; build it once if a fresh checkout has none.
    from torchft_b200.utils import build

    if not build.control_module_path().exists():
        build.build_control()
    if not build.kernels_lib_path().exists():
        build.build_kernels()
    from torchft_b200 import _control

    _control.set_log_enabled(False)


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
