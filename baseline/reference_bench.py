"""Reference arm of ``bench.py``: the reference's own stack on the same metric and config.

The reference (torchft 0.1.1) ships its control plane as a Rust extension built with
maturin; neither maturin nor a Rust toolchain is available offline, so a pip install of the
reference stops at the build backend.  ``baseline/make_ref.py`` therefore lays the reference's
unmodified Python sources under ``baseline/_ref/torchft`` next to this repository's C++ control
plane compiled under the reference's extension name (``torchft.torchft``, same classes and
signatures).  ``baseline/reference_runner.py`` then drives the reference's Manager, DDP wrapper,
optimizer wrapper and NCCL process group.  Without that directory the arm reports itself
unavailable.
"""

from __future__ import annotations

import json
import os


def run_reference(args) -> None:
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "torchft")
    if not os.path.isdir(ref):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({
                "impl": "reference",
                "unavailable": "reference not installed: run baseline/make_ref.py (the Rust extension needs maturin, cargo and protoc, which are missing offline)",
            }), flush=True)
        return
    from baseline.reference_runner import run  # populated only when an install exists

    run(args)
