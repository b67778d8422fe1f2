"""Reference arm of ``bench.py``: the reference's own stack on the same metric and config.

The reference (torchft 0.1.1) ships its control plane as a Rust extension built with
maturin; neither maturin nor a Rust toolchain is available offline, so
``pip install --no-index ... /root/reference`` stops at the build backend.  Until an
install exists under ``baseline/_ref`` this arm reports itself unavailable.
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
                "unavailable": "reference not installable offline: build backend maturin and the Rust toolchain (cargo, rustc, protoc) are missing",
            }), flush=True)
        return
    from baseline.reference_runner import run  # populated only when an install exists

    run(args)
