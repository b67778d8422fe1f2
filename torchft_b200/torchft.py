"""The compiled control plane under the module name the reference uses for its extension.

Code written against the reference imports ``Manager``, ``ManagerClient``, ``Lighthouse`` and
``QuorumResult`` from ``torchft.torchft`` (interface: the reference's ``torchft/torchft.pyi``);
with ``import torchft_b200 as torchft`` the same import path resolves here, to the C++ classes of
``torchft_b200._control``.
"""

from torchft_b200._control import (  # noqa: F401
    Lighthouse,
    LighthouseClient,
    Manager,
    ManagerClient,
    QuorumResult,
    lighthouse_main,
)

__all__ = ("Lighthouse", "LighthouseClient", "Manager", "ManagerClient", "QuorumResult", "lighthouse_main")
