"""The compiled control plane under the module name the reference uses for its extension.

Code written against the reference imports ``Manager``, ``ManagerClient``, ``Lighthouse`` and
``QuorumResult`` from ``torchft.torchft`` (interface: the reference's ``torchft/torchft.pyi``);
replacing the package name in such an import leads here, to the C++ classes of
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
