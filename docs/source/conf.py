"""Sphinx configuration of the API reference (``make -C docs html``).

The pages are autodoc stubs: the text lives in the docstrings of the package.  The native control
plane (``torchft_b200._control``) and the kernel library are mocked when they have not been built, so
the reference can be generated on a machine without a compiler or a GPU."""

import importlib.util
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))

project = "torchft_b200"
author = "torchft_b200 contributors"
extensions = ["sphinx.ext.autodoc", "sphinx.ext.napoleon", "sphinx.ext.viewcode"]
autodoc_member_order = "bysource"
autodoc_default_options = {"members": True, "show-inheritance": True}
autodoc_mock_imports = []
if importlib.util.find_spec("torchft_b200._control") is None:
    autodoc_mock_imports.append("torchft_b200._control")
html_theme = "alabaster"
exclude_patterns = []
