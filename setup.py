"""Builds the native parts in-tree (nvcc for sm_100a, g++ for the control plane) before packaging.

``python setup.py build_ext --inplace`` and ``pip install -e .`` both end up in
``torchft_b200.utils.build.build_all``; the shared objects live inside the package directory.
"""

import os
import sys

from setuptools import setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _build_native() -> None:
    from torchft_b200.utils import build

    build.build_all()


class BuildNative(build_ext):
    def run(self) -> None:
        _build_native()


class BuildPy(build_py):
    def run(self) -> None:
        _build_native()
        super().run()


setup(cmdclass={"build_ext": BuildNative, "build_py": BuildPy})
