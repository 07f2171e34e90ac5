"""Build hook: compile ``dmuon_b200/ops/csrc`` for sm_100a while the package is built.

``pip install .`` (or ``pip install -e .`` / ``python setup.py build_py``) runs
``nvcc -gencode arch=compute_100a,code=sm_100a`` over every ``.cu`` file and
places ``libdmuon_b200.so`` inside the package, so an installed copy never needs
a compiler at import time.  ``DMUON_BUILD_KERNELS=0`` skips the step (the
library is then built on first use if ``nvcc`` is on the machine); a missing
``nvcc`` is reported and skipped as well, a failing compile is an error.

Role of the reference's ``setup.py:21-30`` (one ``CUDAExtension`` without an
architecture flag); here there is one library for exactly one architecture and
no torch extension machinery.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop

ROOT = Path(__file__).resolve().parent


def _load_builder():
    # import ops/build.py by path: importing the package would import torch
    spec = importlib.util.spec_from_file_location("_dmuon_b200_build", ROOT / "dmuon_b200" / "ops" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def build_kernels() -> None:
    off = ("0", "false", "no", "off")
    # DMUON_BUILD_FAST_CLIP is the reference's switch for its only compiled extension; honoured as an alias
    if (os.environ.get("DMUON_BUILD_KERNELS", "1").strip().lower() in off
            or os.environ.get("DMUON_BUILD_FAST_CLIP", "1").strip().lower() in off):
        print("dmuon_b200: DMUON_BUILD_KERNELS=0, not compiling the sm_100a kernel library")
        return
    builder = _load_builder()
    if builder._nvcc() is None:
        print("dmuon_b200: nvcc not found, the sm_100a kernel library will be built on first use")
        return
    path = builder.build()
    print(f"dmuon_b200: built {path}")


class BuildPyWithKernels(build_py):
    def run(self):
        build_kernels()
        super().run()


class DevelopWithKernels(develop):
    def run(self):
        build_kernels()
        super().run()


setup(cmdclass={"build_py": BuildPyWithKernels, "develop": DevelopWithKernels})
