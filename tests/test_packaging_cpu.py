"""The package can be built and installed: ``pyproject.toml`` names it, ships
the kernel sources and the built library as package data, and ``setup.py``'s
build hook compiles ``ops/csrc`` for sm_100a through ``ops/build.py``."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pyproject_declares_package_and_kernel_data():
    tomllib = pytest.importorskip("tomllib")
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as fh:
        cfg = tomllib.load(fh)
    assert cfg["project"]["name"] == "dmuon-b200"
    assert any(d.startswith("torch") for d in cfg["project"]["dependencies"])
    data = cfg["tool"]["setuptools"]["package-data"]["dmuon_b200.ops"]
    assert "csrc/*.cu" in data and "csrc/*.cuh" in data and "lib/*.so" in data
    assert cfg["tool"]["setuptools"]["packages"]["find"]["include"] == ["dmuon_b200*"]


def test_setup_build_hook_uses_the_sm100a_builder(monkeypatch):
    spec = importlib.util.spec_from_file_location("_setup_under_test", os.path.join(ROOT, "setup.py"))
    src = open(os.path.join(ROOT, "setup.py")).read()
    assert "build_kernels" in src and "BuildPyWithKernels" in src
    # load only the helper functions: executing setup() itself would run a build command
    ns: dict = {"__file__": os.path.join(ROOT, "setup.py"), "__name__": "_setup_under_test"}
    exec(compile(src.split("\nsetup(")[0], spec.origin, "exec"), ns)
    builder = ns["_load_builder"]()
    assert "arch=compute_100a,code=sm_100a" in builder.NVCC_FLAGS
    assert {p.name for p in builder._sources()} >= {"gemm_sm100.cu", "peer_sm100.cu", "multi_tensor.cu"}
    # the opt-out leaves the tree untouched
    monkeypatch.setenv("DMUON_BUILD_KERNELS", "0")
    called = []
    monkeypatch.setattr(builder, "build", lambda *a, **k: called.append(1))
    ns["build_kernels"]()
    assert not called
    sys.modules.pop("_dmuon_b200_build", None)
