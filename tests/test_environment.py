"""The box has what the framework needs (the reference checks its own requirements and logins in
tests/test_setup.py:5-31; nothing here needs a network or an account)."""
import importlib
import shutil

import pytest


@pytest.mark.parametrize("module", ["torch", "numpy", "yaml", "pydantic", "pandas"])
def test_required_packages_import(module):
    importlib.import_module(module)


def test_distributed_backends():
    import torch.distributed as dist
    assert dist.is_available() and dist.is_gloo_available()


def test_toolchain_builds_the_host_library():
    from diloco_swarm_b200.ops import _build
    assert shutil.which("g++") or shutil.which("c++"), "a C++17 compiler is needed for libdswarm_host.so"
    assert _build.build_host().endswith("libdswarm_host.so")


def test_nvcc_targets_sm_100a():
    from diloco_swarm_b200.ops import _build
    try:
        nvcc = _build.nvcc_path()
    except RuntimeError:
        pytest.skip("no nvcc on this box: the kernels cannot be rebuilt here")
    import subprocess
    archs = subprocess.run([nvcc, "--list-gpu-arch"], capture_output=True, text=True).stdout
    assert "compute_100" in archs, "this nvcc cannot build for Blackwell (compute_100a)"
    assert "arch=compute_100a,code=sm_100a" in _build.NVCC_FLAGS
