import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (HERE, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

# Development aid: with ULLM_B200_CPU_DOUBLE=1 and no GPU, the gpu-marked tests
# that go through the engine run on the CPU against tests/cpu_kernels.py, a
# plain-torch stand-in for the kernels.  It checks the tests' own logic and the
# engine's host side; it says nothing about the CUDA kernels.
CPU_DOUBLE = os.environ.get("ULLM_B200_CPU_DOUBLE") == "1"


def pytest_configure(config):
    # no test may hang a run: with the pytest-timeout plugin present, every test gets five minutes at most
    if config.pluginmanager.hasplugin("timeout") and not getattr(config.option, "timeout", None):
        config.option.timeout = 300
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "needs_cuda: cannot run against the CPU stand-in")


def device() -> str:
    import torch

    return "cuda:0" if torch.cuda.is_available() else "cpu"


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    if CPU_DOUBLE:
        from cpu_kernels import CpuKernels
        from ullm_b200.csrc import set_kernels

        set_kernels(CpuKernels())
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords and (not CPU_DOUBLE or "needs_cuda" in item.keywords):
            item.add_marker(skip)
