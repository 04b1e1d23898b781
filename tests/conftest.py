import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_pkg():
    return importlib.import_module("dist-gpu-sampling_b200")


def load_synth():
    return importlib.import_module("dist-gpu-sampling_b200.synth")


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


@pytest.fixture(scope="session")
def synth():
    return load_synth()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def abi(pkg):
    return pkg.load_abi()


@pytest.fixture(scope="session")
def ops(pkg):
    """torch.ops.dgs_ops / torch.classes.dgs_classes backed by the CUDA library."""
    import torch
    pkg.load_ops()
    return torch.ops.dgs_ops
