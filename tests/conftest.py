"""Shared fixtures.  `-m "not gpu"` runs here on CPU (oracle vs golden vectors,
host logic, C-ABI surface); `-m gpu` runs the parity tests on a B200."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """The oracle and the CUDA library are built in-tree; build whichever is missing."""
    from oracle import escha_oracle
    escha_oracle.build()
    from escha_mlx_b200.csrc import build as cuda_build
    if not os.path.exists(cuda_build.LIB):
        cuda_build.build()


@pytest.fixture(scope="session")
def oracle():
    from oracle import escha_oracle
    return escha_oracle


def _npz(name):
    return np.load(os.path.join(GOLDEN, name))


@pytest.fixture(scope="session")
def ref_codec():
    return _npz("ref_codec.npz")


@pytest.fixture(scope="session")
def ref_dense_linear():
    return _npz("ref_dense_linear.npz")


@pytest.fixture(scope="session")
def ref_w8a16():
    return _npz("ref_w8a16.npz")


@pytest.fixture(scope="session")
def seeded_decode():
    return _npz("seeded_decode.npz")


@pytest.fixture(scope="session")
def seeded_linear():
    return _npz("seeded_linear.npz")


@pytest.fixture(scope="session")
def seeded_moe_block():
    return _npz("seeded_moe_block.npz")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda", 0)
