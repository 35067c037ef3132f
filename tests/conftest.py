from __future__ import annotations

import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.0 (B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "moe_golden.npz")


@pytest.fixture(scope="session")
def golden_hashes():
    table = {}
    for line in (ROOT / "tests" / "golden" / "moe_golden_inputs.sha256").read_text().splitlines():
        digest, name = line.split()
        table[name] = digest
    return table
