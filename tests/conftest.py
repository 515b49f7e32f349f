"""Shared test plumbing: import paths, the `gpu` marker, golden-fixture access."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO / "ascend-ops_b200"))
sys.path.insert(0, str(REPO))
GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def f16(bits: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> float16 tensor."""
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.float16)


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def knob(monkeypatch, name, value):
    """Set (value None: unset) a B200OPS_* tuning variable for the rest of the test.  The library
    reads its variables once per process, so it is told to read them again."""
    if value is None:
        monkeypatch.delenv(name, raising=False)
    else:
        monkeypatch.setenv(name, str(value))
    from ascend910a_extras import cabi as m
    m.reload_options()


@pytest.fixture(autouse=True)
def _fresh_tuning_options():
    """A test's tuning variables end with it (monkeypatch restores the environment first)."""
    yield
    lib = os.path.join(str(REPO), "ascend-ops_b200", "ascend910a_extras", "lib", "libb200ops.so")
    if os.path.exists(lib):
        from ascend910a_extras import cabi as m
        m.reload_options()


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(GOLDEN / f"{name}.npz")
    return load


@pytest.fixture(scope="session")
def cabi():
    """The ctypes binding of libb200ops.so; fails (not skips) if the library is not built."""
    from ascend910a_extras import cabi as m
    m.load()
    return m


@pytest.fixture(scope="session")
def ops():
    import ascend910a_extras.ops as m
    return m
