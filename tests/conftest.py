import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
LUT_DIR = os.path.join(GOLDEN, "lut")
SMALL_LUTS = ["ACC_7", "MBM_1", "MBM_3", "MBM_5", "MBM_7", "MIT_1", "MIT_3", "MIT_5", "MIT_7"]
BIG_LUT = os.path.join(ROOT, "oracle", "_ref", "lut", "MBM_11.bin")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def lut_path(name: str) -> str:
    return os.path.join(LUT_DIR, name + ".bin")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle.get()


@pytest.fixture(scope="session")
def luts():
    """name -> (uint8 array, m) for the nine small LUTs."""
    from oracle.oracle import load_lut
    return {n: load_lut(lut_path(n)) for n in SMALL_LUTS}


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / (den if den > 0 else 1.0))


def set_switch(monkeypatch, name: str, value) -> None:
    """Sets (or, with value None, removes) one of the library's AMSIM_* debug switches for the rest
    of the test and makes the library re-read its switches (it reads the environment once)."""
    from approxtrain_b200 import _lib
    if value is None:
        monkeypatch.delenv(name, raising=False)
    else:
        monkeypatch.setenv(name, str(value))
    _lib.lib.amsim_debug_reload_env()


@pytest.fixture(autouse=True)
def _restore_switches():
    """After a test (and after monkeypatch has put the environment back) the library re-reads its switches."""
    yield
    try:
        from approxtrain_b200 import _lib
    except Exception:
        return
    _lib.lib.amsim_debug_reload_env()
