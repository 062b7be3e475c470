"""Test tiers: files are named ``test_<tier>_<subject>.py`` (unit / integration / gpu / dist).

GPU tests carry ``@pytest.mark.gpu`` and are skipped automatically when no CUDA device is present.
"""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


TIERS = ("unit", "integration", "gpu", "dist", "zz")


def pytest_addoption(parser):
    parser.addoption("--suite", default="all", choices=["unit", "integration", "gpu", "dist", "all"],
                     help="run one tier of the test files (test_<tier>_<subject>.py); default: all")


def _tier_of(path: str) -> str:
    name = os.path.basename(path)
    for t in TIERS:
        if name.startswith(f"test_{t}_"):
            return t
    return "unit"


@pytest.fixture(autouse=True)
def _restore_he_environment():
    """Every ``HE_*`` switch a test sets is put back afterwards, so tests cannot leak configuration into each other."""
    before = {k: v for k, v in os.environ.items() if k.startswith("HE_")}
    yield
    for k in [k for k in os.environ if k.startswith("HE_") and k not in before]:
        del os.environ[k]
    os.environ.update(before)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "dist: spawns multiple ranks")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    suite = config.getoption("--suite")
    if suite != "all":
        keep = [it for it in items if _tier_of(str(it.fspath)) == suite]
        drop = [it for it in items if _tier_of(str(it.fspath)) != suite]
        if drop:
            config.hook.pytest_deselected(items=drop)
            items[:] = keep
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
