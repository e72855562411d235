import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """The CUDA library and the oracle are built artefacts; build them if they are missing."""
    from cubek_b200 import _ffi

    if not _ffi.LIB_PATH.exists():
        from cubek_b200.build import build

        build()
    if not _ffi.LIB_PATH_HALF_AWAY.exists():
        from cubek_b200.build import build

        build(half_away=True)
    from oracle import oracle

    oracle.build()
    from tests.device_api.build_probe import build_probe

    build_probe()
    yield
