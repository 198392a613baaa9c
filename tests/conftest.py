import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


HAS_GPU = _has_gpu()


def pytest_collection_modifyitems(config, items):
    if HAS_GPU:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def built():
    """The CUDA library and the oracle, built in-tree if they are missing."""
    from cuqwen_b200 import _abi, build
    if not _abi.LIB_PATH.exists() or not build.GEN_BIN.exists():
        build.build_cuda()
        build.build_gen()
    build.build_oracle()
    return True


@pytest.fixture(scope="session")
def tmpdir_big(tmp_path_factory):
    base = Path("/dev/shm") if Path("/dev/shm").is_dir() and os.access("/dev/shm", os.W_OK) else None
    if base is not None:
        d = base / f"cuqwen_test_{os.getpid()}"
        d.mkdir(exist_ok=True)
        yield d
        for f in d.iterdir():
            f.unlink()
        d.rmdir()
    else:
        yield tmp_path_factory.mktemp("big")
