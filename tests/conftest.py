import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def reference_file(rel: str):
    """Path of a file of the reference tree: the offline install under ``baseline/_ref`` first, then the
    checkout named by ``TELETRON_REFERENCE`` (default: a ``reference`` folder beside this repository)."""
    mount = Path(os.environ.get("TELETRON_REFERENCE", str(ROOT.parent / "reference")))
    for base in (ROOT / "baseline" / "_ref", mount):
        p = base / rel
        if p.exists():
            return p
    return None
