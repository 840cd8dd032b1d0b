"""Shared pytest configuration.

``gpu`` marks tests that need a CUDA device; everything else runs on CPU (multi-rank tests
start real ``gloo`` processes on 127.0.0.1).  ``--output-folder`` keeps the reference's
per-test ``*_l2.log`` convention (``tests/conftest.py:6-23`` of the reference).
"""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_addoption(parser):
    parser.addoption("--output-folder", action="store", default=None,
                     help="directory for '<test>_l2.log' files (matrix_shape relative_l2_error)")


@pytest.fixture
def output_folder(request):
    folder = request.config.getoption("--output-folder")
    if folder is None:
        return None
    path = Path(folder)
    path.mkdir(parents=True, exist_ok=True)
    return path


def pytest_collection_modifyitems(config, items):
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
