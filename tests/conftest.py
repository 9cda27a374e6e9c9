import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; everything else runs on CPU")
    # the native pieces are build products (git-ignored): make sure they exist before anything imports the package
    # (run as a script: importing the package would already need the library it builds)
    import subprocess

    subprocess.run([sys.executable, os.path.join(ROOT, "quant_ops_b200", "build.py")], check=True)


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        have_gpu = torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no sm_100 GPU on this machine")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
