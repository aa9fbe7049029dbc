import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


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


@pytest.fixture
def parity_report(request):
    """Records achieved errors: report(kind, **numbers) prints one line per record and, when
    $VOLTA_B200_PARITY_REPORT names a file, appends it there as JSON (the tables of achieved parity in the
    design notes are made from such a file)."""
    import json

    def report(kind, **numbers):
        rec = dict(test=request.node.name, kind=kind, **numbers)
        print("parity:", json.dumps(rec))
        path = os.environ.get("VOLTA_B200_PARITY_REPORT")
        if path:
            with open(path, "a") as f:
                f.write(json.dumps(rec) + "\n")

    return report
