"""pytest configuration: registers the ``gpu`` marker and puts the repository root on ``sys.path``."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_sessionfinish(session, exitstatus):
    """After a GPU run: every comparison the parity tests made, with the error each assertion used and, beside it, the
    plain norm-scaled error max|a-b|/rms(b). Written to $CGPT_PARITY_REPORT when that is set."""
    import os
    path = os.environ.get("CGPT_PARITY_REPORT")
    try:
        from gpu_util import REPORT
    except Exception:  # pragma: no cover
        return
    if not path or not REPORT:
        return
    with open(path, "w") as f:
        f.write("comparison\tmetric\terror\ttolerance\tplain max|a-b|/rms(b)\n")
        for what, metric, e, tol, plain in REPORT:
            f.write(f"{what}\t{metric}\t{e:.3e}\t{tol:.1e}\t{plain:.3e}\n")
