import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, when no device is present."""
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover - torch is part of the image
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.hookimpl(hookwrapper=True)
def pytest_runtest_makereport(item, call):
    """A failed GPU test also reports the CUDA error behind the library's last launch failure."""
    outcome = yield
    report = outcome.get_result()
    if report.when == "call" and report.failed and "gpu" in item.keywords:
        try:
            from attnarc_b200 import _native

            name = _native.library().loom_cuda_last_launch_failure().decode()
            report.sections.append(("loom library", f"last launch failure on this thread: {name}"))
        except Exception:  # the library itself may be what is missing
            pass
