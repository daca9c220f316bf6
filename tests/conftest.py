import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


# The reference package, when oracle/build_ref.py has built it (test infrastructure; used by the drop-in tests).
# Appended, so that a reference the user put on PYTHONPATH wins.
_REF_SITE = os.path.join(ROOT, "oracle", "_ref", "site")
if os.path.isdir(os.path.join(_REF_SITE, "falkon")) and _REF_SITE not in sys.path:
    sys.path.append(_REF_SITE)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)
