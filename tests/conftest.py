"""Test configuration: the `gpu` marker, import paths, shared fixtures."""

import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for path in (ROOT, HERE):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The worst error each comparison with the plain implementation saw, by dtype and
    schedule (harness.record_error): how far the engine stays from its bars."""
    import harness

    if not harness.WORST:
        return
    terminalreporter.write_sep("-", "worst relative error against the plain implementation")
    for (dtype, what), (err, bar) in sorted(harness.WORST.items()):
        terminalreporter.write_line(f"{dtype:9s} {what:60s} {err:.3e}  (bar {bar:.0e})")
