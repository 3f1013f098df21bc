"""pytest configuration: the ``gpu`` marker and import paths.

Tests marked ``gpu`` need a CUDA device and the built shared library; everything else runs
on the CPU.  The oracle (``oracle/``) is importable from the tests only.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (ROOT, ROOT / "oracle"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """Achieved output errors of the labelled parity cases (tolerance: 1e-2 * RMS + half an ulp)."""
    try:
        from helpers import MARGINS
    except Exception:
        return
    if not MARGINS:
        return
    terminalreporter.write_sep("-", "parity margins: max|err|/RMS(ref), and the part beyond half an ulp of the output")
    for label, rel, beyond in MARGINS:
        terminalreporter.write_line(f"{label:<58s} {rel:9.5f}  {beyond:9.5f}")
