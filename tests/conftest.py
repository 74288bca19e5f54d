"""pytest configuration: registers the `gpu` marker and puts the repository root on sys.path."""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# Make every kernel call in the tests verify the device-side status words.
os.environ.setdefault("FBA_CHECK_STATUS", "1")
# Outputs and scratch are allocated NaN-filled instead of uninitialised, so a tile that a kernel
# fails to write cannot pass a comparison by luck.
os.environ.setdefault("FBA_POISON_OUTPUTS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    """One line per compared tensor of the benchmark-configuration tests: raw max-abs error, cosine
    and the magnitude of the expected tensor, so the distance from the absolute 2e-2 bound is on record."""
    from tests.util import PARITY_LOG

    rows = [r for r in PARITY_LOG if r[0].startswith(("C2", "C3", "C4", "C5"))]
    if rows:
        terminalreporter.write_sep("-", "parity of the benchmark configurations (raw max-abs, cosine, max|ref|)")
        for what, ma, cos, mx in rows:
            terminalreporter.write_line(f"PARITY {what}: max_abs={ma:.3e} cos={cos:.7f} max|ref|={mx:.3f}")
