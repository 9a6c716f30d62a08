import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))


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
    """Largest relative difference between engine and plain logits that the replay tests saw,
    per compute dtype and configuration: the bfloat16 bounds of the tests are set from these."""
    import helpers
    if helpers.OBSERVED:
        terminalreporter.write_line("largest engine-plain logit difference relative to max(1, |logit|):")
        for label in sorted(helpers.OBSERVED):
            terminalreporter.write_line(f"  {label}: {helpers.OBSERVED[label]:.3e}")
