import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """Worst observed parity statistic per test and quantity (tests/common.py: STATS); also
    written as JSON to $LH_PARITY_STATS_FILE when that is set."""
    try:
        from tests.common import STATS
    except Exception:
        return
    if not STATS:
        return
    agg = {}
    for (test, what, key), v in STATS.items():
        k = (test, key)
        agg[k] = max(agg.get(k, 0.0), v)
    terminalreporter.write_line("")
    terminalreporter.write_line("observed parity statistics (worst per test):")
    for (test, key), v in sorted(agg.items()):
        terminalreporter.write_line(f"  {test:55s} {key:22s} {v:.3e}")
    out = os.environ.get("LH_PARITY_STATS_FILE")
    if out:
        import json
        with open(out, "w") as fh:
            json.dump([{"test": t, "quantity": k, "worst": v} for (t, k), v in sorted(agg.items())], fh, indent=1)
