import os
import sys

import pytest

# make every operator call synchronise and raise if a kernel reported a problem through its status word
os.environ.setdefault("SBATTN_CHECK_STATUS", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


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


def pytest_terminal_summary(terminalreporter):
    """Lists the worst measured error per test and tensor, so that the margin to each bar is on record in the log."""
    try:
        import util
    except Exception:  # pragma: no cover
        return
    if not util.MARGINS:
        return
    worst = {}
    for test, what, name, err, tol in util.MARGINS:
        key = (test.split("::", 1)[-1], name)
        if key not in worst or err / tol > worst[key][0] / worst[key][1]:
            worst[key] = (err, tol)
    terminalreporter.write_sep("-", "parity margins: worst max-abs error per test and tensor (bar)")
    tests = {}
    for (test, name), (err, tol) in worst.items():
        tests.setdefault(test, []).append(f"{name} {err:.2e}")
        tests[test + "::bar"] = tol
    for test in [t for t in tests if not t.endswith("::bar")]:
        terminalreporter.write_line(f"{test}: " + ", ".join(tests[test]) + f" (bar {tests[test + '::bar']:g})")
