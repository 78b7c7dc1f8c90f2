import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    """Which branch of the parity rule every comparison passed by (tests/helpers.py::assert_parity)."""
    from tests import helpers
    log = helpers.PARITY_LOG
    if not log:
        return
    tr = terminalreporter
    counts = {}
    for _test, _name, branch, _fo, _mx, _note in log:
        counts[branch] = counts.get(branch, 0) + 1
    tr.write_sep("-", "parity branches")
    tr.write_line("comparisons: " + ", ".join(f"{k}: {v}" for k, v in sorted(counts.items())))
    for test, name, branch, fo, mx, note in log:
        if branch != "strict":
            tr.write_line(f"  {branch:15s} {test} [{name}] outside {fo:.4%} max|err| {mx:.3e} {note}")
    # the benchmark-size cases, one line per test: how many comparisons were strict, and the largest error
    per_test = {}
    for test, name, branch, fo, mx, note in log:
        if "baseline" in test:
            n, strict, worst = per_test.get(test, (0, 0, 0.0))
            per_test[test] = (n + 1, strict + (branch == "strict"), max(worst, mx))
    for test, (n, strict, worst) in per_test.items():
        tr.write_line(f"  {test}: {strict}/{n} comparisons strict, largest |err| {worst:.3e}")
