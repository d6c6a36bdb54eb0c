import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_terminal_summary(terminalreporter):
    """The worst error of every test that compared logits with the plain implementation."""
    try:
        import helpers
    except Exception:
        return
    if not helpers.WORST:
        return
    terminalreporter.section("worst errors against the plain implementation (fraction of the logit scale)")
    for test, (err, tol) in sorted(helpers.WORST.items()):
        terminalreporter.write_line(f"{err:.3e} (allowed {tol:.1e})  {test}")
