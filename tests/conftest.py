import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-multi-token-attention_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test: no bounded wait inside a tensor-core kernel may have run out unnoticed."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch
    if not torch.cuda.is_available():
        return
    import fmta_b200
    fmta_b200.check_device_status()


def pytest_sessionfinish(session, exitstatus):
    """Per-configuration error table of a GPU session: the largest absolute and relative error of every
    output over the comparisons made through helpers.check_outputs, written to parity_errors.txt in the
    folder named by the environment variable FMTA_REPORT_DIR (nothing is written without it)."""
    try:
        import helpers
    except Exception:
        return
    if not helpers.ERROR_LOG:
        return
    worst = {}
    for label, key, err, ref in helpers.ERROR_LOG:
        worst[(label, key)] = (err, ref)
    lines = ["%-78s %-7s %10s %10s %9s" % ("comparison", "output", "max-abs", "max|ref|", "relative")]
    for (label, key), (err, ref) in worst.items():
        lines.append("%-78s %-7s %10.3e %10.3g %9.1e" % (label, key, err, ref, err / ref if ref > 0 else 0.0))
    text = "\n".join(lines)
    out = os.environ.get("FMTA_REPORT_DIR", "")
    if out and os.path.isdir(out):
        with open(os.path.join(out, "parity_errors.txt"), "w") as f:
            f.write(text + "\n")
