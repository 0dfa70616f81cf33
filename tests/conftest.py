import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def error_log():
    """Measured max-abs errors of the GPU parity cases, printed at the end of the session
    (visible with -s) and written to $SPA_ARTIFACT_DIR/parity_errors.json when that is set."""
    import json
    log = {}
    yield log
    if log:
        out_dir = os.environ.get("SPA_ARTIFACT_DIR")
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)
            with open(os.path.join(out_dir, "parity_errors.json"), "w") as f:
                json.dump(log, f, indent=1, sort_keys=True)
        print("\nparity errors:", json.dumps(log, sort_keys=True))
