import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "slow: full-size model cases (minutes of CPU oracle time)")


@pytest.fixture(scope="session")
def golden():
    """Vectors generated from the reference's numeric tests (tests/golden/make_golden.py)."""
    data = np.load(ROOT / "tests" / "golden" / "llmcp_numeric.npz")

    class Cases:
        def __call__(self, case):
            prefix = case + "/"
            return {k[len(prefix):]: data[k] for k in data.files if k.startswith(prefix)}

        def names(self):
            return sorted({k.split("/")[0] for k in data.files})

    return Cases()


def assert_close(got, want, tol, what=""):
    """math.isclose semantics of the reference harness (run_numeric.py:599-604)."""
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    rel, abs_ = float(tol[0]), float(tol[1])
    bound = np.maximum(rel * np.maximum(np.abs(got), np.abs(want)), abs_)
    bad = np.abs(got - want) > bound
    assert not bad.any(), (
        f"{what}: {bad.sum()} of {got.size} outside tolerance; first at {np.argmax(bad)}: "
        f"got {got[np.argmax(bad)]} want {want[np.argmax(bad)]}")
