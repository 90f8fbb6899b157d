import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    """Vectors produced by the reference's own CPU operators (tests/golden/make_golden.py)."""
    with np.load(ROOT / "tests" / "golden" / "reference_vectors.npz") as data:
        return {k: data[k] for k in data.files}


def assert_close_rel(actual, expected, rel=1e-5, what=""):
    """|a - b| <= rel * max(|b|, rms(row of b), rms(b)) element-wise.

    The stated floating-point bar of the hot path is rel 1e-5 in fp32.  A purely
    element-wise relative bound cannot hold for sums that cancel to ~0 under any change of
    summation order (the CPU reference itself is that far from the exact sum), so small
    entries are measured against the RMS of their own output row -- rows are sums of very
    different lengths on power-law graphs -- and of the whole tensor.
    ``test_accuracy_against_fp64`` backs this with an fp64 computation.
    """
    a = np.asarray(actual, dtype=np.float64)
    b = np.asarray(expected, dtype=np.float64)
    assert a.shape == b.shape, f"{what}: shape {a.shape} != {b.shape}"
    if b.size == 0:
        return
    scale = np.maximum(np.abs(b), float(np.sqrt(np.mean(b * b))))
    if b.ndim == 2:
        scale = np.maximum(scale, np.sqrt(np.mean(b * b, axis=1, keepdims=True)))
    bound = rel * scale + 1e-30
    err = np.abs(a - b)
    worst = int(np.argmax(err - bound))
    assert np.all(err <= bound), (
        f"{what}: max excess at flat index {worst}: got {a.flat[worst]!r}, expected "
        f"{b.flat[worst]!r}, |err|={err.flat[worst]:.3e}, bound={bound.flat[worst]:.3e}")


def golden_blocks(golden):
    """The golden rule-DAG graph as the oracle's ``blocks`` dict."""
    blocks = {name: tuple(golden[f"dag_{name}_{p}"] for p in ("rowptr", "col", "val"))
              for name in ("v2v", "v2r", "r2v")}
    blocks["r2r"] = [tuple(golden[f"dag_level{i}_{p}"] for p in ("rowptr", "col", "val"))
                     for i in range(int(golden["dag_step"]))]
    return blocks
