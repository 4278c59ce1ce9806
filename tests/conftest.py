import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden_forest():
    return np.load(os.path.join(GOLDEN, "forest.npz"))


def forest_case(golden, idx):
    p = "forest%02d_" % idx
    names = ["x", "thr", "ord", "w", "g", "out", "gx", "gthr", "gw", "margin", "margin_ord", "leaf", "reach"]
    case = {n: golden[p + n] for n in names}
    case["kind"] = str(golden[p + "kind"])
    return case


def forest_case_ids(golden=None):
    data = np.load(os.path.join(GOLDEN, "forest.npz"))
    return list(range(int(data["forest_count"])))


def random_forest_inputs(seed, kind, B, C, inner, T, depth, extra, scale_thr=3.0, quantise=False):
    """Seeded synthetic inputs with the reference's init distributions (thr U(-3,3), w N(0,1))."""
    rng = np.random.default_rng(seed)
    N = depth if kind == "fern" else 2 ** depth - 1
    x = rng.standard_normal((B, C) + tuple(inner)).astype(np.float32)
    thr = rng.uniform(-scale_thr, scale_thr, (T, N)).astype(np.float32)
    ord_ = rng.integers(0, C, (T, N)).astype(np.int64)
    w = rng.standard_normal((T, 2 ** depth) + tuple(extra)).astype(np.float32)
    if quantise:
        x = np.round(x * 2) / 2
        thr = np.round(thr * 2) / 2
    return x, thr, ord_, w


def grad_close(t, ref, scale, rel=1e-5):
    """The backward bar for sums whose order is free: |t - ref| <= 1e-5 * scale per element, where
    scale is the sum of |terms| the oracle added into that element (hinge_oracle.magnitudes)."""
    got = t.detach().cpu().numpy() if hasattr(t, "detach") else np.asarray(t)
    got = got.astype(np.float64)
    return bool(np.all(np.abs(got - np.asarray(ref, dtype=np.float64)) <= rel * np.asarray(scale, dtype=np.float64) + 1e-30))
