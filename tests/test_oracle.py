"""The CPU oracle against the golden vectors produced by the unmodified reference, and
against hand-checkable known-answer cases.  No GPU needed."""
import numpy as np
import pytest

from conftest import forest_case, forest_case_ids
from oracle import hinge_oracle as ho


@pytest.mark.parametrize("idx", forest_case_ids())
def test_oracle_matches_reference_golden(golden_forest, idx):
    c = forest_case(golden_forest, idx)
    kind = c["kind"]
    assert np.array_equal(ho.forward(kind, c["x"], c["thr"], c["ord"], c["w"]), c["out"], equal_nan=True)
    leaf, margin, mord, reach = ho.maps(kind, c["x"], c["thr"], c["ord"], c["w"])
    assert np.array_equal(leaf, c["leaf"])
    assert np.array_equal(margin, c["margin"], equal_nan=True)
    assert np.array_equal(mord, c["margin_ord"])
    assert np.array_equal(reach, c["reach"])
    gx, gthr, gw = ho.backward(kind, c["x"], c["thr"], c["ord"], c["w"], c["g"])
    assert np.array_equal(gx, c["gx"], equal_nan=True)
    assert np.array_equal(gthr, c["gthr"], equal_nan=True)
    assert np.array_equal(gw, c["gw"], equal_nan=True)


def test_known_answer_depth2_tree():
    # depth-2 tree on three hand-made samples: row 0 is an ordinary case, row 1 has a margin
    # of exactly zero (goes left, zero gradient), row 2 has a tie in |margin| (root wins).
    thr = np.array([[0.5, -1.0, 2.0]], np.float32)
    ord_ = np.array([[0, 1, 2]], np.int64)
    w = np.array([[10, 20, 30, 40]], np.float32)
    x = np.array([[1, 0, 1.75], [0, -1, 9], [1, 5, 2.5]], np.float32)
    assert ho.forward("tree", x, thr, ord_, w).tolist() == [[5.0], [0.0], [20.0]]
    leaf, margin, mord, reach = ho.maps("tree", x, thr, ord_, w)
    assert leaf.tolist() == [[1], [0], [3]]
    assert margin.tolist() == [[-0.25], [0.0], [0.5]]
    assert mord.tolist() == [[2], [1], [0]]
    assert reach.tolist() == [[1, 1, 0, 1]]
    gx, gthr, gw = ho.backward("tree", x, thr, ord_, w, np.ones((3, 1), np.float32))
    assert gx.tolist() == [[0, 0, -20], [0, 0, 0], [40, 0, 0]]
    assert gthr.tolist() == [[-40, 0, 20]]
    assert gw.tolist() == [[0, 0.25, 0, 0.5]]


def test_known_answer_fern():
    thr = np.array([[0.5, -1.0]], np.float32)
    ord_ = np.array([[0, 1]], np.int64)
    w = np.array([[10, 20, 30, 40]], np.float32)
    x = np.array([[1, 0, 1.75], [0, -1, 9], [1, 5, 2.5]], np.float32)
    assert ho.forward("fern", x, thr, ord_, w).tolist() == [[20.0], [0.0], [20.0]]
    assert ho.maps("fern", x, thr, ord_, w)[0].tolist() == [[3], [0], [3]]


def test_output_shape_with_inner_dims():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 7, 3, 2)).astype(np.float32)
    thr = rng.standard_normal((4, 7)).astype(np.float32)
    ord_ = rng.integers(0, 7, (4, 7))
    w = rng.standard_normal((4, 8, 2, 2)).astype(np.float32)
    assert ho.forward("tree", x, thr, ord_, w).shape == (2, 4, 3, 2, 2, 2)


def test_oracle_against_live_reference_if_built():
    """Where the reference build is present (the build container), compare on fresh random cases."""
    from oracle import build_ref
    try:
        ref = build_ref.load()
    except ImportError:
        pytest.skip("reference build not present on this machine")
    import torch
    from conftest import random_forest_inputs
    for seed, kind in enumerate(["tree", "fern"] * 3):
        x, thr, ord_, w = random_forest_inputs(seed, kind, 13, 9, (2,), 5, 4, (3,), quantise=seed % 2 == 0)
        tx, tt, to, tw = map(torch.from_numpy, (x, thr, ord_, w))
        out = getattr(ref, kind + "_forward")(tx, tt, to, tw)
        assert np.array_equal(out.numpy(), ho.forward(kind, x, thr, ord_, w))
        g = torch.randn(out.shape, generator=torch.Generator().manual_seed(seed))
        gr = getattr(ref, kind + "_backward")(tx, True, tt, True, to, False, tw, True, g)
        gm = ho.backward(kind, x, thr, ord_, w, g.numpy())
        for a, b in zip((gr[0], gr[1], gr[3]), gm):
            assert np.array_equal(a.numpy(), b)
