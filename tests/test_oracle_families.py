"""The CPU oracle for fused linear, image+vector fusion, convolution and contract/expand against
golden vectors produced by the unmodified reference (tests/golden/make_golden.py).  No GPU needed.
Everything is bit-exact except the bias gradient, which the reference computes with Tensor::sum
(pairwise summation): rtol 1e-5."""
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import hinge_oracle as ho

FAMILIES = np.load(os.path.join(GOLDEN, "families.npz"))


def case(prefix):
    n = len(prefix)
    return {k[n:]: FAMILIES[k] for k in FAMILIES.files if k.startswith(prefix)}


@pytest.mark.parametrize("idx", range(int(FAMILIES["linear_count"])))
def test_fused_linear_and_fusion_oracle(idx):
    c = case("linear%02d_" % idx)
    kind, vec = str(c["kind"]), c.get("vec")
    out = ho.linear_forward(kind, c["x"], c["thr"], c["ord"], c["w"], c["lin"], c["bias"], vec=vec)
    assert np.array_equal(out, c["out"])
    grads = ho.linear_backward(kind, c["x"], c["thr"], c["ord"], c["w"], c["lin"], c["g"], vec=vec)
    names = ["gx", "gvec", "gthr", "gw", "glin"] if vec is not None else ["gx", "gthr", "gw", "glin"]
    for name, got in zip(names, grads):
        assert np.array_equal(got, c[name]), name
    assert np.allclose(grads[-1], c["gbias"], rtol=1e-5, atol=1e-6)
    if vec is not None:
        assert np.array_equal(ho.forward(kind, c["x"], c["thr"], c["ord"], c["w"], vec=vec), c["fusion_out"])
        got = ho.backward(kind, c["x"], c["thr"], c["ord"], c["w"], c["fusion_g"], vec=vec)
        for name, g in zip(["fusion_gx", "fusion_gvec", "fusion_gthr", "fusion_gw"], got):
            assert np.array_equal(g, c[name]), name


@pytest.mark.parametrize("idx", range(int(FAMILIES["conv_count"])))
def test_convolution_oracle(idx):
    c = case("conv%02d_" % idx)
    kind = str(c["kind"])
    geometry = [tuple(int(v) for v in row) for row in c["geometry"]]
    assert np.array_equal(ho.conv_forward(kind, c["x"], c["thr"], c["ord"], c["w"], *geometry), c["out"])
    gx, gthr, gw = ho.conv_backward(kind, c["x"], c["thr"], c["ord"], c["w"], c["g"], *geometry)
    assert np.array_equal(gx, c["gx"]) and np.array_equal(gthr, c["gthr"]) and np.array_equal(gw, c["gw"])


@pytest.mark.parametrize("idx", range(int(FAMILIES["patch_count"])))
def test_contract_expand_oracle(idx):
    c = case("patch%02d_" % idx)
    window, padding = tuple(int(v) for v in c["window"]), tuple(int(v) for v in c["padding"])
    contracted = ho.contract(c["x"], window, padding)
    assert np.array_equal(contracted, c["contracted"])
    assert np.array_equal(ho.expand(contracted, padding), c["expanded"])


@pytest.mark.parametrize("idx", range(int(FAMILIES["trie_count"])))
def test_trie_oracle(idx):
    c = case("trie%02d_" % idx)
    assert np.array_equal(ho.trie_forward(c["x"], c["thr"], c["ord"], c["w"]), c["out"])
    gx, gthr, gw = ho.trie_backward(c["x"], c["thr"], c["ord"], c["w"], c["g"])
    assert np.array_equal(gx, c["gx"]) and np.array_equal(gthr, c["gthr"]) and np.array_equal(gw, c["gw"])
